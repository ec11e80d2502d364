// Segment gather/scatter for the uncompressed tensors of a bucket, the
// random-block compressor, and the 8-bit group-quantised error store.
//
// Replaces of the reference: torch.cat + all_reduce + per-tensor copy-back of
// uncompressed tensors (communication/powerSGD_hook.py:424-428,503-514) and the
// per-tensor Python loops of the random-block hooks
// (communication/RandomBlock_hook.py:213-245,271-288,
//  communication/UnbiasedRandomBlock_hook.py:153-168,196-213).
// The scatter kernels read every peer's staging buffer directly (peer memory),
// so the all-reduce of the staged values happens inside the kernel that writes
// them back into the bucket.
#include <string.h>
#include "common.cuh"

constexpr int QGROUP = 256;  // elements per quantisation group

template <typename T>
__device__ __forceinline__ int find_seg(const T* segs, int n, long long pos, long long T::*key) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (segs[mid].*key <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

__global__ void k_gather_segments(const ConefSeg* __restrict__ segs, int nsegs, const float* __restrict__ bucket,
                                  float* __restrict__ dense_err, float* __restrict__ staging, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    const int s = find_seg(segs, nsegs, e, &ConefSeg::dst_off);
    const long long src = segs[s].src_off + (e - segs[s].dst_off);
    float v = bucket[src];
    if (dense_err) { v += dense_err[src]; dense_err[src] = v; }  // error slot keeps the local value
    staging[e] = v;
  }
}

extern "C" int conef_gather_segments(const ConefSeg* segs, int nsegs, const float* bucket,
                                     const float* dense_err, float* staging, long long total,
                                     cudaStream_t stream) {
  if (total <= 0 || nsegs <= 0) return 0;
  const int grid = (int)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256);
  k_gather_segments<<<grid, 256, 0, stream>>>(segs, nsegs, bucket, const_cast<float*>(dense_err), staging, total);
  CONEF_CHECK_LAUNCH("k_gather_segments");
  return 0;
}

__global__ void k_scatter_segments(const ConefSeg* __restrict__ segs, int nsegs, float* __restrict__ bucket,
                                   const float* const* __restrict__ peer_staging, int world,
                                   const float* __restrict__ local_staging, float scale,
                                   float* __restrict__ dense_err, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    float v;
    if (peer_staging) {
      v = 0.f;
      for (int p = 0; p < world; ++p) v += ld_relaxed_sys_f32(peer_staging[p] + e);
    } else {
      v = local_staging[e];
    }
    v *= scale;
    const int s = find_seg(segs, nsegs, e, &ConefSeg::dst_off);
    const long long src = segs[s].src_off + (e - segs[s].dst_off);
    bucket[src] = v;
    if (dense_err) dense_err[src] -= v;  // local value (stored by the gather) minus the average
  }
}

extern "C" int conef_scatter_segments(const ConefSeg* segs, int nsegs, float* bucket,
                                      const float* const* peer_staging, int world,
                                      const float* local_staging, float scale, float* dense_err,
                                      long long total, cudaStream_t stream) {
  if (total <= 0 || nsegs <= 0) return 0;
  const int grid = (int)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256);
  k_scatter_segments<<<grid, 256, 0, stream>>>(segs, nsegs, bucket, peer_staging, world, local_staging, scale,
                                             dense_err, total);
  CONEF_CHECK_LAUNCH("k_scatter_segments");
  return 0;
}

// ---------------------------------------------------------------------------
// random block
//
// Two launches per bucket and step:
//   gather : selected elements (+ remembered error) -> staging, error store updated in the same pass;
//            spare CTAs copy the uncompressed tensors into their staging; the CTA that finishes last
//            publishes the step's epoch in every peer's flag array.
//   reduce+scatter : every CTA waits (bounded) for the peers' epoch, then sums the peers' staged
//            values over NVLink and writes the averages back into the bucket.  Small payloads are
//            summed in one shot (every rank reads every peer's whole staging).  Large ones in two
//            shots: a rank sums only its 1/world slice, stores the result into every peer's
//            `reduced` buffer, publishes a second epoch, and after the peers' second epoch scatters
//            from its own `reduced` buffer: the bytes a rank pulls over NVLink drop from
//            world x payload to payload (plus payload pushed).
__device__ __forceinline__ bool in_block(const ConefBlk& B, long long idx, long long* stage_pos) {
  const long long end = B.start + B.block;
  if (idx >= B.start && idx < end) { *stage_pos = B.stage_off + (idx - B.start); return true; }
  const long long wrap = end - B.numel;  // > 0 when the block wraps to index 0
  if (idx < wrap) { *stage_pos = B.stage_off + (B.numel - B.start) + idx; return true; }
  return false;
}

// Uncompressed tensors riding along with the gather kernels: spare CTAs copy them into staging.
struct SegGather {
  const ConefSeg* segs;
  int nsegs, tile_ctas;      // CTAs [tile_ctas, gridDim.x) do the segments
  long long total;
  float* staging;
};
__device__ __forceinline__ void seg_gather_ctas(const SegGather& S, const float* __restrict__ bucket) {
  const long long stride = (long long)(gridDim.x - S.tile_ctas) * blockDim.x;
  for (long long e = (long long)(blockIdx.x - S.tile_ctas) * blockDim.x + threadIdx.x; e < S.total; e += stride) {
    const int s = find_seg(S.segs, S.nsegs, e, &ConefSeg::dst_off);
    S.staging[e] = bucket[S.segs[s].src_off + (e - S.segs[s].dst_off)];
  }
}

// Flat mapping: tile = (tensor, run of `groups_per_tile` groups of 256 consecutive elements), one warp
// per tile.  Modes NONE / DENSE / QUANT8.
//   v = g + error ; selected -> staging (times gather_scale), kept error 0
//                 ; not selected -> gradient zeroed, kept error v
// A warp walks its groups with the loads of the next group in flight while it works on the current
// one: with a single group per warp the two dependent loads in front of the data (tile, tensor
// record) left the memory pipe idle for most of a warp's life.
// Element k of lane `lane` in a group: PACK = false: base + lane + 32 k (4-byte accesses, any alignment);
// PACK = true: base + 128 (k / 4) + 4 lane + k % 4, i.e. two chunks of 128 elements, four consecutive elements
// per lane and chunk, moved as one 16-byte word (gradient, dense error) or one 4-byte word (codes) per chunk: a
// warp's access is contiguous either way.  The packed form needs the tensor's gradient (and dense error)
// 16-byte aligned, its codes 4-byte aligned, and a whole group (no ragged end).
struct FlatLoad {
  float v[QGROUP / 32];      // gradient
  float e[QGROUP / 32];      // dense error, or the 8-bit code as a float
  float old_scale;
};
template <bool PACK>
__device__ __forceinline__ long long flat_index(long long base, int lane, int k) {
  return PACK ? base + 128 * (k >> 2) + 4 * lane + (k & 3) : base + lane + 32 * k;
}
template <bool PACK>
__device__ __forceinline__ void flat_load(const ConefBlk& B, long long group, int lane, const float* __restrict__ g,
                                          const float* __restrict__ dense_err, const int8_t* __restrict__ qcodes,
                                          const float* __restrict__ qscales, int ef_mode, FlatLoad& L) {
  static_assert(QGROUP == 256, "the packed form moves eight elements per lane");
  const long long base = group * QGROUP;
  L.old_scale = ef_mode == CONEF_EF_QUANT8 ? qscales[(long long)B.scale_off + group] : 0.f;
  if (PACK) {
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      const long long i0 = base + 128 * c + 4 * lane;
      const float4 a = *reinterpret_cast<const float4*>(g + i0);
      L.v[4 * c] = a.x; L.v[4 * c + 1] = a.y; L.v[4 * c + 2] = a.z; L.v[4 * c + 3] = a.w;
      if (ef_mode == CONEF_EF_DENSE) {
        const float4 d = *reinterpret_cast<const float4*>(dense_err + B.sk_off + i0);
        L.e[4 * c] = d.x; L.e[4 * c + 1] = d.y; L.e[4 * c + 2] = d.z; L.e[4 * c + 3] = d.w;
      } else if (ef_mode == CONEF_EF_QUANT8) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(qcodes + B.sk_off + i0);
#pragma unroll
        for (int j = 0; j < 4; ++j) L.e[4 * c + j] = (float)(int8_t)((w >> (8 * j)) & 0xffu);
      } else {
#pragma unroll
        for (int j = 0; j < 4; ++j) L.e[4 * c + j] = 0.f;
      }
    }
    return;
  }
#pragma unroll
  for (int k = 0; k < QGROUP / 32; ++k) {
    const long long idx = base + lane + 32 * k;
    L.v[k] = 0.f;
    L.e[k] = 0.f;
    if (idx < B.numel) {
      L.v[k] = g[idx];
      if (ef_mode == CONEF_EF_DENSE) L.e[k] = dense_err[B.sk_off + idx];
      else if (ef_mode == CONEF_EF_QUANT8) L.e[k] = (float)qcodes[B.sk_off + idx];
    }
  }
}

// One tile (tensor, run of groups) of the flat gather; see k_randblock_gather_flat.
template <bool PACK>
__device__ __forceinline__ void flat_tile(const ConefBlk& B, long long first, int count, int lane, float* __restrict__ g,
                                          float* __restrict__ staging, float gs, float* __restrict__ dense_err,
                                          int8_t* __restrict__ qcodes, float* __restrict__ qscales, float alpha,
                                          float beta, int ef_mode) {
  FlatLoad cur, nxt;
  if (count > 0) flat_load<PACK>(B, first, lane, g, dense_err, qcodes, qscales, ef_mode, cur);
#pragma unroll 1
  for (int q = 0; q < count; ++q) {
    const long long group = first + q;
    if (q + 1 < count) flat_load<PACK>(B, group + 1, lane, g, dense_err, qcodes, qscales, ef_mode, nxt);
    const long long base = group * QGROUP;
    float keep[QGROUP / 32], gout[QGROUP / 32];
    float amax = 0.f;
#pragma unroll
    for (int k = 0; k < QGROUP / 32; ++k) {
      const long long idx = flat_index<PACK>(base, lane, k);
      keep[k] = 0.f;
      gout[k] = cur.v[k];
      if (PACK || idx < B.numel) {
        float v = cur.v[k];
        float carry = 0.f;
        if (ef_mode == CONEF_EF_DENSE) v += cur.e[k];
        else if (ef_mode == CONEF_EF_QUANT8) {
          const float e = cur.e[k] * cur.old_scale;
          v += alpha * e;
          carry = beta * e;
        }
        long long sp;
        if (in_block(B, idx, &sp)) {
          staging[sp] = v * gs;
          keep[k] = carry;
        } else {
          gout[k] = 0.f;
          if (!PACK) g[idx] = 0.f;
          keep[k] = carry + v;
        }
        if (!PACK && ef_mode == CONEF_EF_DENSE) dense_err[B.sk_off + idx] = keep[k];
        amax = fmaxf(amax, fabsf(keep[k]));
      }
    }
    if (PACK) {      // selected elements keep their gradient value: the scatter overwrites them later
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        const long long i0 = base + 128 * c + 4 * lane;
        *reinterpret_cast<float4*>(g + i0) = make_float4(gout[4 * c], gout[4 * c + 1], gout[4 * c + 2], gout[4 * c + 3]);
        if (ef_mode == CONEF_EF_DENSE)
          *reinterpret_cast<float4*>(dense_err + B.sk_off + i0) =
              make_float4(keep[4 * c], keep[4 * c + 1], keep[4 * c + 2], keep[4 * c + 3]);
      }
    }
    if (ef_mode == CONEF_EF_QUANT8) {
      amax = warp_max(amax);
      const float scale = amax / 127.f;
      const float inv = scale > 0.f ? 1.f / scale : 0.f;
      uint32_t packed[2] = {0u, 0u};
#pragma unroll
      for (int k = 0; k < QGROUP / 32; ++k) {
        const long long idx = flat_index<PACK>(base, lane, k);
        if (PACK || idx < B.numel) {
          float qv = rintf(keep[k] * inv);
          qv = fminf(fmaxf(qv, -127.f), 127.f);
          if (PACK) packed[k >> 2] |= ((uint32_t)(int)qv & 0xffu) << (8 * (k & 3));
          else qcodes[B.sk_off + idx] = (int8_t)qv;
        }
      }
      if (PACK) {
#pragma unroll
        for (int c = 0; c < 2; ++c)
          *reinterpret_cast<uint32_t*>(qcodes + B.sk_off + base + 128 * c + 4 * lane) = packed[c];
      }
      if (lane == 0) qscales[(long long)B.scale_off + group] = scale;
    }
    cur = nxt;
  }
}

__global__ void __launch_bounds__(256, 3)
k_randblock_gather_flat(const ConefBlk* __restrict__ blks, const int2* __restrict__ tiles, int ntiles,
                        int groups_per_tile, float* __restrict__ bucket, float* __restrict__ staging,
                        float gather_scale, float* __restrict__ dense_err, int8_t* __restrict__ qcodes,
                        float* __restrict__ qscales, float alpha, float beta, int ef_mode, const SegGather SG,
                        const ConefPublish pub) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * 8 + warp;
  if ((int)blockIdx.x >= SG.tile_ctas) {
    seg_gather_ctas(SG, bucket);
  } else if (tile < ntiles) {
    const int2 t = tiles[tile];
    const ConefBlk B = blks[t.x];
    float* g = bucket + B.g_off;
    // gather_scale == 0 selects the unbiased estimator: divide by the selection probability
    const float gs = gather_scale != 0.f ? gather_scale : (float)B.numel / (float)B.block;
    // the tensor's codes start at sk_off in the code arena; its groups are aligned to the tensor start
    const long long ngroups = (B.numel + QGROUP - 1) / QGROUP;
    const long long first = (long long)t.y * groups_per_tile;
    int count = (int)min((long long)groups_per_tile, ngroups - first);
    // packed accesses for the whole groups of a tensor whose arrays are aligned for them
    bool pack = (reinterpret_cast<uintptr_t>(g) & 15) == 0;
    if (ef_mode == CONEF_EF_DENSE) pack = pack && (reinterpret_cast<uintptr_t>(dense_err + B.sk_off) & 15) == 0;
    if (ef_mode == CONEF_EF_QUANT8) pack = pack && (reinterpret_cast<uintptr_t>(qcodes + B.sk_off) & 3) == 0;
    if (pack) {
      const int whole = (int)max(0LL, min((long long)count, B.numel / QGROUP - first));
      flat_tile<true>(B, first, whole, lane, g, staging, gs, dense_err, qcodes, qscales, alpha, beta, ef_mode);
      flat_tile<false>(B, first + whole, count - whole, lane, g, staging, gs, dense_err, qcodes, qscales, alpha, beta,
                       ef_mode);
    } else {
      flat_tile<false>(B, first, count, lane, g, staging, gs, dense_err, qcodes, qscales, alpha, beta, ef_mode);
    }
  }
  conef_publish_if_last(pub, gridDim.x);
}

// Row mapping for the count-sketch error store: tile = (tensor, row block).  The sketch update is
// linear in the remembered term (s_j^2 = 1):
//   S'[i, w] = S[i, w] (1 - (1 - beta) k_w) + sum over the NOT selected columns j of cell w of (s_j g_ij + alpha S[i, w])
// so a row none of whose elements are selected (nine rows in ten at a 10 % block) needs no gather of
// the old sketch value: its remembered term is alpha k_w S[i, w], applied when the accumulator is
// flushed, and the pass over its elements is one shared-memory atomic each.  A row the block covers
// or cuts needs the old sketch values for what it sends; a tile that has such a row first copies its
// sketch rows into shared memory.  All rows of the tile are walked together, column by column, so
// that a thread has one load per row in flight: walking the rows one after another leaves a single
// load in flight per thread and ran eight times slower.
constexpr int RB_MAX_ROWS = 8;

__global__ void __launch_bounds__(256, 4)      // 64 registers: four CTAs of 37 KB per SM
k_randblock_gather_sketch(const ConefBlk* __restrict__ blks, const int2* __restrict__ tiles, int rows_per_cta,
                          float* __restrict__ bucket, float* __restrict__ staging, float gather_scale,
                          float* __restrict__ sketch, const int32_t* __restrict__ tables,
                          const int32_t* __restrict__ counts, float alpha, float beta, const SegGather SG,
                          const ConefPublish pub) {
  extern __shared__ float sm[];  // acc: rows_per_cta * W, then the old sketch rows: rows_per_cta * W
  if ((int)blockIdx.x >= SG.tile_ctas) {
    seg_gather_ctas(SG, bucket);
  } else {
    const int2 t = tiles[blockIdx.x];
    const ConefBlk B = blks[t.x];
    const int m = B.m, W = B.W;
    const int row0 = t.y * rows_per_cta;
    const int rows = min(rows_per_cta, B.n - row0);
    float* acc = sm;
    float* old = sm + (size_t)rows_per_cta * W;
    const int32_t* tab = tables + B.tab_off;
    const int32_t* cnt = counts + B.cnt_off;
    const float gs = gather_scale != 0.f ? gather_scale : (float)B.numel / (float)B.block;
    const float omb = 1.f - beta;
    float* g = bucket + B.g_off + (size_t)row0 * m;
    float* srow0 = sketch + B.sk_off + (size_t)row0 * W;
    const long long end = B.start + B.block, wrap = end - B.numel;
    // bit ii of `touched`: the block covers or cuts row ii (the same value in every thread)
    unsigned touched = 0;
#pragma unroll
    for (int ii = 0; ii < RB_MAX_ROWS; ++ii) {
      if (ii < rows) {
        const long long r0 = (long long)(row0 + ii) * m, r1 = r0 + m;
        const long long c1 = max(0LL, min(r1, end) - max(r0, B.start)) + max(0LL, min(r1, wrap) - r0);
        if (c1 > 0) touched |= 1u << ii;
      }
    }
    for (int i = threadIdx.x; i < rows * W; i += blockDim.x) {
      acc[i] = 0.f;
      if (touched) old[i] = srow0[i];
    }
    __syncthreads();
    for (int j = threadIdx.x; j < m; j += blockDim.x) {
      const int e = __ldg(tab + j);
      const int h = unpack_bucket(e);
      const float s = unpack_sign(e);
      float v[RB_MAX_ROWS];
#pragma unroll
      for (int ii = 0; ii < RB_MAX_ROWS; ++ii) v[ii] = ii < rows ? g[(size_t)ii * m + j] : 0.f;
#pragma unroll
      for (int ii = 0; ii < RB_MAX_ROWS; ++ii) {
        if (ii < rows) {
          if (!((touched >> ii) & 1u)) {
            g[(size_t)ii * m + j] = 0.f;
            atomicAdd(&acc[ii * W + h], s * v[ii]);
          } else {
            const float vv = v[ii] + alpha * s * old[ii * W + h];
            long long sp;
            if (in_block(B, (long long)(row0 + ii) * m + j, &sp)) {
              staging[sp] = vv * gs;
            } else {
              g[(size_t)ii * m + j] = 0.f;
              atomicAdd(&acc[ii * W + h], s * vv);
            }
          }
        }
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < rows * W; i += blockDim.x) {
      const int ii = i / W, w = i - ii * W;
      const float k = (float)__ldg(cnt + w);
      if ((touched >> ii) & 1u) srow0[i] = old[i] * (1.f - omb * k) + acc[i];
      else srow0[i] = srow0[i] * (1.f + (alpha - omb) * k) + acc[i];
    }
  }
  conef_publish_if_last(pub, gridDim.x);
}

static int seg_cta_count(long long total) {
  if (total <= 0) return 0;
  long long n = (total + 1023) / 1024;
  return (int)(n > 32 ? 32 : n);
}

// The same pass over the block layout of the hash (conef_cell, layout 1; the table arena holds the
// matrix's S x nb records {g | x_g << 27, sign bits}, window-major, at cb_off).  A warp's unit is
// (block of RB_MAX_ROWS rows, cell block c): it walks the S column groups of its cell block, lane l
// handles column 32 g + (l xor x_g), whose cell is 32 c + l for every group.  The cell block's sums and
// its old sketch values therefore sit in the lanes' registers: no atomics and no copy of sketch rows in
// shared memory; the gradient travels through a per-warp cp.async ring (three groups in flight).
// Tile = (tensor, chunk of eight consecutive units).
constexpr int RBK_STAGES = 4;
__global__ void __launch_bounds__(256, 3)
k_randblock_gather_sketch_blk(const ConefBlk* __restrict__ blks, const int2* __restrict__ tiles,
                              float* __restrict__ bucket, float* __restrict__ staging, float gather_scale,
                              float* __restrict__ sketch, const int32_t* __restrict__ tables,
                              const int32_t* __restrict__ counts, float alpha, float beta, const SegGather SG,
                              const ConefPublish pub) {
  constexpr int RB = RB_MAX_ROWS;
  __shared__ float ring_all[8][RBK_STAGES][RB][32];
  if ((int)blockIdx.x >= SG.tile_ctas) {
    seg_gather_ctas(SG, bucket);
  } else {
    const int2 t = tiles[blockIdx.x];
    const ConefBlk B = blks[t.x];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int m = B.m, W = B.W, nb = W >> 5;
    const int unit = t.y * 8 + warp;
    if (unit < ((B.n + RB - 1) / RB) * nb) {
      const int rbk = unit / nb, c = unit - rbk * nb;
      const int row0 = rbk * RB;
      const int rows = min(RB, B.n - row0);
      const int S = (((m + 31) >> 5) + nb - 1) / nb;
      const int2* recs = reinterpret_cast<const int2*>(tables + B.cb_off) + c;
      const float gs = gather_scale != 0.f ? gather_scale : (float)B.numel / (float)B.block;
      const float omb = 1.f - beta;
      float* g0 = bucket + B.g_off + (size_t)row0 * m;
      const int cell = (c << 5) + lane;
      float* sc0 = sketch + B.sk_off + (size_t)row0 * W + cell;
      const float kcnt = (float)__ldg(counts + B.cnt_off + cell);
      const long long end = B.start + B.block, wrap = end - B.numel;
      // bit ii of `touched`: the block covers or cuts row ii (the same value in every thread)
      unsigned touched = 0;
      float so[RB], acc[RB];
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        acc[ii] = 0.f;
        so[ii] = 0.f;
        if (ii < rows) {
          const long long r0 = (long long)(row0 + ii) * m, r1 = r0 + m;
          const long long c1 = max(0LL, min(r1, end) - max(r0, B.start)) + max(0LL, min(r1, wrap) - r0);
          if (c1 > 0) touched |= 1u << ii;
          so[ii] = sc0[(size_t)ii * W];
        }
      }
      const uint32_t ring = (uint32_t)__cvta_generic_to_shared(&ring_all[warp][0][0][lane]);
      const unsigned pitch = (unsigned)m * 4u;
      auto row_ptr = [&](float* base, int ii) {
        return reinterpret_cast<float*>(reinterpret_cast<char*>(base) + (unsigned long long)pitch * (unsigned)ii);
      };
      for (int s0 = 0; s0 < S; s0 += 32) {
        int2 mine = make_int2(0x7ffffff, 0);
        if (s0 + lane < S) mine = __ldg(recs + (size_t)(s0 + lane) * nb);
        const int cnt = min(32, S - s0);
        auto column = [&](int i) {      // this lane's column in group i of the chunk (m: none)
          const int rx = __shfl_sync(0xffffffffu, mine.x, i & 31);
          const int g = rx & 0x7ffffff;
          return (i < cnt && g != 0x7ffffff) ? (g << 5) + (lane ^ (int)((uint32_t)rx >> 27)) : m;
        };
        auto issue = [&](int i) {
          const int cl = column(i);
          if (cl < m) {
            const uint32_t dst = ring + (uint32_t)(i & (RBK_STAGES - 1)) * (RB * 128);
#pragma unroll
            for (int ii = 0; ii < RB; ++ii)
              if (ii < rows) cp_async_f32<0>(dst + ii * 128, row_ptr(g0 + cl, ii));
          }
          cp_async_commit();
        };
#pragma unroll
        for (int k = 0; k < RBK_STAGES - 1; ++k) issue(k);
        for (int i = 0; i < cnt; ++i) {
          issue(i + RBK_STAGES - 1);
          const int col = column(i);
          const uint32_t sbits = (uint32_t)__shfl_sync(0xffffffffu, mine.y, i & 31);
          cp_async_wait<RBK_STAGES - 1>();      // the copies of group i have landed
          if (col < m) {
            const float sgn = ((sbits >> (col & 31)) & 1u) ? 1.f : -1.f;
            const uint32_t src = ring + (uint32_t)(i & (RBK_STAGES - 1)) * (RB * 128);
            float* gp = g0 + col;
#pragma unroll
            for (int ii = 0; ii < RB; ++ii) {
              if (ii < rows) {
                const float v = lds_f32<0>(src + ii * 128);
                if (!((touched >> ii) & 1u)) {
                  *row_ptr(gp, ii) = 0.f;
                  acc[ii] = fmaf(sgn, v, acc[ii]);
                } else {
                  const float vv = v + alpha * sgn * so[ii];
                  long long sp;
                  if (in_block(B, (long long)(row0 + ii) * m + col, &sp)) {
                    staging[sp] = vv * gs;
                  } else {
                    *row_ptr(gp, ii) = 0.f;
                    acc[ii] = fmaf(sgn, vv, acc[ii]);
                  }
                }
              }
            }
          }
        }
        cp_async_wait<0>();
      }
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        if (ii < rows) {
          const float fct = ((touched >> ii) & 1u) ? 1.f - omb * kcnt : 1.f + (alpha - omb) * kcnt;
          sc0[(size_t)ii * W] = fmaf(so[ii], fct, acc[ii]);
        }
      }
    }
  }
  conef_publish_if_last(pub, gridDim.x);
}

// segs / total_unc / staging_unc: the uncompressed tensors (may be empty).  done != NULL with
// world > 1: the CTA that finishes last stores epoch (+ *epoch_base) into peer_flags[p][rank].
extern "C" int conef_randblock_gather_ex(const ConefBlk* blks, const int2* tiles, int ntiles, int nblk_tiles,
                                         int rows_per_cta, float* bucket, float* staging, float gather_scale, float* sketch,
                                         const int32_t* tables, const int32_t* counts, float* dense_err,
                                         int8_t* qcodes, float* qscales, float alpha, float beta, int ef_mode,
                                         size_t smem_bytes, const ConefSeg* segs, int nsegs, long long total_unc,
                                         float* staging_unc, uint32_t* done, uint32_t* const* peer_flags, int world,
                                         int rank, uint32_t epoch, const uint32_t* epoch_base, cudaStream_t stream) {
  if (ntiles < 0) ntiles = 0;
  ConefPublish pub;
  memset(&pub, 0, sizeof(pub));
  if (done != nullptr && peer_flags != nullptr && world > 1) {
    pub.done = done; pub.peer_flags = peer_flags; pub.epoch_base = epoch_base;
    pub.epoch = epoch; pub.world = world; pub.rank = rank;
  }
  SegGather SG;
  SG.segs = segs; SG.nsegs = nsegs; SG.total = (segs != nullptr && nsegs > 0) ? total_unc : 0; SG.staging = staging_unc;
  const int seg_ctas = seg_cta_count(SG.total);
  if (ef_mode == CONEF_EF_SKETCH) {
    if (rows_per_cta > RB_MAX_ROWS) { conef_set_error("randblock_gather: at most %d rows per CTA", RB_MAX_ROWS); return 2; }
    smem_bytes *= 2;      // the accumulators and a copy of the old sketch rows
    if (smem_bytes > 220 * 1024) { conef_set_error("randblock_gather: sketch rows do not fit in shared memory"); return 2; }
    // the first nblk_tiles tiles belong to tensors on the block layout of the hash (cb_off >= 0; a tile is a
    // chunk of eight (row block, cell block) units); the kernel launched last carries the uncompressed
    // tensors and the publishing tail
    const int nblk = nblk_tiles < 0 ? 0 : (nblk_tiles > ntiles ? ntiles : nblk_tiles);
    const int nleg = ntiles - nblk;
    if (ntiles + seg_ctas == 0) return 0;
    if (nleg > 0 || nblk == 0) {
      SegGather SL = SG;
      ConefPublish pl = pub;
      if (nblk > 0) { SL.total = 0; memset(&pl, 0, sizeof(pl)); }
      SL.tile_ctas = nleg;
      const int extra = nblk > 0 ? 0 : seg_ctas;
      CONEF_CUDA(cudaFuncSetAttribute(k_randblock_gather_sketch, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
      CONEF_CUDA(cudaFuncSetAttribute(k_randblock_gather_sketch, cudaFuncAttributePreferredSharedMemoryCarveout,
                                      (int)cudaSharedmemCarveoutMaxShared));
      k_randblock_gather_sketch<<<nleg + extra, 256, smem_bytes, stream>>>(
          blks, tiles + nblk, rows_per_cta, bucket, staging, gather_scale, sketch, tables, counts, alpha, beta, SL, pl);
      CONEF_CHECK_LAUNCH("k_randblock_gather_sketch");
    }
    if (nblk > 0) {
      SG.tile_ctas = nblk;
      k_randblock_gather_sketch_blk<<<nblk + seg_ctas, 256, 0, stream>>>(
          blks, tiles, bucket, staging, gather_scale, sketch, tables, counts, alpha, beta, SG, pub);
    }
  } else {
    SG.tile_ctas = (ntiles + 7) / 8;
    if (SG.tile_ctas + seg_ctas == 0) return 0;
    // rows_per_cta: groups of 256 elements per warp tile in these modes (0 or 1: one)
    k_randblock_gather_flat<<<SG.tile_ctas + seg_ctas, 256, 0, stream>>>(
        blks, tiles, ntiles, rows_per_cta > 1 ? rows_per_cta : 1, bucket, staging, gather_scale, dense_err, qcodes,
        qscales, alpha, beta, ef_mode, SG, pub);
  }
  CONEF_CHECK_LAUNCH("k_randblock_gather");
  return 0;
}

extern "C" int conef_randblock_gather(const ConefBlk* blks, const int2* tiles, int ntiles, int nblk_tiles,
                                      int rows_per_cta,
                                      float* bucket, float* staging, float gather_scale, float* sketch,
                                      const int32_t* tables, const int32_t* counts, float* dense_err,
                                      int8_t* qcodes, float* qscales, float alpha, float beta,
                                      int ef_mode, size_t smem_bytes, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  return conef_randblock_gather_ex(blks, tiles, ntiles, nblk_tiles, rows_per_cta, bucket, staging, gather_scale, sketch, tables,
                                   counts, dense_err, qcodes, qscales, alpha, beta, ef_mode, smem_bytes, nullptr, 0,
                                   0, nullptr, nullptr, nullptr, 1, 0, 0, nullptr, stream);
}

__global__ void k_randblock_scatter(const ConefBlk* __restrict__ blks, int nblks, float* __restrict__ bucket,
                                    const float* const* __restrict__ peer_staging, int world,
                                    const float* __restrict__ local_staging, float scale, long long total) {
  for (long long e = (long long)blockIdx.x * blockDim.x + threadIdx.x; e < total;
       e += (long long)gridDim.x * blockDim.x) {
    float v;
    if (peer_staging) {
      v = 0.f;
      for (int p = 0; p < world; ++p) v += ld_relaxed_sys_f32(peer_staging[p] + e);
    } else {
      v = local_staging[e];
    }
    const int b = find_seg(blks, nblks, e, &ConefBlk::stage_off);
    const ConefBlk& B = blks[b];
    long long idx = B.start + (e - B.stage_off);
    if (idx >= B.numel) idx -= B.numel;
    bucket[B.g_off + idx] = v * scale;
  }
}

extern "C" int conef_randblock_scatter(const ConefBlk* blks, int nblks, float* bucket,
                                       const float* const* peer_staging, int world,
                                       const float* local_staging, float scale, long long total_block,
                                       cudaStream_t stream) {
  if (total_block <= 0 || nblks <= 0) return 0;
  const int grid = (int)((total_block + 255) / 256 > 2368 ? 2368 : (total_block + 255) / 256);
  k_randblock_scatter<<<grid, 256, 0, stream>>>(blks, nblks, bucket, peer_staging, world, local_staging, scale,
                                              total_block);
  CONEF_CHECK_LAUNCH("k_randblock_scatter");
  return 0;
}

// Wait + reduce + scatter of a bucket's random blocks AND uncompressed tensors in one launch.
// Elements [0, total_unc) of the combined index space are the uncompressed tensors' staging,
// [total_unc, total_unc + total_blk) the blocks'.
struct RbReduce {
  const ConefBlk* blks;  int nblks;
  const ConefSeg* segs;  int nsegs;
  long long total_unc, total_blk;
  const float* const* peer_unc;      // [world] staged uncompressed tensors
  const float* const* peer_blk;      // [world] staged blocks
  float* const* peer_red;            // [world] `reduced` buffers (two shots only)
  const float* my_red;
  const uint32_t* my_flags;
  uint32_t epoch;                    // epoch of the staged data; two shots publish / wait epoch + 1 as well
  const uint32_t* epoch_base;
  int world, rank, two_shot;
  float scale;
  int* status;
  long long spin_limit;
};

__device__ __forceinline__ void rb_put(const RbReduce& R, float* __restrict__ bucket, long long e, float v) {
  if (e < R.total_unc) {
    const int s = find_seg(R.segs, R.nsegs, e, &ConefSeg::dst_off);
    bucket[R.segs[s].src_off + (e - R.segs[s].dst_off)] = v;
  } else {
    const long long eb = e - R.total_unc;
    const int b = find_seg(R.blks, R.nblks, eb, &ConefBlk::stage_off);
    const ConefBlk& B = R.blks[b];
    long long idx = B.start + (eb - B.stage_off);
    if (idx >= B.numel) idx -= B.numel;
    bucket[B.g_off + idx] = v;
  }
}

__global__ void __launch_bounds__(256)
k_randblock_reduce_scatter(const RbReduce R, float* __restrict__ bucket, const ConefPublish pub) {
  __shared__ int ok;
  const uint32_t epoch = R.epoch + (R.epoch_base != nullptr ? *R.epoch_base : 0u);
  if (R.world > 1) {
    if (threadIdx.x == 0) {
      ok = wait_flags_bounded(R.my_flags, R.world, epoch, R.spin_limit) ? 1 : 0;
      if (!ok) atomicExch(R.status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    if (!ok) return;
  }
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long first = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long one_shot_total = R.total_unc + (R.two_shot ? 0 : R.total_blk);
  for (long long e = first; e < one_shot_total; e += stride) {
    const float* const* peers = e < R.total_unc ? R.peer_unc : R.peer_blk;
    const long long off = e < R.total_unc ? e : e - R.total_unc;
    float v = 0.f;
    for (int p = 0; p < R.world; ++p) v += ld_relaxed_sys_f32(peers[p] + off);
    rb_put(R, bucket, e, v * R.scale);
  }
  if (!R.two_shot) return;
  // ---- first shot: this rank's slice, 16 bytes at a time, summed in rank order and pushed to every peer ----
  const long long quads = (R.total_blk + 3) / 4;
  const long long per = (quads + R.world - 1) / R.world;
  const long long q0 = per * R.rank, q1 = min(quads, q0 + per);
  for (long long q = q0 + first; q < q1; q += stride) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < R.world; ++p) {
      float4 v;
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(R.peer_blk[p] + 4 * q) : "memory");
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    acc.x *= R.scale; acc.y *= R.scale; acc.z *= R.scale; acc.w *= R.scale;
    for (int p = 0; p < R.world; ++p)
      asm volatile("st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
                   ::"l"(R.peer_red[p] + 4 * q), "f"(acc.x), "f"(acc.y), "f"(acc.z), "f"(acc.w) : "memory");
  }
  // ---- the CTA that finishes last publishes epoch + 1; everybody waits for the peers' ----
  conef_publish_if_last(pub, gridDim.x);
  if (threadIdx.x == 0) {
    ok = wait_flags_bounded(R.my_flags, R.world, epoch + 1, R.spin_limit) ? 1 : 0;
    if (!ok) atomicExch(R.status, CONEF_STATUS_FLAG_TIMEOUT);
  }
  __syncthreads();
  if (!ok) return;
  // ---- second shot: scatter from this GPU's own copy of the sums ----
  for (long long e = first; e < R.total_blk; e += stride) {
    float v;
    asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(R.my_red + e) : "memory");
    rb_put(R, bucket, R.total_unc + e, v);
  }
}

// One launch: wait for `epoch` in my_flags (world > 1), reduce over the peers' staging, scatter into
// the bucket.  two_shot needs peer_red / my_red (payload rounded up to 4 floats), done and
// peer_flags; it publishes and waits for epoch + 1.  The grid never exceeds what the device holds
// at once, because in two shots its CTAs wait for one another through the peers.
extern "C" int conef_randblock_reduce_scatter(const ConefBlk* blks, int nblks, const ConefSeg* segs, int nsegs,
                                              long long total_unc, long long total_blk, float* bucket,
                                              const float* const* peer_unc, const float* const* peer_blk,
                                              float* const* peer_red, const float* my_red,
                                              uint32_t* const* peer_flags, const uint32_t* my_flags, int world,
                                              int rank, uint32_t epoch, const uint32_t* epoch_base, float scale,
                                              int two_shot, uint32_t* done, int* status, long long spin_limit,
                                              cudaStream_t stream) {
  if (nblks <= 0) total_blk = 0;
  if (nsegs <= 0) total_unc = 0;
  if (total_unc + total_blk <= 0) return 0;
  if (world <= 1 || peer_red == nullptr || my_red == nullptr || done == nullptr) two_shot = 0;
  RbReduce R;
  R.blks = blks; R.nblks = nblks; R.segs = segs; R.nsegs = nsegs; R.total_unc = total_unc; R.total_blk = total_blk;
  R.peer_unc = peer_unc; R.peer_blk = peer_blk; R.peer_red = peer_red; R.my_red = my_red; R.my_flags = my_flags;
  R.epoch = epoch; R.epoch_base = epoch_base; R.world = world; R.rank = rank; R.two_shot = two_shot; R.scale = scale;
  R.status = status; R.spin_limit = spin_limit;
  ConefPublish pub;
  memset(&pub, 0, sizeof(pub));
  if (two_shot) {
    pub.done = done; pub.peer_flags = peer_flags; pub.epoch_base = epoch_base; pub.epoch = epoch + 1;
    pub.world = world; pub.rank = rank;
  }
  long long want = (total_unc + total_blk + 255) / 256;
  const long long cap = two_shot ? 4 * 148 : 2368;
  const int grid = (int)(want > cap ? cap : want);
  k_randblock_reduce_scatter<<<grid, 256, 0, stream>>>(R, bucket, pub);
  CONEF_CHECK_LAUNCH("k_randblock_reduce_scatter");
  return 0;
}

// ---------------------------------------------------------------------------
// stand-alone 8-bit error store: x += alpha * deq(e) ; e <- Q8(beta * deq(e) + v)
__global__ void k_quant8_query(float* __restrict__ x, const int8_t* __restrict__ codes,
                               const float* __restrict__ scales, long long numel, float alpha) {
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel;
       i += (long long)gridDim.x * blockDim.x)
    x[i] += alpha * (float)codes[i] * scales[i / QGROUP];
}

__global__ void __launch_bounds__(256)
k_quant8_update(const float* __restrict__ v, int8_t* __restrict__ codes, float* __restrict__ scales,
                long long numel, float beta) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long group = (long long)blockIdx.x * 8 + warp;
  const long long base = group * QGROUP;
  if (base >= numel) return;
  const float old_scale = scales[group];
  float keep[QGROUP / 32];
  float amax = 0.f;
#pragma unroll
  for (int k = 0; k < QGROUP / 32; ++k) {
    const long long idx = base + lane + 32 * k;
    keep[k] = 0.f;
    if (idx < numel) {
      keep[k] = beta * (float)codes[idx] * old_scale + v[idx];
      amax = fmaxf(amax, fabsf(keep[k]));
    }
  }
  amax = warp_max(amax);
  const float scale = amax / 127.f;
  const float inv = scale > 0.f ? 1.f / scale : 0.f;
#pragma unroll
  for (int k = 0; k < QGROUP / 32; ++k) {
    const long long idx = base + lane + 32 * k;
    if (idx < numel) {
      float q = rintf(keep[k] * inv);
      codes[idx] = (int8_t)fminf(fmaxf(q, -127.f), 127.f);
    }
  }
  if (lane == 0) scales[group] = scale;
}

extern "C" int conef_quant8_query(float* x, const int8_t* codes, const float* scales, long long numel,
                                  float alpha, cudaStream_t stream) {
  if (numel <= 0) return 0;
  const int grid = (int)((numel + 255) / 256 > 2368 ? 2368 : (numel + 255) / 256);
  k_quant8_query<<<grid, 256, 0, stream>>>(x, codes, scales, numel, alpha);
  CONEF_CHECK_LAUNCH("k_quant8_query");
  return 0;
}

extern "C" int conef_quant8_update(const float* v, int8_t* codes, float* scales, long long numel,
                                   float beta, cudaStream_t stream) {
  if (numel <= 0) return 0;
  const long long groups = (numel + QGROUP - 1) / QGROUP;
  k_quant8_update<<<(unsigned)((groups + 7) / 8), 256, 0, stream>>>(v, codes, scales, numel, beta);
  CONEF_CHECK_LAUNCH("k_quant8_update");
  return 0;
}
