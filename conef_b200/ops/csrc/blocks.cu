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
__device__ __forceinline__ bool in_block(const ConefBlk& B, long long idx, long long* stage_pos) {
  const long long end = B.start + B.block;
  if (idx >= B.start && idx < end) { *stage_pos = B.stage_off + (idx - B.start); return true; }
  const long long wrap = end - B.numel;  // > 0 when the block wraps to index 0
  if (idx < wrap) { *stage_pos = B.stage_off + (B.numel - B.start) + idx; return true; }
  return false;
}

// Flat mapping: tile = (tensor, group of 256 consecutive elements), one warp
// per tile.  Modes NONE / DENSE / QUANT8.
//   v = g + error ; selected -> staging (times gather_scale), kept error 0
//                 ; not selected -> gradient zeroed, kept error v
__global__ void __launch_bounds__(256)
k_randblock_gather_flat(const ConefBlk* __restrict__ blks, const int2* __restrict__ tiles, int ntiles,
                        float* __restrict__ bucket, float* __restrict__ staging, float gather_scale,
                        float* __restrict__ dense_err, int8_t* __restrict__ qcodes,
                        float* __restrict__ qscales, float alpha, float beta, int ef_mode) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x * 8 + warp;
  if (tile >= ntiles) return;
  const int2 t = tiles[tile];
  const ConefBlk B = blks[t.x];
  const long long base = (long long)t.y * QGROUP;
  float* g = bucket + B.g_off;
  // gather_scale == 0 selects the unbiased estimator: divide by the selection probability
  const float gs = gather_scale != 0.f ? gather_scale : (float)B.numel / (float)B.block;
  float keep[QGROUP / 32];
  float amax = 0.f;
  float old_scale = 0.f;
  // the tensor's codes start at sk_off in the code arena; its groups are aligned to the tensor start
  const long long qbase = B.sk_off + base;             // code offset
  const long long sidx = (long long)B.scale_off + t.y;  // scale slot of this group
  if (ef_mode == CONEF_EF_QUANT8) old_scale = qscales[sidx];
#pragma unroll
  for (int k = 0; k < QGROUP / 32; ++k) {
    const long long idx = base + lane + 32 * k;
    keep[k] = 0.f;
    if (idx < B.numel) {
      float v = g[idx];
      float carry = 0.f;
      if (ef_mode == CONEF_EF_DENSE) v += dense_err[B.sk_off + idx];
      else if (ef_mode == CONEF_EF_QUANT8) {
        const float e = (float)qcodes[qbase + lane + 32 * k] * old_scale;
        v += alpha * e;
        carry = beta * e;
      }
      long long sp;
      if (in_block(B, idx, &sp)) {
        staging[sp] = v * gs;
        keep[k] = carry;
      } else {
        g[idx] = 0.f;
        keep[k] = carry + v;
      }
      if (ef_mode == CONEF_EF_DENSE) dense_err[B.sk_off + idx] = keep[k];
      amax = fmaxf(amax, fabsf(keep[k]));
    }
  }
  if (ef_mode == CONEF_EF_QUANT8) {
    amax = warp_max(amax);
    const float scale = amax / 127.f;
    const float inv = scale > 0.f ? 1.f / scale : 0.f;
#pragma unroll
    for (int k = 0; k < QGROUP / 32; ++k) {
      const long long idx = base + lane + 32 * k;
      if (idx < B.numel) {
        float q = rintf(keep[k] * inv);
        q = fminf(fmaxf(q, -127.f), 127.f);
        qcodes[qbase + lane + 32 * k] = (int8_t)q;
      }
    }
    if (lane == 0) qscales[sidx] = scale;
  }
}

// Row mapping for the count-sketch error store: tile = (tensor, row block).
__global__ void __launch_bounds__(256)
k_randblock_gather_sketch(const ConefBlk* __restrict__ blks, const int2* __restrict__ tiles, int rows_per_cta,
                          float* __restrict__ bucket, float* __restrict__ staging, float gather_scale,
                          float* __restrict__ sketch, const int32_t* __restrict__ tables,
                          const int32_t* __restrict__ counts, float alpha, float beta) {
  extern __shared__ float acc[];  // rows_per_cta * W
  const int2 t = tiles[blockIdx.x];
  const ConefBlk B = blks[t.x];
  const int m = B.m, W = B.W;
  const int row0 = t.y * rows_per_cta;
  const int rows = min(rows_per_cta, B.n - row0);
  for (int i = threadIdx.x; i < rows * W; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  const int32_t* tab = tables + B.tab_off;
  const float gs = gather_scale != 0.f ? gather_scale : (float)B.numel / (float)B.block;
  float* srow0 = sketch + B.sk_off + (size_t)row0 * W;
  float* g = bucket + B.g_off;
  for (int j = threadIdx.x; j < m; j += blockDim.x) {
    const int e = tab[j];
    const int h = unpack_bucket(e);
    const float s = unpack_sign(e);
    for (int ii = 0; ii < rows; ++ii) {
      const long long idx = (long long)(row0 + ii) * m + j;
      const float v = g[idx] + alpha * s * srow0[(size_t)ii * W + h];
      long long sp;
      if (in_block(B, idx, &sp)) {
        staging[sp] = v * gs;
      } else {
        g[idx] = 0.f;
        atomicAdd(&acc[ii * W + h], s * v);
      }
    }
  }
  __syncthreads();  // every read of the old sketch row is done
  const float omb = 1.f - beta;
  const int32_t* cnt = counts + B.cnt_off;
  for (int i = threadIdx.x; i < rows * W; i += blockDim.x)
    srow0[i] = srow0[i] * (1.f - omb * (float)cnt[i % W]) + acc[i];
}

extern "C" int conef_randblock_gather(const ConefBlk* blks, const int2* tiles, int ntiles, int rows_per_cta,
                                      float* bucket, float* staging, float gather_scale, float* sketch,
                                      const int32_t* tables, const int32_t* counts, float* dense_err,
                                      int8_t* qcodes, float* qscales, float alpha, float beta,
                                      int ef_mode, size_t smem_bytes, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  if (ef_mode == CONEF_EF_SKETCH) {
    if (smem_bytes > 220 * 1024) { conef_set_error("randblock_gather: sketch rows do not fit in shared memory"); return 2; }
    CONEF_CUDA(cudaFuncSetAttribute(k_randblock_gather_sketch, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
    k_randblock_gather_sketch<<<ntiles, 256, smem_bytes, stream>>>(blks, tiles, rows_per_cta, bucket, staging,
                                                                 gather_scale, sketch, tables, counts, alpha, beta);
  } else {
    k_randblock_gather_flat<<<(ntiles + 7) / 8, 256, 0, stream>>>(blks, tiles, ntiles, bucket, staging, gather_scale,
                                                               dense_err, qcodes, qscales, alpha, beta, ef_mode);
  }
  CONEF_CHECK_LAUNCH("k_randblock_gather");
  return 0;
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
