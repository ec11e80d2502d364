// Grouped PowerSGD pipeline, SIMT edition: every kernel processes all the
// compressed matrices of one DDP bucket in a single launch, driven by a
// device-resident table of ConefMat descriptors and a tile table.
//
// The error-corrected matrix M = G + e is never written: the products are linear, so
//   P = M Q   = G Q   + e Q        and      Q' = M^T P = G^T P + e^T P
// and the error term is one more "matrix" of the same launch.  For the count sketch,
// e = alpha * S H^T with the (n x W) sketch S and the sparse sign matrix H, hence
// e Q = S (alpha H^T Q) and e^T P = alpha H (S^T P): tall-skinny products over S, which is
// sketch_size times the size of G (csrc/sketch.cu has the two small H kernels).  For dense
// error feedback e is the error buffer itself.  The decompress kernel adds e on the fly.
//
// Replaces, per matrix and per step, of the reference (communication/powerSGD_hook.py):
//   :409  DenseCS.query        -> never materialised (see above)
//   :497  torch.matmul(M, Q)   -> k_psgd_p
//   :12-43 _orthogonalize      -> k_gram + k_qr_apply (csrc/orth.cu; all matrices of the bucket per launch)
//   :531  torch.matmul(M^T, P) -> k_psgd_q
//   :550  torch.matmul(P, Q^T), :558/:563 residual, CountSketch.py:27-67 update
//                              -> k_psgd_decompress (one pass, residual kept in registers)
#include <stdlib.h>
#include "common.cuh"

constexpr int P_WARPS = 8;       // warps per CTA in k_psgd_p
constexpr int P_WROWS = 4;       // matrix rows per warp: a Q row is loaded once for the four of them
constexpr int Q_THREADS = 256;   // columns per CTA in k_psgd_q
constexpr int D_THREADS = 256;

// Q[j, 0..r) scaled into registers.  With r a multiple of 4 and a 16-byte aligned block the row
// comes in as 16-byte loads: scalar loads of a stride-r pattern cost r wavefronts of mostly unused
// bytes per warp, which made the Q rows, not the gradient, the dominant load traffic.
template <int RP>
__device__ __forceinline__ void load_q_row(const float* __restrict__ q, int r, float q_scale, bool vec,
                                           float (&qv)[RP]) {
  if (RP >= 4 && vec) {
#pragma unroll
    for (int c = 0; c < RP; c += 4) {
      float4 x = make_float4(0.f, 0.f, 0.f, 0.f);
      if (c < r) x = __ldg(reinterpret_cast<const float4*>(q + c));
      qv[c] = x.x * q_scale;
      if (c + 1 < RP) qv[c + 1] = x.y * q_scale;
      if (c + 2 < RP) qv[c + 2] = x.z * q_scale;
      if (c + 3 < RP) qv[c + 3] = x.w * q_scale;
    }
  } else {
#pragma unroll
    for (int c = 0; c < RP; ++c) qv[c] = c < r ? __ldg(q + c) * q_scale : 0.f;
  }
}

// ---------------------------------------------------------------------------
// P (+)= A Q for every record of the table.  A warp owns P_WROWS matrix rows and walks the columns:
// the lanes read 32 consecutive entries of each row, the Q row of a column is loaded once (16-byte
// loads) for the rows of the warp.  A record reads its matrix from the gradient bucket (src = 0) or
// from the auxiliary buffer (src = 1: sketch arena or dense error buffer).
template <int RP>
__global__ void __launch_bounds__(P_WARPS * 32)
k_psgd_p(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, const float* __restrict__ bucket,
         const float* __restrict__ aux, const float* __restrict__ Q, float* __restrict__ P, int atomic_out) {
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row0 = (t.y * P_WARPS + warp) * P_WROWS;
  if (row0 >= M.n) return;
  const int rows = min(P_WROWS, M.n - row0);
  const int m = M.m, r = M.r;
  const float* g = (M.src ? aux : bucket) + M.g_off + (size_t)row0 * m;
  const float* q = Q + M.q_off;
  const bool qvec = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(q) & 15) == 0;
  float acc[P_WROWS][RP];
#pragma unroll
  for (int rr = 0; rr < P_WROWS; ++rr)
#pragma unroll
    for (int c = 0; c < RP; ++c) acc[rr][c] = 0.f;
  constexpr int PB = 4;      // column groups in flight per lane (times P_WROWS rows)
  for (int j0 = lane; j0 < m; j0 += 32 * PB) {
    float v[PB][P_WROWS];
#pragma unroll
    for (int u = 0; u < PB; ++u) {
      const int j = j0 + 32 * u;
#pragma unroll
      for (int rr = 0; rr < P_WROWS; ++rr) v[u][rr] = (j < m && rr < rows) ? g[(size_t)rr * m + j] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < PB; ++u) {
      const int j = j0 + 32 * u;
      if (j < m) {
        float qv[RP];
        load_q_row<RP>(q + (size_t)j * r, r, 1.f, qvec, qv);
#pragma unroll
        for (int rr = 0; rr < P_WROWS; ++rr)
#pragma unroll
          for (int c = 0; c < RP; ++c) acc[rr][c] = fmaf(v[u][rr], qv[c], acc[rr][c]);
      }
    }
  }
#pragma unroll
  for (int rr = 0; rr < P_WROWS; ++rr)
#pragma unroll
    for (int c = 0; c < RP; ++c) acc[rr][c] = warp_sum(acc[rr][c]);
  if (lane == 0) {
#pragma unroll
    for (int rr = 0; rr < P_WROWS; ++rr) {
      if (rr < rows) {
        float* p = P + M.p_off + (size_t)(row0 + rr) * r;
#pragma unroll
        for (int c = 0; c < RP; ++c) {
          if (c < r) {
            if (atomic_out) atomicAdd(p + c, acc[rr][c]);
            else p[c] = acc[rr][c];
          }
        }
      }
    }
  }
}

template <int RP>
static int launch_p(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket, const float* aux,
                    const float* Q, float* P, int atomic_out, cudaStream_t stream) {
  k_psgd_p<RP><<<ntiles, P_WARPS * 32, 0, stream>>>(mats, tiles, bucket, aux, Q, P, atomic_out);
  CONEF_CHECK_LAUNCH("k_psgd_p");
  return 0;
}

#define DISPATCH_RANK(max_rank, fn, ...)                                   \
  do {                                                                     \
    if ((max_rank) <= 1) return fn<1>(__VA_ARGS__);                        \
    if ((max_rank) <= 2) return fn<2>(__VA_ARGS__);                        \
    if ((max_rank) <= 4) return fn<4>(__VA_ARGS__);                        \
    if ((max_rank) <= 8) return fn<8>(__VA_ARGS__);                        \
    if ((max_rank) <= 16) return fn<16>(__VA_ARGS__);                      \
    if ((max_rank) <= 32) return fn<32>(__VA_ARGS__);                      \
    conef_set_error("rank %d > 32 is not supported by the native kernels", (max_rank)); \
    return 2;                                                              \
  } while (0)

extern "C" int conef_psgd_p(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket,
                            const float* aux, const float* Q, float* P, int atomic_out, int max_rank,
                            cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  DISPATCH_RANK(max_rank, launch_p, mats, tiles, ntiles, bucket, aux, Q, P, atomic_out, stream);
}

// ---------------------------------------------------------------------------
// Packed copies of the small operands for the tensor-core kernel (layout: conef_packed_offset).
__global__ void k_pack_small(const ConefMat* __restrict__ mats, int which, const float* __restrict__ src,
                             float* __restrict__ dst, int np) {
  const ConefMat M = mats[blockIdx.y];
  const int rows = which == 0 ? M.n : M.m;
  const int r = M.r;
  const float* a = src + (which == 0 ? M.p_off : M.q_off);
  const size_t total = (size_t)rows * r;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const long long row = i / r;
    const int c = (int)(i - row * r);
    conef_pack_store(dst, M, which, row, c, a[i], np);
  }
}

extern "C" int conef_pack_small(const ConefMat* mats, int nrec, int which, const float* src, float* dst,
                                int max_rank, cudaStream_t stream) {
  if (nrec <= 0) return 0;
  dim3 grid(16, nrec);
  k_pack_small<<<grid, 256, 0, stream>>>(mats, which, src, dst, max_rank <= 16 ? 16 : 32);
  CONEF_CHECK_LAUNCH("k_pack_small");
  return 0;
}

// ---------------------------------------------------------------------------
// Q = M^T P.  Tile = (matrix, row block, column block); a thread owns one
// column and walks the rows of the block, P rows are broadcast from shared
// memory.  Several row blocks of one matrix combine with fp32 atomics.
template <int RP>
__global__ void __launch_bounds__(Q_THREADS)
k_psgd_q(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, const float* __restrict__ bucket,
         const float* __restrict__ aux, const float* __restrict__ P, float* __restrict__ Q) {
  extern __shared__ float ps[];  // q_rows * RP
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int m = M.m, r = M.r;
  const int ncb = (m + Q_THREADS - 1) / Q_THREADS;
  const int rb = t.y / ncb, cb = t.y - rb * ncb;
  const int row0 = rb * M.q_rows;
  const int rows = min(M.q_rows, M.n - row0);
  const float* p = P + M.p_off + (size_t)row0 * r;
  for (int i = threadIdx.x; i < rows * RP; i += Q_THREADS) {
    const int ii = i / RP, c = i - ii * RP;
    ps[i] = c < r ? p[(size_t)ii * r + c] : 0.f;
  }
  __syncthreads();
  const int j = cb * Q_THREADS + threadIdx.x;
  if (j >= m) return;
  const float* g = (M.src ? aux : bucket) + M.g_off + (size_t)row0 * m + j;
  float acc[RP];
#pragma unroll
  for (int c = 0; c < RP; ++c) acc[c] = 0.f;
#pragma unroll 4
  for (int ii = 0; ii < rows; ++ii) {
    const float v = g[(size_t)ii * m];
#pragma unroll
    for (int c = 0; c < RP; ++c) acc[c] = fmaf(v, ps[ii * RP + c], acc[c]);
  }
  float* q = Q + M.q_off + (size_t)j * r;
  if (M.q_atomic) {
#pragma unroll
    for (int c = 0; c < RP; ++c)
      if (c < r) atomicAdd(q + c, acc[c]);
  } else {
#pragma unroll
    for (int c = 0; c < RP; ++c)
      if (c < r) q[c] = acc[c];
  }
}

template <int RP>
static int launch_q(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket, const float* aux,
                    const float* P, float* Q, size_t smem, cudaStream_t stream) {
  static bool configured[64] = {};      // the attribute is per device
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    CONEF_CUDA(cudaFuncSetAttribute(k_psgd_q<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  k_psgd_q<RP><<<ntiles, Q_THREADS, smem, stream>>>(mats, tiles, bucket, aux, P, Q);
  CONEF_CHECK_LAUNCH("k_psgd_q");
  return 0;
}

// Rows per row block never exceed CONEF_Q_MAX_ROWS (the host builds q_rows).
#define CONEF_Q_MAX_ROWS 1024

extern "C" int conef_psgd_q(const ConefMat* mats, const int2* tiles, int ntiles, const float* bucket,
                            const float* aux, const float* P, float* Q, int max_rank, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  int rp = max_rank <= 1 ? 1 : max_rank <= 2 ? 2 : max_rank <= 4 ? 4 : max_rank <= 8 ? 8 : max_rank <= 16 ? 16 : 32;
  size_t smem = (size_t)CONEF_Q_MAX_ROWS * rp * sizeof(float);
  DISPATCH_RANK(max_rank, launch_q, mats, tiles, ntiles, bucket, aux, P, Q, smem, stream);
}

// ---------------------------------------------------------------------------
// Decompress + error feedback.  Tile = (matrix, block of RB rows).
// A thread owns a column: it loads Q[j, :] (scaled by q_scale) and the column's hash
// entry once, then for the RB rows of the block loads G (all RB loads in flight before
// the first store: M_hat overwrites G in the same buffer), computes M_hat = <P[row, :], Q[j, :]>,
// writes it to the bucket and routes the residual M - M_hat to the error store.  Dense store:
// M = G + E, the residual goes to the buffer.  Count sketch: M = G + alpha * s_j * S[row, h_j], but
// the remembered term is never gathered: the update is linear, s_j^2 = 1, so
//     S'[row, w] = S[row, w] * (1 + (alpha - (1 - beta)) * k_w) + sum_{j: h_j = w} s_j * (G - M_hat)[row, j]
// and only the sum needs per-element work: one shared-memory atomic per element into the row's
// accumulator, flushed by one read-modify-write per sketch cell (a sketch row belongs to one CTA).
// A random shared-memory access per element costs about as much as streaming the element itself
// (measured: 42 us to stream a 147 MB matrix, +45 us per gather or atomic), hence no gather.
template <int RP, int RB>
__global__ void __launch_bounds__(D_THREADS, RP <= 8 ? 4 : 1)      // 64 registers: four CTAs per SM
k_psgd_decompress(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles,
                  float* __restrict__ bucket, const float* __restrict__ P, const float* __restrict__ Q,
                  float q_scale, float* __restrict__ sketch, const int32_t* __restrict__ tables,
                  const int32_t* __restrict__ counts, float* __restrict__ dense_err, float alpha, float beta,
                  int ef_mode) {
  extern __shared__ float sm[];
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int m = M.m, r = M.r, W = M.W, Wp = M.Wp;
  const int row0 = t.y * RB;
  const int rows = min(RB, M.n - row0);
  float* ps = sm;                          // RB * RP
  float* acc = sm + RB * RP;               // RB * W   signed residual sums (sketch mode)
  const float* p = P + M.p_off + (size_t)row0 * r;
  for (int i = threadIdx.x; i < RB * RP; i += D_THREADS) {
    const int ii = i / RP, c = i - ii * RP;
    ps[i] = (c < r && ii < rows) ? p[(size_t)ii * r + c] : 0.f;
  }
  float* srow = ef_mode == CONEF_EF_SKETCH ? sketch + M.sk_off + (size_t)row0 * Wp : nullptr;
  if (ef_mode == CONEF_EF_SKETCH)
    for (int i = threadIdx.x; i < rows * W; i += D_THREADS) acc[i] = 0.f;
  __syncthreads();

  const int32_t* tab = ef_mode == CONEF_EF_SKETCH ? tables + M.tab_off : nullptr;
  float* g0 = bucket + M.g_off + (size_t)row0 * m;
  float* e0 = ef_mode == CONEF_EF_DENSE ? dense_err + M.g_off + (size_t)row0 * m : nullptr;
  const bool qvec = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(Q + M.q_off) & 15) == 0;
  // Software pipeline: the RB loads of the next column are issued before the current column
  // is processed, so that loads stay in flight across the stores of M_hat.
  float v[RB], vn[RB];
  int j = threadIdx.x;
#pragma unroll
  for (int ii = 0; ii < RB; ++ii) {
    v[ii] = (ef_mode != CONEF_EF_NONE && ii < rows && j < m) ? __ldcs(g0 + (size_t)ii * m + j) : 0.f;
    if (ef_mode == CONEF_EF_DENSE && ii < rows && j < m) v[ii] += __ldcs(e0 + (size_t)ii * m + j);
  }
  for (; j < m; j += D_THREADS) {
    const int jn = j + D_THREADS;
#pragma unroll
    for (int ii = 0; ii < RB; ++ii)
      vn[ii] = (ef_mode != CONEF_EF_NONE && ii < rows && jn < m) ? __ldcs(g0 + (size_t)ii * m + jn) : 0.f;
    if (ef_mode == CONEF_EF_DENSE) {
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) if (ii < rows && jn < m) vn[ii] += __ldcs(e0 + (size_t)ii * m + jn);
    }
    float qv[RP];
    load_q_row<RP>(Q + M.q_off + (size_t)j * r, r, q_scale, qvec, qv);
    int h = 0;
    float s = 0.f;
    if (ef_mode == CONEF_EF_SKETCH) {
      const int e = __ldg(tab + j);
      h = unpack_bucket(e);
      s = unpack_sign(e);
    }
#pragma unroll
    for (int ii = 0; ii < RB; ++ii) {
      if (ii < rows) {
        float mh = 0.f;
#pragma unroll
        for (int c = 0; c < RP; ++c) mh = fmaf(ps[ii * RP + c], qv[c], mh);
        g0[(size_t)ii * m + j] = mh;
        if (ef_mode == CONEF_EF_SKETCH) {
          atomicAdd(&acc[ii * W + h], s * (v[ii] - mh));
        } else if (ef_mode == CONEF_EF_DENSE) {
          __stcs(e0 + (size_t)ii * m + j, v[ii] - mh);
        }
      }
    }
#pragma unroll
    for (int ii = 0; ii < RB; ++ii) v[ii] = vn[ii];
  }
  if (ef_mode == CONEF_EF_SKETCH) {
    __syncthreads();
    const float keep = alpha - (1.f - beta);
    const int32_t* cnt = counts + M.cnt_off;
    for (int i = threadIdx.x; i < rows * W; i += D_THREADS) {
      const int ii = i / W, h2 = i - ii * W;
      float* c = srow + (size_t)ii * Wp + h2;
      *c = *c * (1.f + keep * (float)__ldg(cnt + h2)) + acc[i];
    }
  }
}

// Count-sketch decompress over the block layout of the hash (conef_cell, layout 1: columns hashed in
// aligned groups of 32, one group per cell block and window of nb = W / 32 groups).  The table arena
// holds, per matrix, S x nb two-word records, window-major: {g | x_g << 27 (0x7ffffff: none), sign bits
// of the group's 32 columns} = the group cell block c receives from window s.
// Work unit of a warp: (rbu consecutive blocks of RB rows, cell block c).  The warp walks the S groups of
// its cell block once per row block; lane l handles column 32 g + (l xor x_g), whose cell is 32 c + l for
// every one of them, so the 32 sums of the cell block stay in the lanes' registers: no atomics, no
// shared-memory accumulator, all warps do the same amount of work, and every access of a warp is one
// full 128-byte line (G row segment, M_hat row segment, sketch cells).  A CTA's eight warps take
// neighbouring cell blocks of the same rows and therefore read inside the same window of the row at
// about the same time.  The records of the cell block are fetched up front (one per lane) and handed
// round by shuffles, so addresses never wait for a load.  G and the Q rows travel through a per-warp
// ring in shared memory filled by cp.async: D_STAGES - 1 groups (3 KB of G per warp) are in flight at
// no cost in registers, across the boundaries between row blocks; a lane reads back only what it
// copied itself, so the ring needs no barriers.  The kernel moves 4 bytes per lane and instruction,
// which makes the instruction count per row its second limit after load latency: row addresses are one
// multiply-add on a 32-bit byte stride, shared memory is addressed with immediates off one register
// per stage, and row blocks with all RB rows skip the per-row predicates.
// Tile = (matrix, chunk of eight consecutive units of that matrix).
constexpr int D_WARPS = D_THREADS / 32;
constexpr int D_STAGES = 4;       // ring depth (a power of two)
constexpr int D_RBU_MAX = 4;      // most row blocks per unit

// mbarrier + bulk-copy (TMA without a tensor map) helpers of the ring's second filling mode
// Every probe may sleep in hardware for up to the hinted time, so the limit below is seconds, and a
// warp that waits does not spend issue slots on a spin loop.
constexpr int D_MBAR_PROBES = 1 << 18;
constexpr uint32_t D_MBAR_SUSPEND_NS = 2000;
__device__ __forceinline__ void dmbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void dmbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool dmbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity), "r"(D_MBAR_SUSPEND_NS) : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool dmbar_wait(uint32_t bar, uint32_t parity) {      // bounded
  for (int it = 0; it < D_MBAR_PROBES; ++it)
    if (dmbar_try_wait(bar, parity)) return true;
  return false;
}
// untiled bulk copy global -> shared: both addresses 16-byte aligned, size a multiple of 16 bytes
__device__ __forceinline__ void dbulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

template <int RP, int RB>
struct DblkLayout {
  static constexpr int MBAR_BYTES = 64;                           // D_STAGES mbarriers (bulk-copy mode)
  static constexpr int STAGE_BYTES = RB * 128 + 32 * RP * 4;      // G [RB][32] | Q rows [32][RP]
  static constexpr int PS_BYTES = D_RBU_MAX * RB * RP * 4;        // P rows of the unit
  static constexpr int WARP_BYTES = MBAR_BYTES + PS_BYTES + D_STAGES * STAGE_BYTES;
  static constexpr int CTA_BYTES = D_WARPS * WARP_BYTES;
  static_assert(D_STAGES * 8 <= MBAR_BYTES && PS_BYTES % 16 == 0 && STAGE_BYTES % 16 == 0, "ring layout");
};

// One chunk (at most 32 groups) of the walk over `nrbh` row blocks.  FULL: every row block has RB rows.
template <int RP, int RB, bool FULL>
__device__ __forceinline__ void dblk_walk(int2 mine, int cnt, bool last_chunk, bool first_chunk, int nrbh, int m,
                                          int r, int rows_total, float* __restrict__ g0,
                                          const float* __restrict__ q0, float q_scale, bool qvec, uint32_t ps,
                                          uint32_t ring_g, uint32_t ring_q, int lane, float* __restrict__ sc0,
                                          int Wp, float f, float (&acc)[RB], float (&so)[RB]) {
  using L = DblkLayout<RP, RB>;
  const unsigned pitch = (unsigned)m * 4u;      // bytes between rows
  auto row_ptr = [&](float* base, int ii) {
    return reinterpret_cast<float*>(reinterpret_cast<char*>(base) + (unsigned long long)pitch * (unsigned)ii);
  };
  // column of this lane in the i-th group of the chunk (m: none); every lane calls it together
  auto column = [&](int i) {
    const int rx = __shfl_sync(0xffffffffu, mine.x, i & 31);
    const int g = rx & 0x7ffffff;
    return (i < cnt && g != 0x7ffffff) ? (g << 5) + (lane ^ (int)((uint32_t)rx >> 27)) : m;
  };
  const int total = nrbh * cnt;
  // issue side: item k_i = (row block rb_i, group i_i)
  int k_i = 0, rb_i = 0, i_i = 0;
  float* g_i = g0;
  auto issue = [&]() {
    if (k_i < total) {
      const int cl = column(i_i);
      if (cl < m) {
        float* src = g_i + cl;
        const uint32_t stage = (uint32_t)(k_i & (D_STAGES - 1)) * L::STAGE_BYTES;
        const uint32_t dst = ring_g + stage;
        const int rows = FULL ? RB : min(RB, rows_total - rb_i * RB);
#pragma unroll
        for (int ii = 0; ii < RB; ++ii)
          if (FULL || ii < rows) cp_async_f32<0>(dst + ii * 128, row_ptr(src, ii));
        const float* qs = q0 + (size_t)cl * r;
        const uint32_t qd = ring_q + stage;
        if (qvec) {
#pragma unroll
          for (int cc = 0; cc < RP; cc += 4)
            if (cc < r) cp_async_16<0>(qd + cc * 4, qs + cc);
        } else {
#pragma unroll
          for (int cc = 0; cc < RP; ++cc)
            if (cc < r) cp_async_f32<0>(qd + cc * 4, qs + cc);
        }
      }
      ++k_i;
      if (++i_i == cnt) { i_i = 0; ++rb_i; g_i = row_ptr(g_i, RB); }
    }
    cp_async_commit();
  };
#pragma unroll
  for (int k = 0; k < D_STAGES - 1; ++k) issue();
  int rb_p = 0, i_p = 0;
  float* g_p = g0;
  float* sc_p = sc0;
  uint32_t ps_p = ps;
  for (int k = 0; k < total; ++k) {
    issue();
    const int col = column(i_p);
    const uint32_t sbits = (uint32_t)__shfl_sync(0xffffffffu, mine.y, i_p & 31);
    const int rows = FULL ? RB : min(RB, rows_total - rb_p * RB);
    if (i_p == 0) {
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        if (first_chunk) acc[ii] = 0.f;
        if (last_chunk) so[ii] = (FULL || ii < rows) ? sc_p[(size_t)ii * Wp] : 0.f;      // in flight during the walk
      }
    }
    cp_async_wait<D_STAGES - 1>();      // the copies of item k have landed
    if (col < m) {
      const float sgn = ((sbits >> (col & 31)) & 1u) ? 1.f : -1.f;
      float* dstp = g_p + col;
      const uint32_t stage = (uint32_t)(k & (D_STAGES - 1)) * L::STAGE_BYTES;
      const uint32_t src = ring_g + stage;
      float qv[RP];
#pragma unroll
      for (int cc = 0; cc < RP; cc += 4) {
        const float4 q4 = lds_f32x4<0>(ring_q + stage + cc * 4);
        qv[cc] = q4.x * q_scale;
        qv[cc + 1] = q4.y * q_scale;
        qv[cc + 2] = q4.z * q_scale;
        qv[cc + 3] = q4.w * q_scale;
      }
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        if (FULL || ii < rows) {
          float mh = 0.f;
#pragma unroll
          for (int cc = 0; cc < RP; cc += 4) {
            const float4 pv = lds_f32x4<0>(ps_p + (ii * RP + cc) * 4);
            mh = fmaf(pv.x, qv[cc], mh);
            mh = fmaf(pv.y, qv[cc + 1], mh);
            mh = fmaf(pv.z, qv[cc + 2], mh);
            mh = fmaf(pv.w, qv[cc + 3], mh);
          }
          const float v = lds_f32<0>(src + ii * 128);
          *row_ptr(dstp, ii) = mh;
          acc[ii] = fmaf(sgn, v - mh, acc[ii]);
        }
      }
    }
    if (++i_p == cnt) {
      if (last_chunk) {
#pragma unroll
        for (int ii = 0; ii < RB; ++ii)
          if (FULL || ii < rows) sc_p[(size_t)ii * Wp] = fmaf(so[ii], f, acc[ii]);
      }
      i_p = 0;
      ++rb_p;
      g_p = row_ptr(g_p, RB);
      sc_p += (size_t)RB * Wp;
      ps_p += RB * RP * 4;
    }
  }
  cp_async_wait<0>();
}

// The same walk with the ring filled by bulk copies (the TMA engine instead of the load/store unit, which
// otherwise carries every byte of G twice: global -> shared, shared -> register): per item the warp posts
// RB row segments of 128 bytes and the 32 Q rows of the group on the stage's mbarrier; every lane then
// reads column (lane xor x_g) of the stage.  Needs 16-byte aligned row segments (matrix start and row
// pitch), no ragged last group (m a multiple of 32), r == RP and one chunk (at most 32 windows).  Waits
// are bounded: a wait that runs out reports CONEF_STATUS_MBAR_TIMEOUT, the copies still in flight are
// waited for (bounded again), and the unit is given up.  Returns false in that case.
template <int RP, int RB, bool FULL>
__device__ __forceinline__ bool dblk_walk_bulk(int2 mine, int cnt, int nrbh, int m, int rows_total,
                                               float* __restrict__ g0, const float* __restrict__ q0, float q_scale,
                                               uint32_t ps, uint32_t ring0, uint32_t bar0, int lane,
                                               float* __restrict__ sc0, int Wp, float f, int* __restrict__ status) {
  using L = DblkLayout<RP, RB>;
  const unsigned pitch = (unsigned)m * 4u;
  auto row_ptr = [&](float* base, int ii) {
    return reinterpret_cast<float*>(reinterpret_cast<char*>(base) + (unsigned long long)pitch * (unsigned)ii);
  };
  const int total = nrbh * cnt;
  int k_i = 0, rb_i = 0, i_i = 0;
  float* g_i = g0;
  uint32_t pending = 0;      // stages with copies in flight
  auto issue = [&]() {
    if (k_i < total) {
      const int rx = __shfl_sync(0xffffffffu, mine.x, i_i);
      const int g = rx & 0x7ffffff;
      const int st = k_i & (D_STAGES - 1);
      if (g != 0x7ffffff) {
        const int rows = FULL ? RB : min(RB, rows_total - rb_i * RB);
        const uint32_t bar = bar0 + st * 8;
        const uint32_t dst = ring0 + (uint32_t)st * L::STAGE_BYTES;
        __syncwarp();      // every lane is done reading the stage that is refilled
        if (lane == 0) dmbar_expect_tx(bar, (uint32_t)rows * 128u + 32u * RP * 4u);
        __syncwarp();      // the transaction count is posted before any copy can complete
        // lanes 0 .. rows - 1 post one row segment each, lane RB the Q rows: two instructions for the warp
        if (lane < rows) dbulk_load(dst + lane * 128, row_ptr(g_i + (g << 5), lane), 128u, bar);
        else if (lane == RB) dbulk_load(dst + RB * 128, q0 + (size_t)(g << 5) * RP, 32u * RP * 4u, bar);
        pending |= 1u << st;
      }
      ++k_i;
      if (++i_i == cnt) { i_i = 0; ++rb_i; g_i = row_ptr(g_i, RB); }
    }
  };
#pragma unroll
  for (int k = 0; k < D_STAGES - 1; ++k) issue();
  float so[RB], acc[RB];
  int rb_p = 0, i_p = 0;
  float* g_p = g0;
  float* sc_p = sc0;
  uint32_t ps_p = ps;
  uint32_t parity = 0;       // bit st: phase parity the next wait on stage st expects
  for (int k = 0; k < total; ++k) {
    issue();
    const int rx = __shfl_sync(0xffffffffu, mine.x, i_p);
    const uint32_t sbits = (uint32_t)__shfl_sync(0xffffffffu, mine.y, i_p);
    const int g = rx & 0x7ffffff;
    const int rows = FULL ? RB : min(RB, rows_total - rb_p * RB);
    if (i_p == 0) {
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        acc[ii] = 0.f;
        so[ii] = (FULL || ii < rows) ? sc_p[(size_t)ii * Wp] : 0.f;      // in flight during the walk
      }
    }
    if (g != 0x7ffffff) {
      const int st = k & (D_STAGES - 1);
      if (!dmbar_wait(bar0 + st * 8, (parity >> st) & 1u)) {
        if (lane == 0) atomicExch(status, CONEF_STATUS_MBAR_TIMEOUT);
        for (int s2 = 0; s2 < D_STAGES; ++s2)
          if ((pending >> s2) & 1u) dmbar_wait(bar0 + s2 * 8, (parity >> s2) & 1u);
        return false;
      }
      parity ^= 1u << st;
      pending &= ~(1u << st);
      const int lx = lane ^ (int)((uint32_t)rx >> 27);      // this lane's column inside the group
      const float sgn = ((sbits >> lx) & 1u) ? 1.f : -1.f;
      float* dstp = g_p + (g << 5) + lx;
      const uint32_t stage = ring0 + (uint32_t)st * L::STAGE_BYTES;
      const uint32_t src = stage + lx * 4;
      const uint32_t qsrc = stage + RB * 128 + lx * (RP * 4);
      float qv[RP];
#pragma unroll
      for (int cc = 0; cc < RP; cc += 4) {
        const float4 q4 = lds_f32x4<0>(qsrc + cc * 4);
        qv[cc] = q4.x * q_scale;
        qv[cc + 1] = q4.y * q_scale;
        qv[cc + 2] = q4.z * q_scale;
        qv[cc + 3] = q4.w * q_scale;
      }
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        if (FULL || ii < rows) {
          float mh = 0.f;
#pragma unroll
          for (int cc = 0; cc < RP; cc += 4) {
            const float4 pv = lds_f32x4<0>(ps_p + (ii * RP + cc) * 4);
            mh = fmaf(pv.x, qv[cc], mh);
            mh = fmaf(pv.y, qv[cc + 1], mh);
            mh = fmaf(pv.z, qv[cc + 2], mh);
            mh = fmaf(pv.w, qv[cc + 3], mh);
          }
          const float v = lds_f32<0>(src + ii * 128);
          *row_ptr(dstp, ii) = mh;
          acc[ii] = fmaf(sgn, v - mh, acc[ii]);
        }
      }
    }
    if (++i_p == cnt) {
#pragma unroll
      for (int ii = 0; ii < RB; ++ii)
        if (FULL || ii < rows) sc_p[(size_t)ii * Wp] = fmaf(so[ii], f, acc[ii]);
      i_p = 0;
      ++rb_p;
      g_p = row_ptr(g_p, RB);
      sc_p += (size_t)RB * Wp;
      ps_p += RB * RP * 4;
    }
  }
  return true;
}

template <int RP, int RB>
__global__ void __launch_bounds__(D_THREADS, RP <= 8 ? 3 : 1)
k_psgd_decompress_blk(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles,
                      float* __restrict__ bucket, const float* __restrict__ P, const float* __restrict__ Q,
                      float q_scale, float* __restrict__ sketch, const int32_t* __restrict__ tables,
                      const int32_t* __restrict__ counts, float alpha, float beta, int rbu, int bulk,
                      int* __restrict__ status) {
  static_assert((D_STAGES & (D_STAGES - 1)) == 0, "the ring is indexed with a mask");
  using L = DblkLayout<RP, RB>;
  extern __shared__ __align__(16) unsigned char dblk_smem[];
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m = M.m, r = M.r, Wp = M.Wp, nb = M.W >> 5;
  const int S = (((m + 31) >> 5) + nb - 1) / nb;
  const int nrb = (M.n + RB - 1) / RB;
  const int R = S <= 32 ? min(max(rbu, 1), D_RBU_MAX) : 1;      // the host counts units the same way
  const int unit = t.y * D_WARPS + warp;
  if (unit >= ((nrb + R - 1) / R) * nb) return;      // nothing below synchronises the CTA
  const int ru = unit / nb, c = unit - ru * nb;
  const int nrbh = min(R, nrb - ru * R);
  const int row0 = ru * R * RB;
  const int rows_total = min(nrbh * RB, M.n - row0);
  unsigned char* mine_smem = dblk_smem + (size_t)warp * L::WARP_BYTES;
  float* psf = reinterpret_cast<float*>(mine_smem + L::MBAR_BYTES);
  {
    const float* p = P + M.p_off + (size_t)row0 * r;
    for (int i = lane; i < nrbh * RB * RP; i += 32) {
      const int ii = i / RP, cc = i - ii * RP;
      psf[i] = (cc < r && ii < rows_total) ? p[(size_t)ii * r + cc] : 0.f;
    }
    // the pad columns of the Q rows in the ring are never copied: they meet zeros of P, but must be finite
    float* ringf = reinterpret_cast<float*>(mine_smem + L::MBAR_BYTES + L::PS_BYTES);
    for (int st = 0; st < D_STAGES; ++st)
      for (int cc = 0; cc < RP; ++cc) ringf[st * (L::STAGE_BYTES / 4) + RB * 32 + lane * RP + cc] = 0.f;
  }
  __syncwarp();
  const uint32_t bar0 = (uint32_t)__cvta_generic_to_shared(mine_smem);
  const uint32_t ps = bar0 + L::MBAR_BYTES;
  const uint32_t ring0 = ps + L::PS_BYTES;
  // per-lane views of a ring stage: G element (ii, lane) at ring_g + ii * 128, this lane's Q row at ring_q
  const uint32_t ring_g = ring0 + lane * 4;
  const uint32_t ring_q = ring0 + RB * 128 + lane * (RP * 4);
  const int2* recs = reinterpret_cast<const int2*>(tables + M.cb_off) + c;
  float* g0 = bucket + M.g_off + (size_t)row0 * m;
  const float* q0 = Q + M.q_off;
  const bool qvec = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(q0) & 15) == 0;
  const int cell = (c << 5) + lane;
  float* sc0 = sketch + M.sk_off + (size_t)row0 * Wp + cell;
  const float f = 1.f + (alpha - (1.f - beta)) * (float)__ldg(counts + M.cnt_off + cell);
  const bool full = rows_total == nrbh * RB;
  // bulk copies: 16-byte aligned row segments and Q rows, whole groups only, one chunk
  if (bulk && S <= 32 && r == RP && (m & 31) == 0 && (reinterpret_cast<uintptr_t>(bucket + M.g_off) & 15) == 0 &&
      (reinterpret_cast<uintptr_t>(q0) & 15) == 0) {
    if (lane == 0) {
      for (int st = 0; st < D_STAGES; ++st) dmbar_init(bar0 + st * 8, 1);
      asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // the ring was written with plain stores above
    __syncwarp();
    int2 mine = make_int2(0x7ffffff, 0);
    if (lane < S) mine = __ldg(recs + (size_t)lane * nb);
    if (full)
      dblk_walk_bulk<RP, RB, true>(mine, S, nrbh, m, rows_total, g0, q0, q_scale, ps, ring0, bar0, lane, sc0, Wp, f,
                                   status);
    else
      dblk_walk_bulk<RP, RB, false>(mine, S, nrbh, m, rows_total, g0, q0, q_scale, ps, ring0, bar0, lane, sc0, Wp, f,
                                    status);
    return;
  }
  float acc[RB], so[RB];
  for (int s0 = 0; s0 < S; s0 += 32) {
    int2 mine = make_int2(0x7ffffff, 0);
    if (s0 + lane < S) mine = __ldg(recs + (size_t)(s0 + lane) * nb);
    const int cnt = min(32, S - s0);
    if (full)
      dblk_walk<RP, RB, true>(mine, cnt, s0 + cnt == S, s0 == 0, nrbh, m, r, rows_total, g0, q0, q_scale, qvec, ps,
                              ring_g, ring_q, lane, sc0, Wp, f, acc, so);
    else
      dblk_walk<RP, RB, false>(mine, cnt, s0 + cnt == S, s0 == 0, nrbh, m, r, rows_total, g0, q0, q_scale, qvec, ps,
                               ring_g, ring_q, lane, sc0, Wp, f, acc, so);
  }
}

// Decompress for dense error feedback and for no error feedback: M_hat = P Q^T into the bucket and, with dense
// feedback, E' = G + E - M_hat into the error buffer.  Same machinery as k_psgd_decompress_blk without the hash:
// tile = (matrix, block of RB rows); warp w of the CTA walks the column groups w, w + 8, w + 16, ... (the eight
// warps together read 1 KB of every row at a time), lane l owns column 32 g + l.  G, E and the Q rows travel
// through the per-warp cp.async ring (D_STAGES - 1 groups in flight); without error feedback only the Q rows do,
// and the kernel is a pure store stream.  The column-order kernel it replaces for these modes issued the loads
// of one group ahead through registers and reached 0.55 (dense) and 0.31 (none) of copy bandwidth.
template <int RP, int RB, int MODE>      // MODE: CONEF_EF_DENSE or CONEF_EF_NONE
__global__ void __launch_bounds__(D_THREADS, RP <= 8 ? 3 : 1)
k_psgd_decompress_str(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, float* __restrict__ bucket,
                      const float* __restrict__ P, const float* __restrict__ Q, float q_scale,
                      float* __restrict__ dense_err) {
  constexpr int NSRC = MODE == CONEF_EF_DENSE ? 2 : 0;                 // row arrays that go through the ring
  constexpr int STAGE_BYTES = NSRC * RB * 128 + 32 * RP * 4;          // [G [RB][32] | E [RB][32]] | Q rows [32][RP]
  constexpr int PS_BYTES = RB * RP * 4;
  constexpr int WARP_BYTES = D_STAGES * STAGE_BYTES;
  extern __shared__ __align__(16) unsigned char dstr_smem[];
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int m = M.m, r = M.r;
  const int row0 = t.y * RB;
  const int rows = min(RB, M.n - row0);
  float* psf = reinterpret_cast<float*>(dstr_smem);      // P rows of the tile, shared by the warps
  {
    const float* p = P + M.p_off + (size_t)row0 * r;
    for (int i = threadIdx.x; i < RB * RP; i += D_THREADS) {
      const int ii = i / RP, cc = i - ii * RP;
      psf[i] = (cc < r && ii < rows) ? p[(size_t)ii * r + cc] : 0.f;
    }
    // the pad columns of the Q rows in the ring are never copied: they meet zeros of P, but must be finite
    float* ringf = reinterpret_cast<float*>(dstr_smem + PS_BYTES + (size_t)warp * WARP_BYTES);
    for (int st = 0; st < D_STAGES; ++st)
      for (int cc = 0; cc < RP; ++cc) ringf[st * (STAGE_BYTES / 4) + NSRC * RB * 32 + lane * RP + cc] = 0.f;
  }
  __syncthreads();
  const uint32_t ps = (uint32_t)__cvta_generic_to_shared(dstr_smem);
  const uint32_t ring0 = ps + PS_BYTES + warp * WARP_BYTES;
  const uint32_t ring_g = ring0 + lane * 4;                              // G element (ii, lane) at + ii * 128
  const uint32_t ring_q = ring0 + NSRC * RB * 128 + lane * (RP * 4);     // this lane's Q row
  float* g0 = bucket + M.g_off + (size_t)row0 * m;
  float* e0 = MODE == CONEF_EF_DENSE ? dense_err + M.g_off + (size_t)row0 * m : nullptr;
  const float* q0 = Q + M.q_off;
  const bool qvec = (r & 3) == 0 && (reinterpret_cast<uintptr_t>(q0) & 15) == 0;
  const unsigned pitch = (unsigned)m * 4u;
  auto row_ptr = [&](float* base, int ii) {
    return reinterpret_cast<float*>(reinterpret_cast<char*>(base) + (unsigned long long)pitch * (unsigned)ii);
  };
  const int ng = (m + 31) >> 5;
  const int total = (ng - warp + D_WARPS - 1) / D_WARPS;      // groups of this warp: warp, warp + 8, ...
  const bool full = rows == RB;
  int k_i = 0;
  auto issue = [&]() {
    if (k_i < total) {
      const int cl = ((warp + k_i * D_WARPS) << 5) + lane;
      if (cl < m) {
        const uint32_t stage = (uint32_t)(k_i & (D_STAGES - 1)) * STAGE_BYTES;
        if (MODE == CONEF_EF_DENSE) {
#pragma unroll
          for (int ii = 0; ii < RB; ++ii) {
            if (full || ii < rows) {
              cp_async_f32<0>(ring_g + stage + ii * 128, row_ptr(g0 + cl, ii));
              cp_async_f32<0>(ring_g + stage + (RB + ii) * 128, row_ptr(e0 + cl, ii));
            }
          }
        }
        const float* qs = q0 + (size_t)cl * r;
        if (qvec) {
#pragma unroll
          for (int cc = 0; cc < RP; cc += 4)
            if (cc < r) cp_async_16<0>(ring_q + stage + cc * 4, qs + cc);
        } else {
#pragma unroll
          for (int cc = 0; cc < RP; ++cc)
            if (cc < r) cp_async_f32<0>(ring_q + stage + cc * 4, qs + cc);
        }
      }
      ++k_i;
    }
    cp_async_commit();
  };
#pragma unroll
  for (int k = 0; k < D_STAGES - 1; ++k) issue();
  for (int k = 0; k < total; ++k) {
    issue();
    const int col = ((warp + k * D_WARPS) << 5) + lane;
    cp_async_wait<D_STAGES - 1>();      // the copies of group k have landed
    if (col < m) {
      const uint32_t stage = (uint32_t)(k & (D_STAGES - 1)) * STAGE_BYTES;
      float qv[RP];
#pragma unroll
      for (int cc = 0; cc < RP; cc += 4) {
        const float4 q4 = lds_f32x4<0>(ring_q + stage + cc * 4);
        qv[cc] = q4.x * q_scale;
        qv[cc + 1] = q4.y * q_scale;
        qv[cc + 2] = q4.z * q_scale;
        qv[cc + 3] = q4.w * q_scale;
      }
      float* gp = g0 + col;
      float* ep = MODE == CONEF_EF_DENSE ? e0 + col : nullptr;
#pragma unroll
      for (int ii = 0; ii < RB; ++ii) {
        if (full || ii < rows) {
          float mh = 0.f;
#pragma unroll
          for (int cc = 0; cc < RP; cc += 4) {
            const float4 pv = lds_f32x4<0>(ps + (ii * RP + cc) * 4);
            mh = fmaf(pv.x, qv[cc], mh);
            mh = fmaf(pv.y, qv[cc + 1], mh);
            mh = fmaf(pv.z, qv[cc + 2], mh);
            mh = fmaf(pv.w, qv[cc + 3], mh);
          }
          *row_ptr(gp, ii) = mh;
          if (MODE == CONEF_EF_DENSE) {
            const float v = lds_f32<0>(ring_g + stage + ii * 128) + lds_f32<0>(ring_g + stage + (RB + ii) * 128);
            __stcs(row_ptr(ep, ii), v - mh);
          }
        }
      }
    }
  }
  cp_async_wait<0>();
}

template <int RP, int RB, int MODE>
static int launch_d_str(const ConefMat* mats, const int2* tiles, int ntiles, float* bucket, const float* P,
                        const float* Q, float q_scale, float* dense_err, cudaStream_t stream) {
  constexpr int NSRC = MODE == CONEF_EF_DENSE ? 2 : 0;
  constexpr int smem = RB * RP * 4 + D_WARPS * D_STAGES * (NSRC * RB * 128 + 32 * RP * 4);
  static bool opted[64] = {};
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || !opted[dev])) {
    CONEF_CUDA(cudaFuncSetAttribute(k_psgd_decompress_str<RP, RB, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64) opted[dev] = true;
  }
  k_psgd_decompress_str<RP, RB, MODE><<<ntiles, D_THREADS, smem, stream>>>(mats, tiles, bucket, P, Q, q_scale, dense_err);
  CONEF_CHECK_LAUNCH("k_psgd_decompress_str");
  return 0;
}

template <int RP, int RB>
static int launch_d_rb(const ConefMat* mats, const int2* tiles, int ntiles, int nblk, int rbu, int bulk, int* status,
                       float* bucket, const float* P,
                       const float* Q, float q_scale, float* sketch, const int32_t* tables,
                       const int32_t* counts, float* dense_err, float alpha, float beta, int ef_mode,
                       size_t smem, cudaStream_t stream) {
  smem += (size_t)RB * RP * sizeof(float);
  if (smem > 220 * 1024) { conef_set_error("decompress: %zu bytes of shared memory needed", smem); return 2; }
  static size_t configured[64] = {};    // largest opt-in so far, per device (the attribute is per device)
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
    CONEF_CUDA(cudaFuncSetAttribute(k_psgd_decompress<RP, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = smem;
  }
  if (nblk > 0) {
    constexpr int RQ = RP < 4 ? 4 : RP;
    constexpr int blk_smem = DblkLayout<RQ, RB>::CTA_BYTES;
    static bool opted[64] = {};
    if (blk_smem > 48 * 1024 && (dev < 0 || dev >= 64 || !opted[dev])) {
      CONEF_CUDA(cudaFuncSetAttribute(k_psgd_decompress_blk<RQ, RB>, cudaFuncAttributeMaxDynamicSharedMemorySize, blk_smem));
      if (dev >= 0 && dev < 64) opted[dev] = true;
    }
    k_psgd_decompress_blk<RQ, RB><<<nblk, D_THREADS, blk_smem, stream>>>(mats, tiles, bucket, P, Q, q_scale, sketch,
                                                                        tables, counts, alpha, beta, rbu, bulk, status);
    CONEF_CHECK_LAUNCH("k_psgd_decompress_blk");
  }
  if (ef_mode == CONEF_EF_DENSE || ef_mode == CONEF_EF_NONE) {
    const char* legacy = getenv("CONEF_D_STREAM");      // "0": the column-order kernel for these modes too
    if (!(legacy && legacy[0] == '0')) {
      constexpr int RQ = RP < 4 ? 4 : RP;
      if (ef_mode == CONEF_EF_DENSE)
        return launch_d_str<RQ, RB, CONEF_EF_DENSE>(mats, tiles, ntiles, bucket, P, Q, q_scale, dense_err, stream);
      return launch_d_str<RQ, RB, CONEF_EF_NONE>(mats, tiles, ntiles, bucket, P, Q, q_scale, dense_err, stream);
    }
  }
  if (ntiles > nblk) {
    k_psgd_decompress<RP, RB><<<ntiles - nblk, D_THREADS, smem, stream>>>(mats, tiles + nblk, bucket, P, Q, q_scale,
                                                                       sketch, tables, counts, dense_err, alpha,
                                                                       beta, ef_mode);
    CONEF_CHECK_LAUNCH("k_psgd_decompress");
  }
  return 0;
}

template <int RP>
static int launch_d(const ConefMat* mats, const int2* tiles, int ntiles, int nblk, int rbu, int bulk, int* status,
                    int rows_per_cta, float* bucket,
                    const float* P, const float* Q, float q_scale, float* sketch, const int32_t* tables,
                    const int32_t* counts, float* dense_err, float alpha, float beta, int ef_mode, size_t smem,
                    cudaStream_t stream) {
#define CONEF_D_CASE(RB)                                                                              \
  case RB: return launch_d_rb<RP, RB>(mats, tiles, ntiles, nblk, rbu, bulk, status, bucket, P, Q, q_scale, sketch, tables, counts, \
                                      dense_err, alpha, beta, ef_mode, smem, stream)
  switch (rows_per_cta) {
    CONEF_D_CASE(8);
    CONEF_D_CASE(4);
    CONEF_D_CASE(2);
    CONEF_D_CASE(1);
  }
#undef CONEF_D_CASE
  conef_set_error("decompress: rows_per_cta must be 1, 2, 4 or 8 (got %d)", rows_per_cta);
  return 2;
}

extern "C" int conef_psgd_decompress(const ConefMat* mats, const int2* tiles, int ntiles, int nblk_tiles, int rbu,
                                     int rows_per_cta,
                                     float* bucket, const float* P, const float* Q, float q_scale,
                                     float* sketch, const int32_t* tables, const int32_t* counts,
                                     float* dense_err, float alpha, float beta, int ef_mode, int max_rank,
                                     size_t smem_bytes, int* status, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  const char* bulk_env = getenv("CONEF_D_BULK");      // "0": fill the ring with cp.async everywhere
  const int bulk = (status != nullptr && !(bulk_env && bulk_env[0] == '0')) ? 1 : 0;
  if (ef_mode != CONEF_EF_SKETCH || nblk_tiles < 0) nblk_tiles = 0;
  if (nblk_tiles > ntiles) nblk_tiles = ntiles;
  DISPATCH_RANK(max_rank, launch_d, mats, tiles, ntiles, nblk_tiles, rbu, bulk, status, rows_per_cta, bucket, P, Q, q_scale, sketch, tables,
                counts, dense_err, alpha, beta, ef_mode, smem_bytes, stream);
}

// ---------------------------------------------------------------------------
// Counter-based standard normal fill (Philox-4x32-10 + Box-Muller, common.cuh): the value
// of element e depends only on (seed, e).
__global__ void k_fill_normal(float* __restrict__ buf, long long numel, uint64_t seed) {
  const long long quad = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long base = quad * 4;
  if (base >= numel) return;
  float out[4];
  conef_philox_normal4(seed, (uint64_t)quad, out);
  for (int i = 0; i < 4; ++i)
    if (base + i < numel) buf[base + i] = out[i];
}

extern "C" int conef_fill_normal(float* buf, long long numel, uint64_t seed, cudaStream_t stream) {
  if (numel <= 0) return 0;
  const long long quads = (numel + 3) / 4;
  k_fill_normal<<<(unsigned)((quads + 255) / 256), 256, 0, stream>>>(buf, numel, seed);
  CONEF_CHECK_LAUNCH("k_fill_normal");
  return 0;
}

