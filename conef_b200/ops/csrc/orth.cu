// Row-parallel orthogonalisation and small-factor corrections for tall-skinny blocks.
//
// The reference orthogonalises every P and Q with a Python Gram-Schmidt loop, ~6 tiny kernels
// per column per matrix (communication/powerSGD_hook.py:12-43).  A tall block (30,528 x 8 for
// BERT's embedding) must not be walked by one CTA, so Gram-Schmidt is done through the Gram
// matrix, which needs only row-parallel passes:
//   k_gram      : G = A^T A, one CTA per (matrix, chunk of rows), partial sums by atomics.
//                 With world > 1 the chunk first sums the peers' copies of its rows
//                 (all-reduce over NVLink peer loads fused into the pass, bounded flag wait).
//   k_qr_apply  : every CTA factors G = R^T R (r <= 32: a warp does it in shared memory),
//                 inverts R and writes A R^-1 for its rows.  A R^-1 is exactly what column-by-
//                 column Gram-Schmidt produces in exact arithmetic (the QR factorisation with a
//                 positive diagonal is unique).  The pass also accumulates the Gram matrix of its
//                 output, and a second k_qr_apply re-orthogonalises with it ("twice is enough"),
//                 which restores orthogonality to rounding level for conditioned inputs.
//                 A numerically dependent column comes out as zero instead of normalised noise.
// The same two-pass structure serves the corrections of the low-rank error store:
//   k_corr_reduce : C_t = L_t^T Rm_t   (up to two terms per matrix)
//   k_corr_apply  : T += sum_t coef_t X_t C_t
#include "common.cuh"

constexpr int OC_ROWS = 512;     // rows per CTA
constexpr int OC_THREADS = 256;
constexpr int OC_MAXR = 32;
constexpr int GRAM_STRIDE = OC_MAXR * OC_MAXR;

// Csm[c2 x c1] = L[rows x c2]^T Rm[rows x c1] over `rows` rows; all threads of the CTA take part.
// The summation order is fixed (no atomics): every rank must obtain bit-identical factors from
// bit-identical inputs, otherwise the replicas drift apart.  `scratch` holds OC_THREADS floats.
__device__ __forceinline__ void pair_reduce(const float* __restrict__ L, const float* __restrict__ Rm, int rows,
                                            int c2, int c1, float* Csm, float* scratch) {
  const int pairs = c1 * c2;
  if (pairs <= OC_THREADS) {
    const int groups = OC_THREADS / pairs;
    const int g = threadIdx.x / pairs, pr = threadIdx.x - g * pairs;
    if (g < groups) {
      const int a = pr / c1, b = pr - a * c1;
      float acc = 0.f;
      for (int i = g; i < rows; i += groups) acc = fmaf(L[(size_t)i * c2 + a], Rm[(size_t)i * c1 + b], acc);
      scratch[g * pairs + pr] = acc;
    }
    __syncthreads();
    if (threadIdx.x < pairs) {
      float acc = 0.f;
      for (int gg = 0; gg < groups; ++gg) acc += scratch[gg * pairs + threadIdx.x];
      Csm[threadIdx.x] = acc;
    }
  } else {
    for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
      const int a = pr / c1, b = pr - a * c1;
      float acc = 0.f;
      for (int i = 0; i < rows; ++i) acc = fmaf(L[(size_t)i * c2 + a], Rm[(size_t)i * c1 + b], acc);
      Csm[pr] = acc;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(OC_THREADS)
k_gram(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, int which, float* __restrict__ buf,
       float* __restrict__ gram, const float* const* __restrict__ peer_bufs, const uint32_t* __restrict__ flags,
       int world, uint32_t epoch, int* __restrict__ status, long long spin_limit,
       const uint32_t* __restrict__ epoch_base) {
  __shared__ float Csm[GRAM_STRIDE];
  __shared__ float scratch[OC_THREADS];
  __shared__ int ok;
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int rows_total = which == 0 ? M.n : M.m, r = M.r;
  const size_t off = (which == 0 ? M.p_off : M.q_off) + (size_t)t.y * OC_ROWS * r;
  const int rows = min(OC_ROWS, rows_total - t.y * OC_ROWS);
  float* a = buf + off;
  if (world > 1) {
    if (threadIdx.x == 0) {
      if (epoch_base != nullptr) epoch += *epoch_base;
      ok = wait_flags_bounded(flags, world, epoch, spin_limit) ? 1 : 0;
      if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    if (!ok) return;      // leave local values untouched; the host raises
    for (int i = threadIdx.x; i < rows * r; i += OC_THREADS) {
      float s = 0.f;
      for (int p = 0; p < world; ++p) s += ld_relaxed_sys_f32(peer_bufs[p] + off + i);
      a[i] = s;
    }
  }
  __syncthreads();
  pair_reduce(a, a, rows, r, r, Csm, scratch);
  float* g = gram + (size_t)blockIdx.x * GRAM_STRIDE;      // one partial per tile, summed in order by k_qr_apply
  for (int i = threadIdx.x; i < r * r; i += OC_THREADS) g[i] = Csm[i];
}

__global__ void __launch_bounds__(OC_THREADS)
k_qr_apply(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, int which, float* __restrict__ buf,
           const float* __restrict__ gram_in, float* __restrict__ gram_out, float eps, float* __restrict__ packed,
           int packed_np) {
  __shared__ float G[OC_MAXR][OC_MAXR + 1];
  __shared__ float R[OC_MAXR][OC_MAXR + 1];
  __shared__ float Ri[OC_MAXR][OC_MAXR + 1];
  __shared__ float Csm[GRAM_STRIDE];
  __shared__ float scratch[OC_THREADS];
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int rows_total = which == 0 ? M.n : M.m, r = M.r;
  const size_t off = (which == 0 ? M.p_off : M.q_off) + (size_t)t.y * OC_ROWS * r;
  const int rows = min(OC_ROWS, rows_total - t.y * OC_ROWS);
  float* a = buf + off;
  // the tiles of one matrix are consecutive: sum their Gram partials in tile order
  const int first = blockIdx.x - t.y, count = (rows_total + OC_ROWS - 1) / OC_ROWS;
  for (int i = threadIdx.x; i < r * r; i += OC_THREADS) {
    float acc = 0.f;
    for (int c = 0; c < count; ++c) acc += gram_in[(size_t)(first + c) * GRAM_STRIDE + i];
    G[i / r][i % r] = acc;
    R[i / r][i % r] = 0.f;
    Ri[i / r][i % r] = 0.f;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    // Cholesky G = R^T R, row j of R at a time; lanes own the columns i >= j
    for (int j = 0; j < r; ++j) {
      float d = G[j][j];
      for (int k = 0; k < j; ++k) d -= R[k][j] * R[k][j];
      const bool dead = !(d > 1e-10f * G[j][j]) || !(G[j][j] > 0.f);   // dependent (or empty) column
      const float rjj = dead ? 0.f : sqrtf(d);
      if (lane == j) R[j][j] = rjj;
      if (lane > j && lane < r) {
        float v = G[j][lane];
        for (int k = 0; k < j; ++k) v -= R[k][j] * R[k][lane];
        R[j][lane] = dead ? 0.f : v / rjj;
      }
      __syncwarp();
    }
    // inverse of the upper-triangular R (diagonal + eps), lane c owns column c; dead columns stay zero
    if (lane < r && R[lane][lane] > 0.f) {
      const int c = lane;
      for (int i = c; i >= 0; --i) {
        if (!(R[i][i] > 0.f)) { Ri[i][c] = 0.f; continue; }
        float v = (i == c) ? 1.f : 0.f;
        for (int k = i + 1; k <= c; ++k) v -= R[i][k] * Ri[k][c];
        Ri[i][c] = v / (R[i][i] + eps);
      }
    }
  }
  __syncthreads();
  float* pk = packed ? packed + (which == 0 ? M.ppk_off : M.qpk_off) : nullptr;
  const long long grow0 = (long long)t.y * OC_ROWS;
  for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
    float av[OC_MAXR];
    float* rowp = a + (size_t)i * r;
#pragma unroll
    for (int k = 0; k < OC_MAXR; ++k) av[k] = k < r ? rowp[k] : 0.f;
#pragma unroll
    for (int c = 0; c < OC_MAXR; ++c) {
      if (c < r) {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < OC_MAXR; ++k)
          if (k <= c) v = fmaf(av[k], Ri[k][c], v);
        rowp[c] = v;
        if (pk) pk[conef_packed_offset(grow0 + i, c, packed_np)] = v;
      }
    }
  }
  if (gram_out != nullptr) {
    __syncthreads();
    pair_reduce(a, a, rows, r, r, Csm, scratch);
    float* go = gram_out + (size_t)blockIdx.x * GRAM_STRIDE;
    for (int i = threadIdx.x; i < r * r; i += OC_THREADS) go[i] = Csm[i];
  }
}

// gram: scratch of 2 * ntiles * 1024 floats (one Gram partial per tile and round).
extern "C" int conef_orthogonalize_packed_ex(const ConefMat* mats, const int2* tiles, int ntiles, int nrecords,
                                             int which, float* buf, float eps, const float* const* peer_bufs,
                                             const uint32_t* flags, int world, uint32_t epoch, int* status,
                                             long long spin_limit, float* packed, int packed_np, float* gram,
                                             const uint32_t* epoch_base, cudaStream_t stream) {
  if (ntiles <= 0) return 0;
  (void)nrecords;
  float* gram2 = gram + (size_t)ntiles * GRAM_STRIDE;
  k_gram<<<ntiles, OC_THREADS, 0, stream>>>(mats, tiles, which, buf, gram, peer_bufs, flags, world, epoch, status,
                                           spin_limit, epoch_base);
  CONEF_CHECK_LAUNCH("k_gram");
  k_qr_apply<<<ntiles, OC_THREADS, 0, stream>>>(mats, tiles, which, buf, gram, gram2, eps, nullptr, 0);
  CONEF_CHECK_LAUNCH("k_qr_apply");
  k_qr_apply<<<ntiles, OC_THREADS, 0, stream>>>(mats, tiles, which, buf, gram2, nullptr, 0.f, packed, packed_np);
  CONEF_CHECK_LAUNCH("k_qr_apply");
  return 0;
}

extern "C" int conef_orthogonalize_packed(const ConefMat* mats, const int2* tiles, int ntiles, int nrecords,
                                          int which, float* buf, float eps, const float* const* peer_bufs,
                                          const uint32_t* flags, int world, uint32_t epoch, int* status,
                                          long long spin_limit, float* packed, int packed_np, float* gram,
                                          cudaStream_t stream) {
  return conef_orthogonalize_packed_ex(mats, tiles, ntiles, nrecords, which, buf, eps, peer_bufs, flags, world,
                                       epoch, status, spin_limit, packed, packed_np, gram, nullptr, stream);
}

// ---------------------------------------------------------------------------
// Corrections of the low-rank error store.
__global__ void __launch_bounds__(OC_THREADS)
k_corr_reduce(const ConefCorr* __restrict__ table, const int2* __restrict__ tiles, const float* __restrict__ L0b,
              const float* __restrict__ R0b, const float* __restrict__ L1b, const float* __restrict__ R1b,
              float* __restrict__ cbuf) {
  __shared__ float Csm[GRAM_STRIDE];
  __shared__ float scratch[OC_THREADS];
  const int2 t = tiles[blockIdx.x];
  const ConefCorr K = table[t.x];
  const int row0 = t.y * OC_ROWS;
  const int rows = min(OC_ROWS, K.rows_l - row0);
  for (int term = 0; term < K.nterms; ++term) {
    const int c2 = K.c2[term], c1 = K.c1;
    const float* L = (term ? L1b : L0b) + K.l_off[term] + (size_t)row0 * c2;
    const float* Rm = (term ? R1b : R0b) + K.r_off[term] + (size_t)row0 * c1;
    __syncthreads();
    pair_reduce(L, Rm, rows, c2, c1, Csm, scratch);
    float* c = cbuf + ((size_t)t.x * 2 + term) * GRAM_STRIDE;
    for (int i = threadIdx.x; i < c1 * c2; i += OC_THREADS) atomicAdd(c + i, Csm[i]);
  }
}

__global__ void __launch_bounds__(OC_THREADS)
k_corr_apply(const ConefCorr* __restrict__ table, const int2* __restrict__ tiles, float* __restrict__ Tb,
             const float* __restrict__ X0b, const float* __restrict__ X1b, const float* __restrict__ cbuf,
             float coef0, float coef1) {
  __shared__ float Csm[2][GRAM_STRIDE];
  const int2 t = tiles[blockIdx.x];
  const ConefCorr K = table[t.x];
  const int c1 = K.c1;
  for (int term = 0; term < K.nterms; ++term) {
    const float* c = cbuf + ((size_t)t.x * 2 + term) * GRAM_STRIDE;
    for (int i = threadIdx.x; i < c1 * K.c2[term]; i += OC_THREADS) Csm[term][i] = c[i];
  }
  __syncthreads();
  const int row0 = t.y * OC_ROWS;
  const int rows = min(OC_ROWS, K.rows_t - row0);
  float* T = Tb + K.t_off + (size_t)row0 * c1;
  for (int e = threadIdx.x; e < rows * c1; e += OC_THREADS) {
    const int i = e / c1, b = e - i * c1;
    float add = 0.f;
    for (int term = 0; term < K.nterms; ++term) {
      const int c2 = K.c2[term];
      const float* X = (term ? X1b : X0b) + K.x_off[term] + (size_t)(row0 + i) * c2;
      float acc = 0.f;
      for (int a = 0; a < c2; ++a) acc = fmaf(X[a], Csm[term][a * c1 + b], acc);
      add += (term ? coef1 : coef0) * acc;
    }
    T[e] += add;
  }
}

// cbuf: scratch of nmats * 2 * 1024 floats.  reduce_tiles chunk rows_l, apply_tiles chunk rows_t.
extern "C" int conef_lowrank_correct(const ConefCorr* table, int nmats, const int2* reduce_tiles, int n_reduce,
                                     const int2* apply_tiles, int n_apply, float* T, const float* X0,
                                     const float* L0, const float* R0, float coef0, const float* X1,
                                     const float* L1, const float* R1, float coef1, float* cbuf,
                                     cudaStream_t stream) {
  if (nmats <= 0 || n_reduce <= 0 || n_apply <= 0) return 0;
  CONEF_CUDA(cudaMemsetAsync(cbuf, 0, sizeof(float) * (size_t)nmats * 2 * GRAM_STRIDE, stream));
  k_corr_reduce<<<n_reduce, OC_THREADS, 0, stream>>>(table, reduce_tiles, L0, R0, L1, R1, cbuf);
  CONEF_CHECK_LAUNCH("k_corr_reduce");
  k_corr_apply<<<n_apply, OC_THREADS, 0, stream>>>(table, apply_tiles, T, X0, X1, cbuf, coef0, coef1);
  CONEF_CHECK_LAUNCH("k_corr_apply");
  return 0;
}
