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
//                 which restores orthogonality to rounding level.  The Gram matrix squares the
//                 condition number, so a pivot that comes out below ORTH_SHIFT times its column's
//                 squared norm cannot be told from rounding noise in fp32; such a pivot is raised to
//                 that floor (a shifted Cholesky factor).  The column then leaves the first pass
//                 short and almost orthogonal, and the second pass, whose Gram matrix is well
//                 conditioned, finishes it: columns with a relative residual down to 1e-6 come out
//                 orthonormal to 1e-6, where the column-by-column loop in fp32 loses orthogonality.
//                 Only a column that is exactly zero has no direction to keep; the last pass fills
//                 it with fixed pseudo-random values of unit expected norm (the same on every rank),
//                 so that under warm start a rank of the factorisation is never lost for good.
// The same two-pass structure serves the corrections of the low-rank error store:
//   k_corr_reduce : C_t = L_t^T Rm_t   (up to two terms per matrix)
//   k_corr_apply  : T += sum_t coef_t X_t C_t
#include <string.h>
#include "common.cuh"

constexpr int OC_ROWS = 512;     // rows per CTA
constexpr int OC_THREADS = 256;
constexpr int OC_MAXR = 32;
constexpr int GRAM_STRIDE = OC_MAXR * OC_MAXR;
constexpr float ORTH_SHIFT = 1e-5f;          // pivot floor of the first pass, relative to the column's squared norm
constexpr float ORTH_SHIFT_FINAL = 1e-7f;    // and of the last pass, whose input is nearly orthonormal
constexpr unsigned long long ORTH_REFILL_SEED = 0x5EEDC01DF00DULL;

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

// Segment index whose dst_off is the largest one <= pos.
__device__ __forceinline__ int orth_find_seg(const ConefSeg* segs, int n, long long pos) {
  int lo = 0, hi = n - 1;
  while (lo < hi) {
    const int mid = (lo + hi + 1) >> 1;
    if (segs[mid].dst_off <= pos) lo = mid; else hi = mid - 1;
  }
  return lo;
}

// CTAs [0, ntiles): one (matrix, 512-row chunk) each.  CTAs [ntiles, gridDim.x): the uncompressed
// tensors of the bucket (X.seg_mode).  All CTAs share the clearing of X.zero0 / X.zero1.
__global__ void __launch_bounds__(OC_THREADS)
k_gram(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, int ntiles, int which,
       float* __restrict__ buf, float* __restrict__ gram, const float* const* __restrict__ peer_bufs,
       const uint32_t* __restrict__ flags, int world, uint32_t epoch, int* __restrict__ status, long long spin_limit,
       const uint32_t* __restrict__ epoch_base, const ConefOrthExtra X) {
  __shared__ float Csm[GRAM_STRIDE];
  __shared__ float scratch[OC_THREADS];
  __shared__ int ok;
  if (world > 1) {
    if (threadIdx.x == 0) {
      if (epoch_base != nullptr) epoch += *epoch_base;
      ok = wait_flags_bounded(flags, world, epoch, spin_limit) ? 1 : 0;
      if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    if (!ok) return;      // leave local values untouched; the host raises
  }
  {
    const long long stride = (long long)gridDim.x * OC_THREADS;
    const long long first = (long long)blockIdx.x * OC_THREADS + threadIdx.x;
    for (long long i = first; i < X.zero0_n; i += stride) X.zero0[i] = 0.f;
    for (long long i = first; i < X.zero1_n; i += stride) X.zero1[i] = 0.f;
  }
  if ((int)blockIdx.x >= ntiles) {
    const long long stride = (long long)(gridDim.x - ntiles) * OC_THREADS;
    for (long long e = (long long)(blockIdx.x - ntiles) * OC_THREADS + threadIdx.x; e < X.seg_total; e += stride) {
      const int s = orth_find_seg(X.segs, X.nsegs, e);
      const long long src = X.segs[s].src_off + (e - X.segs[s].dst_off);
      if (X.seg_mode == 1) {
        float v = X.bucket[src];
        if (X.dense_err) { v += X.dense_err[src]; X.dense_err[src] = v; }   // the error slot keeps the local value
        X.staging[e] = v;
      } else {
        float v = 0.f;
        for (int p = 0; p < world; ++p) v += ld_relaxed_sys_f32(X.peer_staging[p] + e);
        v *= X.seg_scale;
        X.bucket[src] = v;
        if (X.dense_err) X.dense_err[src] -= v;     // local value (stored by the gather) minus the average
      }
    }
    return;
  }
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int rows_total = which == 0 ? M.n : M.m, r = M.r;
  const size_t off = (which == 0 ? M.p_off : M.q_off) + (size_t)t.y * OC_ROWS * r;
  const int rows = min(OC_ROWS, rows_total - t.y * OC_ROWS);
  float* a = buf + off;
  if (peer_bufs != nullptr) {
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
           const float* __restrict__ gram_in, float* __restrict__ gram_out, float eps, float shift,
           float* __restrict__ packed, int packed_np, const int32_t* __restrict__ proj_tables, int proj_nm,
           float proj_alpha) {
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
      const bool dead = !(G[j][j] > 0.f);                 // an all-zero (or non-finite) column
      const float floor_d = shift * G[j][j];
      if (!(d > floor_d)) d = floor_d;                    // numerically dependent: shifted pivot
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
  // last pass only: zero columns are refilled (see the header); value of (matrix, row, column)
  const bool refill = gram_out == nullptr;
  const float refill_scale = rsqrtf((float)rows_total);
  // projection onto the sketch cells (last pass of Q): Z[h_j, :] += alpha s_j Q[j, :], packed layout
  const bool project = proj_tables != nullptr && refill && which == 1 && pk != nullptr && M.tab_off >= 0;
  const int32_t* tab = project ? proj_tables + M.tab_off : nullptr;
  float* zpk = project ? packed + mats[proj_nm + t.x].qpk_off : nullptr;
  for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
    float av[OC_MAXR];
    float* rowp = a + (size_t)i * r;
#pragma unroll
    for (int k = 0; k < OC_MAXR; ++k) av[k] = k < r ? rowp[k] : 0.f;
    float psc = 0.f;
    long long ph = 0;
    if (project) {
      const int e = tab[grow0 + i];
      psc = unpack_sign(e) * proj_alpha;
      ph = unpack_bucket(e);
    }
#pragma unroll
    for (int c = 0; c < OC_MAXR; ++c) {
      if (c < r) {
        float v = 0.f;
#pragma unroll
        for (int k = 0; k < OC_MAXR; ++k)
          if (k <= c) v = fmaf(av[k], Ri[k][c], v);
        rowp[c] = v;
        if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
        if (project) atomicAdd(zpk + conef_packed_offset(ph, c, packed_np), psc * v);
      }
    }
  }
  if (refill) {       // columns that were exactly zero (rare; not unrolled)
#pragma unroll 1
    for (int c = 0; c < r; ++c) {
      if (R[c][c] > 0.f) continue;
      for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
        float z[4];
        conef_philox_normal4(ORTH_REFILL_SEED + (unsigned long long)t.x * 64ull + (unsigned long long)which * 32ull + c,
                             (uint64_t)(grow0 + i), z);
        const float v = z[0] * refill_scale;
        a[(size_t)i * r + c] = v;
        if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
        if (project) {
          const int e = tab[grow0 + i];
          atomicAdd(zpk + conef_packed_offset(unpack_bucket(e), c, packed_np), unpack_sign(e) * proj_alpha * v);
        }
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

// ---------------------------------------------------------------------------
// The whole orthogonalisation in ONE launch: Gram partial -> barrier -> factor, apply, Gram partial of
// the result -> barrier -> factor, apply, write.  The rows of a chunk stay in shared memory between
// the rounds, so they are read from global memory once and written once, and the two launch
// boundaries of the three-kernel form become two barriers among the CTAs of the launch.  Those
// barriers need every tile CTA resident at once: the host checks the grid against the device's
// capacity for this kernel and otherwise uses the three-kernel form.  Every wait is bounded.
//
// Sense-reversing barrier over two device words {arrivals, generation}; usable launch after launch
// without a reset.  Returns false when the wait ran out.
__device__ __forceinline__ bool cta_group_barrier(uint32_t* bar, unsigned expected, long long limit) {
  __shared__ int bar_ok;
  __syncthreads();
  if (threadIdx.x == 0) {
    bar_ok = 1;
    const uint32_t gen = ld_acquire_gpu(bar + 1);
    __threadfence();                                   // this CTA's partials, then the arrival
    if (atomicAdd(bar, 1u) == expected - 1) {
      atomicExch(bar, 0u);
      __threadfence();
      atomicAdd(bar + 1, 1u);                          // releases the others
    } else {
      long long n = 0;
      while (ld_acquire_gpu(bar + 1) == gen) {
        if (++n > limit) { bar_ok = 0; break; }
        if (n > 64) __nanosleep(20);                   // the others are usually a microsecond away
      }
    }
    __threadfence();
  }
  __syncthreads();
  return bar_ok != 0;
}

constexpr long long ORTH_BARRIER_LIMIT = 2LL * 1000 * 1000;

// Shifted Cholesky factor R of G (r x r, row stride RP + 1) by the first warp; see the file header.  R must
// be zero on entry.  rd[c] = 1 / (R[c][c] + eps), or 0 for a column without a direction.  The rows are then
// multiplied by (R + eps I)^-1 through a forward substitution per row (apply_factor), which needs no explicit
// inverse: this serial section runs on one warp while the SM's other warps compete for issue slots, so its
// cost is its instruction count (measured 3.5 us at r = 4 and 6 us at r = 8 with the inverse, per call).
template <int RP>
__device__ __forceinline__ void chol_factor(const float (*G)[RP + 1], float (*R)[RP + 1], float* rd, int r,
                                            float shift, float eps) {
  const int lane = threadIdx.x;
  for (int j = 0; j < r; ++j) {
    float d = G[j][j];
    for (int k = 0; k < j; ++k) d -= R[k][j] * R[k][j];
    const bool dead = !(G[j][j] > 0.f);
    const float floor_d = shift * G[j][j];
    if (!(d > floor_d)) d = floor_d;
    const float rjj = dead ? 0.f : sqrtf(d);
    if (lane == j) { R[j][j] = rjj; rd[j] = dead ? 0.f : 1.f / (rjj + eps); }
    if (lane > j && lane < r) {
      float v = G[j][lane];
      for (int k = 0; k < j; ++k) v -= R[k][j] * R[k][lane];
      R[j][lane] = dead ? 0.f : v / rjj;
    }
    __syncwarp();
  }
}

// y = x (R + eps I)^-1 for one row: y[c] = (x[c] - sum_{k<c} y[k] R[k][c]) rd[c]; a column without a direction
// gives y[c] = 0 and so drops out of the later columns.
template <int RP>
__device__ __forceinline__ void apply_factor(const float (&x)[RP], const float (*R)[RP + 1], const float* rd, int r,
                                             float (&y)[RP]) {
#pragma unroll
  for (int c = 0; c < RP; ++c) {
    y[c] = 0.f;
    if (c < r) {
      float v = x[c];
#pragma unroll
      for (int k = 0; k < c; ++k) v = fmaf(-y[k], R[k][c], v);
      y[c] = v * rd[c];
    }
  }
}

template <int RP>
__global__ void __launch_bounds__(OC_THREADS, RP <= 16 ? 2 : 1)
k_orth_one(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, int ntiles, int which,
           float* __restrict__ buf, float* __restrict__ gram, const float* const* __restrict__ peer_bufs,
           const uint32_t* __restrict__ flags, int world, uint32_t epoch, int* __restrict__ status, long long spin_limit,
           const uint32_t* __restrict__ epoch_base, float eps, float* __restrict__ packed, int packed_np,
           uint32_t* __restrict__ bar, const ConefOrthExtra X) {
  extern __shared__ float xs[];                    // OC_ROWS x (RP + 1): the chunk's rows
  constexpr int S = RP + 1;
  __shared__ float G[RP][RP + 1], R[RP][RP + 1], rd[RP];
  __shared__ float part[OC_THREADS / 32][RP * RP < 32 ? 32 : RP * RP > 256 ? 256 : RP * RP];
  __shared__ int ok;
  bool peers_ok = true;
  if (world > 1) {
    if (threadIdx.x == 0) {
      if (epoch_base != nullptr) epoch += *epoch_base;
      ok = wait_flags_bounded(flags, world, epoch, spin_limit) ? 1 : 0;
      if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    peers_ok = ok != 0;     // on a timeout the CTA still takes part in the barriers, on zeros
  }
  if (peers_ok) {
    const long long stride = (long long)gridDim.x * OC_THREADS;
    const long long first = (long long)blockIdx.x * OC_THREADS + threadIdx.x;
    for (long long i = first; i < X.zero0_n; i += stride) X.zero0[i] = 0.f;
    for (long long i = first; i < X.zero1_n; i += stride) X.zero1[i] = 0.f;
  }
  if ((int)blockIdx.x >= ntiles) {                 // spare CTAs: the uncompressed tensors; no barriers
    if (!peers_ok) return;
    const long long stride = (long long)(gridDim.x - ntiles) * OC_THREADS;
    for (long long e = (long long)(blockIdx.x - ntiles) * OC_THREADS + threadIdx.x; e < X.seg_total; e += stride) {
      const int s = orth_find_seg(X.segs, X.nsegs, e);
      const long long src = X.segs[s].src_off + (e - X.segs[s].dst_off);
      if (X.seg_mode == 1) {
        float v = X.bucket[src];
        if (X.dense_err) { v += X.dense_err[src]; X.dense_err[src] = v; }
        X.staging[e] = v;
      } else {
        float v = 0.f;
        for (int p = 0; p < world; ++p) v += ld_relaxed_sys_f32(X.peer_staging[p] + e);
        v *= X.seg_scale;
        X.bucket[src] = v;
        if (X.dense_err) X.dense_err[src] -= v;
      }
    }
    return;
  }
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const int rows_total = which == 0 ? M.n : M.m, r = M.r;
  const size_t off = (which == 0 ? M.p_off : M.q_off) + (size_t)t.y * OC_ROWS * r;
  const int rows = min(OC_ROWS, rows_total - t.y * OC_ROWS);
  float* a = buf + off;
  // ---- load the chunk (summing the peers' copies), four loads per thread (times the peers) in flight ----
  const int nel = rows * r;
  const bool vec4 = peer_bufs == nullptr && (r & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  if (vec4) {      // 16-byte loads of this GPU's own rows: an element group never straddles a row
    for (int q0 = 0; q0 < (nel >> 2); q0 += 4 * OC_THREADS) {
      float4 v4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u * OC_THREADS + threadIdx.x;
        if (q < (nel >> 2)) v4[u] = __ldcg(reinterpret_cast<const float4*>(a) + q);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u * OC_THREADS + threadIdx.x;
        if (q < (nel >> 2)) {
          const int i = q << 2, row = i / r;
          float* x = xs + row * S + (i - row * r);
          x[0] = v4[u].x; x[1] = v4[u].y; x[2] = v4[u].z; x[3] = v4[u].w;
        }
      }
    }
  }
  for (int base = vec4 ? nel : 0; base < nel; base += 4 * OC_THREADS) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * OC_THREADS + threadIdx.x;
      v[u] = 0.f;
      if (i < nel) {
        if (peer_bufs != nullptr) {
          if (peers_ok) for (int p = 0; p < world; ++p) v[u] += ld_relaxed_sys_f32(peer_bufs[p] + off + i);
        } else {
          v[u] = a[i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * OC_THREADS + threadIdx.x;
      if (i < nel) {
        const int row = i / r;
        xs[row * S + (i - row * r)] = v[u];
      }
    }
  }
  const int first = blockIdx.x - t.y, count = (rows_total + OC_ROWS - 1) / OC_ROWS;
  const int pairs = r * r;
  float* pk = packed ? packed + (which == 0 ? M.ppk_off : M.qpk_off) : nullptr;
  const long long grow0 = (long long)t.y * OC_ROWS;
  const bool project = X.tables != nullptr && which == 1 && pk != nullptr && M.tab_off >= 0;
  const int32_t* tab = project ? X.tables + M.tab_off : nullptr;
  float* zpk = project ? packed + mats[X.nm + t.x].qpk_off : nullptr;
  const float refill_scale = rsqrtf((float)rows_total);

#pragma unroll 1
  for (int round = 0; round < 2; ++round) {
    __syncthreads();
    // ---- Gram partial of the chunk, fixed summation order: warps over row slices, then warps 0..7 in order ----
    {
      float* g = gram + ((size_t)round * ntiles + blockIdx.x) * GRAM_STRIDE;
      if (pairs <= 256) {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        const int per = (rows + (OC_THREADS / 32) - 1) / (OC_THREADS / 32);
        const int i0 = warp * per, i1 = min(rows, i0 + per);
        for (int pr = lane; pr < pairs; pr += 32) {
          const int ca = pr / r, cb = pr - ca * r;
          float acc = 0.f;
          for (int i = i0; i < i1; ++i) acc = fmaf(xs[i * S + ca], xs[i * S + cb], acc);
          part[warp][pr] = acc;
        }
        __syncthreads();
        if ((int)threadIdx.x < pairs) {
          float acc = 0.f;
#pragma unroll
          for (int w = 0; w < OC_THREADS / 32; ++w) acc += part[w][threadIdx.x];
          g[threadIdx.x] = acc;
        }
      } else {
        for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
          const int ca = pr / r, cb = pr - ca * r;
          float acc = 0.f;
          for (int i = 0; i < rows; ++i) acc = fmaf(xs[i * S + ca], xs[i * S + cb], acc);
          g[pr] = acc;
        }
      }
    }
    if (!cta_group_barrier(bar, (unsigned)ntiles, ORTH_BARRIER_LIMIT) && threadIdx.x == 0)
      atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    // ---- the matrix's Gram matrix: partials in tile order; factor; inverse ----
    for (int i = threadIdx.x; i < RP * (RP + 1); i += OC_THREADS) (&R[0][0])[i] = 0.f;
    for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
      const float* g = gram + ((size_t)round * ntiles + first) * GRAM_STRIDE + pr;
      float acc = 0.f;
      int c = 0;
      for (; c + 8 <= count; c += 8) {          // eight loads in flight; the order of the additions is fixed
        float gv[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) gv[u] = __ldcg(g + (size_t)(c + u) * GRAM_STRIDE);
#pragma unroll
        for (int u = 0; u < 8; ++u) acc += gv[u];
      }
      for (; c < count; ++c) acc += __ldcg(g + (size_t)c * GRAM_STRIDE);
      G[pr / r][pr % r] = acc;
    }
    __syncthreads();
    if (threadIdx.x < 32) chol_factor<RP>(G, R, rd, r, round == 0 ? ORTH_SHIFT : ORTH_SHIFT_FINAL, round == 0 ? eps : 0.f);
    __syncthreads();
    // ---- apply: every thread its rows ----
    for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
      float av[RP];
#pragma unroll
      for (int k = 0; k < RP; ++k) av[k] = xs[i * S + k];
      float psc = 0.f;
      long long ph = 0;
      if (round == 1 && project) {
        const int e = tab[grow0 + i];
        psc = unpack_sign(e) * X.alpha;
        ph = unpack_bucket(e);
      }
      float yv[RP];
      apply_factor<RP>(av, R, rd, r, yv);
#pragma unroll
      for (int c = 0; c < RP; ++c) {
        if (c < r) {
          const float v = yv[c];
          if (round == 0) {
            xs[i * S + c] = v;
          } else {
            a[(size_t)i * r + c] = v;
            if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
            if (project) atomicAdd(zpk + conef_packed_offset(ph, c, packed_np), psc * v);
          }
        }
      }
    }
  }
  // ---- columns that were exactly zero: fixed pseudo-random values instead (rare; not unrolled) ----
#pragma unroll 1
  for (int c = 0; c < r; ++c) {
    if (R[c][c] > 0.f) continue;
    for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
      float z[4];
      conef_philox_normal4(ORTH_REFILL_SEED + (unsigned long long)t.x * 64ull + (unsigned long long)which * 32ull + c,
                           (uint64_t)(grow0 + i), z);
      const float v = z[0] * refill_scale;
      a[(size_t)i * r + c] = v;
      if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
      if (project) {
        const int e = tab[grow0 + i];
        atomicAdd(zpk + conef_packed_offset(unpack_bucket(e), c, packed_np), unpack_sign(e) * X.alpha * v);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// The same orthogonalisation with one thread-block cluster per block of rows to orthogonalise: the
// OCL CTAs of a cluster split the block's rows evenly, keep their rows in shared memory for the whole
// kernel, exchange their Gram partials through distributed shared memory and meet at the cluster's
// hardware barrier.  Against k_orth_one (one barrier over ALL CTAs of the launch through two words in
// global memory, partials through L2) a round costs a cluster barrier and eight remote shared-memory
// reads per Gram entry.  Every CTA sums the partials in rank order, so all CTAs (and all GPUs) hold the
// same bits.  `list[c].x` is the record of cluster c.
constexpr int OCL = 8;      // CTAs per cluster (the portable maximum)
constexpr int OCL_MAX_ROWS = 1024;

__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ float ld_dsmem_f32(const float* local_smem, uint32_t rank) {
  const uint32_t la = (uint32_t)__cvta_generic_to_shared(local_smem);
  uint32_t ra;
  float v;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(ra) : "r"(la), "r"(rank));
  asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(ra) : "memory");
  return v;
}

template <int RP>
__global__ void __launch_bounds__(OC_THREADS)
k_orth_cluster(const ConefMat* __restrict__ mats, const int2* __restrict__ list, int nmat, int which,
               float* __restrict__ buf, const float* const* __restrict__ peer_bufs,
               const uint32_t* __restrict__ flags, int world, uint32_t epoch, int* __restrict__ status,
               long long spin_limit, const uint32_t* __restrict__ epoch_base, float eps, float* __restrict__ packed,
               int packed_np, const ConefOrthExtra X) {
  extern __shared__ float xs[];                    // this CTA's rows, row stride RP + 1
  constexpr int S = RP + 1;
  constexpr int PAIRS_MAX = RP * RP;
  __shared__ float G[RP][RP + 1], R[RP][RP + 1], rd[RP];
  __shared__ float part[OC_THREADS / 32][PAIRS_MAX < 32 ? 32 : PAIRS_MAX > 256 ? 256 : PAIRS_MAX];
  __shared__ float gpart[2][PAIRS_MAX];            // this CTA's Gram partial of each round, read by the cluster
  __shared__ int ok;
  bool peers_ok = true;
  if (world > 1) {
    if (threadIdx.x == 0) {
      if (epoch_base != nullptr) epoch += *epoch_base;
      ok = wait_flags_bounded(flags, world, epoch, spin_limit) ? 1 : 0;
      if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    peers_ok = ok != 0;     // on a timeout the CTA still takes part in the barriers, on zeros
  }
  if (peers_ok) {
    const long long stride = (long long)gridDim.x * OC_THREADS;
    const long long first = (long long)blockIdx.x * OC_THREADS + threadIdx.x;
    for (long long i = first; i < X.zero0_n; i += stride) X.zero0[i] = 0.f;
    for (long long i = first; i < X.zero1_n; i += stride) X.zero1[i] = 0.f;
  }
  const int tile_ctas = nmat * OCL;
  if ((int)blockIdx.x >= tile_ctas) {              // spare clusters: the uncompressed tensors; no barriers
    if (!peers_ok) return;
    const long long stride = (long long)(gridDim.x - tile_ctas) * OC_THREADS;
    for (long long e = (long long)(blockIdx.x - tile_ctas) * OC_THREADS + threadIdx.x; e < X.seg_total; e += stride) {
      const int s = orth_find_seg(X.segs, X.nsegs, e);
      const long long src = X.segs[s].src_off + (e - X.segs[s].dst_off);
      if (X.seg_mode == 1) {
        float v = X.bucket[src];
        if (X.dense_err) { v += X.dense_err[src]; X.dense_err[src] = v; }
        X.staging[e] = v;
      } else {
        float v = 0.f;
        for (int p = 0; p < world; ++p) v += ld_relaxed_sys_f32(X.peer_staging[p] + e);
        v *= X.seg_scale;
        X.bucket[src] = v;
        if (X.dense_err) X.dense_err[src] -= v;
      }
    }
    return;
  }
  const int rec = list[blockIdx.x / OCL].x;
  const uint32_t rank = cluster_rank();
  const ConefMat M = mats[rec];
  const int rows_total = which == 0 ? M.n : M.m, r = M.r;
  const int rows_per = (rows_total + OCL - 1) / OCL;
  const long long grow0 = (long long)rank * rows_per;
  const int rows = max(0, min(rows_per, rows_total - (int)grow0));
  const size_t off = (which == 0 ? M.p_off : M.q_off) + (size_t)grow0 * r;
  float* a = buf + off;
  // ---- load this CTA's rows (summing the peers' copies), four loads per thread (times the peers) in flight:
  //      one at a time, the 11 KB of a 720 x 4 block took 7 us ----
  const int nel = rows * r;
  const bool vec4 = peer_bufs == nullptr && (r & 3) == 0 && (reinterpret_cast<uintptr_t>(a) & 15) == 0;
  if (vec4) {      // 16-byte loads of this GPU's own rows: an element group never straddles a row
    for (int q0 = 0; q0 < (nel >> 2); q0 += 4 * OC_THREADS) {
      float4 v4[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u * OC_THREADS + threadIdx.x;
        if (q < (nel >> 2)) v4[u] = __ldcg(reinterpret_cast<const float4*>(a) + q);
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int q = q0 + u * OC_THREADS + threadIdx.x;
        if (q < (nel >> 2)) {
          const int i = q << 2, row = i / r;
          float* x = xs + row * S + (i - row * r);
          x[0] = v4[u].x; x[1] = v4[u].y; x[2] = v4[u].z; x[3] = v4[u].w;
        }
      }
    }
  }
  for (int base = vec4 ? nel : 0; base < nel; base += 4 * OC_THREADS) {
    float v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * OC_THREADS + threadIdx.x;
      v[u] = 0.f;
      if (i < nel) {
        if (peer_bufs != nullptr) {
          if (peers_ok) for (int p = 0; p < world; ++p) v[u] += ld_relaxed_sys_f32(peer_bufs[p] + off + i);
        } else {
          v[u] = a[i];
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int i = base + u * OC_THREADS + threadIdx.x;
      if (i < nel) {
        const int row = i / r;
        xs[row * S + (i - row * r)] = v[u];
      }
    }
  }
  const int pairs = r * r;
  float* pk = packed ? packed + (which == 0 ? M.ppk_off : M.qpk_off) : nullptr;
  const bool project = X.tables != nullptr && which == 1 && pk != nullptr && M.tab_off >= 0;
  const int32_t* tab = project ? X.tables + M.tab_off : nullptr;
  float* zpk = project ? packed + mats[X.nm + rec].qpk_off : nullptr;
  const float refill_scale = rsqrtf((float)rows_total);

#pragma unroll 1
  for (int round = 0; round < 2; ++round) {
    __syncthreads();
    // ---- Gram partial of this CTA's rows, fixed summation order: warps over row slices, then warps in order ----
    if (pairs <= 256) {
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      const int per = (rows + (OC_THREADS / 32) - 1) / (OC_THREADS / 32);
      const int i0 = warp * per, i1 = min(rows, i0 + per);
      for (int pr = lane; pr < pairs; pr += 32) {
        const int ca = pr / r, cb = pr - ca * r;
        float acc = 0.f;
        for (int i = i0; i < i1; ++i) acc = fmaf(xs[i * S + ca], xs[i * S + cb], acc);
        part[warp][pr] = acc;
      }
      __syncthreads();
      if ((int)threadIdx.x < pairs) {
        float acc = 0.f;
#pragma unroll
        for (int w = 0; w < OC_THREADS / 32; ++w) acc += part[w][threadIdx.x];
        gpart[round][threadIdx.x] = acc;
      }
    } else {
      for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
        const int ca = pr / r, cb = pr - ca * r;
        float acc = 0.f;
        for (int i = 0; i < rows; ++i) acc = fmaf(xs[i * S + ca], xs[i * S + cb], acc);
        gpart[round][pr] = acc;
      }
    }
    cluster_sync_all();      // every CTA's partial of this round is in its shared memory
    // ---- the block's Gram matrix: the cluster's partials in rank order; factor; inverse ----
    for (int i = threadIdx.x; i < RP * (RP + 1); i += OC_THREADS) (&R[0][0])[i] = 0.f;
    for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
      float gv[OCL];
#pragma unroll
      for (int c = 0; c < OCL; ++c) gv[c] = ld_dsmem_f32(&gpart[round][pr], (uint32_t)c);
      float acc = 0.f;
#pragma unroll
      for (int c = 0; c < OCL; ++c) acc += gv[c];
      G[pr / r][pr % r] = acc;
    }
    __syncthreads();
    if (threadIdx.x < 32) chol_factor<RP>(G, R, rd, r, round == 0 ? ORTH_SHIFT : ORTH_SHIFT_FINAL, round == 0 ? eps : 0.f);
    __syncthreads();
    // ---- apply: every thread its rows ----
    for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
      float av[RP];
#pragma unroll
      for (int k = 0; k < RP; ++k) av[k] = xs[i * S + k];
      float psc = 0.f;
      long long ph = 0;
      if (round == 1 && project) {
        const int e = tab[grow0 + i];
        psc = unpack_sign(e) * X.alpha;
        ph = unpack_bucket(e);
      }
      float yv[RP];
      apply_factor<RP>(av, R, rd, r, yv);
#pragma unroll
      for (int c = 0; c < RP; ++c) {
        if (c < r) {
          const float v = yv[c];
          if (round == 0) {
            xs[i * S + c] = v;
          } else {
            a[(size_t)i * r + c] = v;
            if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
            if (project) atomicAdd(zpk + conef_packed_offset(ph, c, packed_np), psc * v);
          }
        }
      }
    }
  }
  // ---- columns that were exactly zero: fixed pseudo-random values instead (rare; not unrolled) ----
#pragma unroll 1
  for (int c = 0; c < r; ++c) {
    if (R[c][c] > 0.f) continue;
    for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
      float z[4];
      conef_philox_normal4(ORTH_REFILL_SEED + (unsigned long long)rec * 64ull + (unsigned long long)which * 32ull + c,
                           (uint64_t)(grow0 + i), z);
      const float v = z[0] * refill_scale;
      a[(size_t)i * r + c] = v;
      if (packed) conef_pack_store(packed, M, which, grow0 + i, c, v, packed_np);
      if (project) {
        const int e = tab[grow0 + i];
        atomicAdd(zpk + conef_packed_offset(unpack_bucket(e), c, packed_np), unpack_sign(e) * X.alpha * v);
      }
    }
  }
  cluster_sync_all();      // no CTA leaves while a neighbour may still read its partials
}

// *launched: false when the rows of the largest block do not fit in shared memory or the device cannot
// hold one cluster; the caller then takes another form.
template <int RP>
static int launch_orth_cluster(const ConefMat* mats, const int2* list, int nmat, int max_rows, int seg_ctas, int which,
                               float* buf, float eps, const float* const* peer_bufs, const uint32_t* flags, int world,
                               uint32_t epoch, int* status, long long spin_limit, float* packed, int packed_np,
                               const uint32_t* epoch_base, const ConefOrthExtra& X, cudaStream_t stream,
                               bool* launched) {
  *launched = false;
  // a cluster has eight CTAs for a block however tall it is: beyond OCL_MAX_ROWS rows per CTA the form that
  // splits every block into 512-row chunks over as many CTAs as it takes is faster
  if ((max_rows + OCL - 1) / OCL > OCL_MAX_ROWS) return 0;
  const size_t smem = (size_t)((max_rows + OCL - 1) / OCL) * (RP + 1) * sizeof(float);
  if (smem > 180 * 1024) return 0;
  static size_t configured[64] = {};      // largest opt-in so far, per device
  static int cluster_ok[64] = {};         // 1: clusters of OCL CTAs can be scheduled, -1: they cannot
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return 0;
  if (smem > configured[dev]) {      // static + dynamic shared memory may pass 48 KB well before the dynamic part does
    CONEF_CUDA(cudaFuncSetAttribute(k_orth_cluster<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    configured[dev] = smem;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  const int spare = (seg_ctas + OCL - 1) / OCL * OCL;
  cfg.gridDim = dim3((unsigned)(nmat * OCL + spare), 1, 1);
  cfg.blockDim = dim3(OC_THREADS, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = OCL;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  static size_t probed[64] = {};          // shared memory the answer below was obtained with
  if (cluster_ok[dev] == 0 || smem > probed[dev]) {
    probed[dev] = smem;
    int nclusters = 0;
    const cudaError_t e = cudaOccupancyMaxActiveClusters(&nclusters, k_orth_cluster<RP>, &cfg);
    cluster_ok[dev] = (e == cudaSuccess && nclusters > 0) ? 1 : -1;
    if (e != cudaSuccess) (void)cudaGetLastError();
  }
  if (cluster_ok[dev] < 0) return 0;
  CONEF_CUDA(cudaLaunchKernelEx(&cfg, k_orth_cluster<RP>, mats, list, nmat, which, buf, peer_bufs, flags, world, epoch,
                                status, spin_limit, epoch_base, eps, packed, packed_np, X));
  *launched = true;
  return 0;
}

template <int RP>
static int launch_orth_one(const ConefMat* mats, const int2* tiles, int ntiles, int seg_ctas, int which, float* buf,
                           float eps, const float* const* peer_bufs, const uint32_t* flags, int world, uint32_t epoch,
                           int* status, long long spin_limit, float* packed, int packed_np, float* gram,
                           const uint32_t* epoch_base, uint32_t* bar, const ConefOrthExtra& X, cudaStream_t stream,
                           bool* launched) {
  *launched = false;
  constexpr size_t smem = (size_t)OC_ROWS * (RP + 1) * sizeof(float);
  static int capacity[64] = {};          // tile CTAs that can be resident at once, per device
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return 0;
  if (capacity[dev] == 0) {
    if (smem > 48 * 1024)
      CONEF_CUDA(cudaFuncSetAttribute(k_orth_one<RP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int per_sm = 0, sms = 0;
    CONEF_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, k_orth_one<RP>, OC_THREADS, smem));
    CONEF_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    capacity[dev] = per_sm * sms > 0 ? per_sm * sms : -1;
  }
  if (ntiles + seg_ctas > capacity[dev]) return 0;      // the caller uses the three-kernel form
  k_orth_one<RP><<<ntiles + seg_ctas, OC_THREADS, smem, stream>>>(mats, tiles, ntiles, which, buf, gram, peer_bufs,
                                                                 flags, world, epoch, status, spin_limit, epoch_base,
                                                                 eps, packed, packed_np, bar, X);
  CONEF_CHECK_LAUNCH("k_orth_one");
  *launched = true;
  return 0;
}

static thread_local int g_orth_launches = 0;
// Kernels enqueued by this thread's most recent conef_orthogonalize_* call (1 or 3).
extern "C" int conef_orth_last_launches(void) { return g_orth_launches; }

// gram: scratch of 2 * ntiles * 1024 floats (one Gram partial per tile and round).
extern "C" int conef_orthogonalize_fused(const ConefMat* mats, const int2* tiles, int ntiles, int which, float* buf,
                                         float eps, const float* const* peer_bufs, const uint32_t* flags, int world,
                                         uint32_t epoch, int* status, long long spin_limit, float* packed,
                                         int packed_np, float* gram, const uint32_t* epoch_base,
                                         const ConefOrthExtra* extra, cudaStream_t stream) {
  ConefOrthExtra X;
  if (extra) X = *extra; else memset(&X, 0, sizeof(X));
  if (X.seg_total <= 0 || X.nsegs <= 0) { X.seg_mode = 0; X.seg_total = 0; }
  int seg_ctas = 0;
  if (X.seg_mode) {
    seg_ctas = (int)((X.seg_total + 4 * OC_THREADS - 1) / (4 * OC_THREADS));
    if (seg_ctas > 64) seg_ctas = 64;
  }
  if (ntiles <= 0 && seg_ctas == 0 && X.zero0_n <= 0 && X.zero1_n <= 0) return 0;
  if (ntiles < 0) ntiles = 0;
  if (ntiles > 0 && X.cl_list != nullptr && X.cl_nmat > 0 && X.cl_max_rows > 0 && X.max_rank > 0 &&
      X.max_rank <= OC_MAXR) {
    // one cluster per block when a CTA's share of the largest block fits in shared memory
    bool launched = false;
    int rc;
#define CONEF_ORTH_CL(RP)                                                                                        \
    rc = launch_orth_cluster<RP>(mats, X.cl_list, X.cl_nmat, X.cl_max_rows, seg_ctas, which, buf, eps, peer_bufs, \
                                 flags, world, epoch, status, spin_limit, packed, packed_np, epoch_base, X, stream, \
                                 &launched)
    if (X.max_rank <= 4) CONEF_ORTH_CL(4);
    else if (X.max_rank <= 8) CONEF_ORTH_CL(8);
    else if (X.max_rank <= 16) CONEF_ORTH_CL(16);
    else CONEF_ORTH_CL(32);
#undef CONEF_ORTH_CL
    if (rc != 0) return rc;
    if (launched) { g_orth_launches = 1; return 0; }
  }
  if (ntiles > 0 && X.bar != nullptr && X.max_rank > 0 && X.max_rank <= OC_MAXR) {
    // one launch when all tile CTAs can be resident together
    bool launched = false;
    int rc;
#define CONEF_ORTH_ONE(RP)                                                                                     \
    rc = launch_orth_one<RP>(mats, tiles, ntiles, seg_ctas, which, buf, eps, peer_bufs, flags, world, epoch, \
                             status, spin_limit, packed, packed_np, gram, epoch_base, X.bar, X, stream, &launched)
    if (X.max_rank <= 4) CONEF_ORTH_ONE(4);
    else if (X.max_rank <= 8) CONEF_ORTH_ONE(8);
    else if (X.max_rank <= 16) CONEF_ORTH_ONE(16);
    else CONEF_ORTH_ONE(32);
#undef CONEF_ORTH_ONE
    if (rc != 0) return rc;
    if (launched) { g_orth_launches = 1; return 0; }
  }
  g_orth_launches = ntiles > 0 ? 3 : 1;
  int grid = ntiles + seg_ctas;
  if (grid == 0) grid = 1;      // only regions to clear (after the flag wait)
  float* gram2 = gram + (size_t)ntiles * GRAM_STRIDE;
  k_gram<<<grid, OC_THREADS, 0, stream>>>(mats, tiles, ntiles, which, buf, gram,
                                         peer_bufs, flags, world, epoch, status, spin_limit, epoch_base, X);
  CONEF_CHECK_LAUNCH("k_gram");
  if (ntiles <= 0) return 0;
  k_qr_apply<<<ntiles, OC_THREADS, 0, stream>>>(mats, tiles, which, buf, gram, gram2, eps, ORTH_SHIFT, nullptr, 0,
                                               nullptr, 0, 0.f);
  CONEF_CHECK_LAUNCH("k_qr_apply");
  k_qr_apply<<<ntiles, OC_THREADS, 0, stream>>>(mats, tiles, which, buf, gram2, nullptr, 0.f, ORTH_SHIFT_FINAL, packed,
                                               packed_np, X.tables, X.nm, X.alpha);
  CONEF_CHECK_LAUNCH("k_qr_apply");
  return 0;
}

extern "C" int conef_orthogonalize_packed_ex(const ConefMat* mats, const int2* tiles, int ntiles, int nrecords,
                                             int which, float* buf, float eps, const float* const* peer_bufs,
                                             const uint32_t* flags, int world, uint32_t epoch, int* status,
                                             long long spin_limit, float* packed, int packed_np, float* gram,
                                             const uint32_t* epoch_base, cudaStream_t stream) {
  (void)nrecords;
  if (ntiles <= 0) return 0;
  return conef_orthogonalize_fused(mats, tiles, ntiles, which, buf, eps, world > 1 ? peer_bufs : nullptr, flags,
                                   world, epoch, status, spin_limit, packed, packed_np, gram, epoch_base, nullptr,
                                   stream);
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
//
// k_corr_reduce: C = L^T Rm over the chunk's rows.  The rows come into shared memory in sub-chunks
// with coalesced loads first: summing straight from global memory leaves one load in flight per
// thread (the loop over rows is a chain of dependent-latency iterations) and took 70-130 us per
// launch on a Transformer-sized bucket.
constexpr int CR_SUB = 128;                       // rows per sub-chunk
__global__ void __launch_bounds__(OC_THREADS)
k_corr_reduce(const ConefCorr* __restrict__ table, const int2* __restrict__ tiles, const float* __restrict__ L0b,
              const float* __restrict__ R0b, const float* __restrict__ L1b, const float* __restrict__ R1b,
              float* __restrict__ cbuf) {
  __shared__ float Ls[CR_SUB * OC_MAXR];
  __shared__ float Rs[CR_SUB * OC_MAXR];
  __shared__ float part[OC_THREADS / 32][256];
  const int2 t = tiles[blockIdx.x];
  const ConefCorr K = table[t.x];
  const int row0 = t.y * OC_ROWS;
  const int rows = min(OC_ROWS, K.rows_l - row0);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int term = 0; term < K.nterms; ++term) {
    const int c2 = K.c2[term], c1 = K.c1;
    const int pairs = c1 * c2;
    const float* L = (term ? L1b : L0b) + K.l_off[term] + (size_t)row0 * c2;
    const float* Rm = (term ? R1b : R0b) + K.r_off[term] + (size_t)row0 * c1;
    float* c = cbuf + ((size_t)t.x * 2 + term) * GRAM_STRIDE;
    // every warp owns a slice of each sub-chunk's rows; lanes own pairs (a, b) = (pr / c1, pr % c1)
    float acc[8];                                  // pairs handled by this lane: pr = lane + 32 u (pairs <= 256)
#pragma unroll
    for (int u = 0; u < 8; ++u) acc[u] = 0.f;
    for (int s0 = 0; s0 < rows; s0 += CR_SUB) {
      const int sub = min(CR_SUB, rows - s0);
      __syncthreads();
      for (int i = threadIdx.x; i < sub * c2; i += OC_THREADS) Ls[i] = L[(size_t)s0 * c2 + i];
      for (int i = threadIdx.x; i < sub * c1; i += OC_THREADS) Rs[i] = Rm[(size_t)s0 * c1 + i];
      __syncthreads();
      if (pairs <= 256) {
        const int per = (sub + (OC_THREADS / 32) - 1) / (OC_THREADS / 32);
        const int i0 = warp * per, i1 = min(sub, i0 + per);
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int pr = lane + 32 * u;
          if (pr < pairs) {
            const int a = pr / c1, b = pr - a * c1;
            float v = acc[u];
            for (int i = i0; i < i1; ++i) v = fmaf(Ls[i * c2 + a], Rs[i * c1 + b], v);
            acc[u] = v;
          }
        }
      } else {                                     // ranks above 16: every thread its pairs over all rows
        for (int pr = threadIdx.x; pr < pairs; pr += OC_THREADS) {
          const int a = pr / c1, b = pr - a * c1;
          float v = 0.f;
          for (int i = 0; i < sub; ++i) v = fmaf(Ls[i * c2 + a], Rs[i * c1 + b], v);
          atomicAdd(c + pr, v);
        }
      }
    }
    if (pairs <= 256) {
      __syncthreads();
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (lane + 32 * u < pairs) part[warp][lane + 32 * u] = acc[u];
      __syncthreads();
      if ((int)threadIdx.x < pairs) {
        float v = 0.f;
#pragma unroll
        for (int w = 0; w < OC_THREADS / 32; ++w) v += part[w][threadIdx.x];
        atomicAdd(c + threadIdx.x, v);
      }
    }
  }
}

// k_corr_apply: T += sum_t coef_t X_t C_t.  A thread owns whole rows (its X row in registers, the small
// C matrices in shared memory), so every row is one pass of wide loads and stores.
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
  for (int i = threadIdx.x; i < rows; i += OC_THREADS) {
    float out[OC_MAXR];
#pragma unroll
    for (int b = 0; b < OC_MAXR; ++b) out[b] = 0.f;
    for (int term = 0; term < K.nterms; ++term) {
      const int c2 = K.c2[term];
      const float coef = term ? coef1 : coef0;
      const float* X = (term ? X1b : X0b) + K.x_off[term] + (size_t)(row0 + i) * c2;
      for (int a = 0; a < c2; ++a) {
        const float xa = coef * X[a];
#pragma unroll
        for (int b = 0; b < OC_MAXR; ++b)
          if (b < c1) out[b] = fmaf(xa, Csm[term][a * c1 + b], out[b]);
      }
    }
    float* trow = T + (size_t)i * c1;
#pragma unroll
    for (int b = 0; b < OC_MAXR; ++b)
      if (b < c1) trow[b] += out[b];
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
