// Column sums of a row-major (rows x cols) matrix: the bias gradient of a convolution whose output gradient
// lies in channels-last memory ((N, H, W, C) = (N H W) rows of C channels).  PyTorch computes it with its
// generic reduction kernel, which on a 42 MB bf16 gradient of WRN-28-10 takes 78 us (0.5 TB/s); 28 of them are
// 2.3 ms of an 18 ms training step.  Here a CTA streams a slab of rows with 16-byte loads (a thread owns
// eight adjacent columns and every (256 / (cols / 8))-th row of the slab), adds up in fp32, combines its row
// groups through shared memory and writes one partial row; a second small kernel adds the partials in CTA
// order, so the result does not depend on scheduling.
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "common.cuh"

constexpr int CS_THREADS = 256;
constexpr int CS_MAX_COLS = 8 * CS_THREADS;      // one column chunk per thread at least

template <typename T> struct Chunk8;      // eight elements = one 16-byte (bf16 / fp16) or two 16-byte (fp32) loads
template <> struct Chunk8<__nv_bfloat16> {
  static __device__ __forceinline__ void add(const __nv_bfloat16* p, float (&acc)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
  }
};
template <> struct Chunk8<__half> {
  static __device__ __forceinline__ void add(const __half* p, float (&acc)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); acc[2 * i] += f.x; acc[2 * i + 1] += f.y; }
  }
};
template <> struct Chunk8<float> {
  static __device__ __forceinline__ void add(const float* p, float (&acc)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    acc[0] += a.x; acc[1] += a.y; acc[2] += a.z; acc[3] += a.w; acc[4] += b.x; acc[5] += b.y; acc[6] += b.z; acc[7] += b.w;
  }
};

// partial[blockIdx.x][0..cols) = sum over the CTA's slab of rows.  cols % 8 == 0, cols <= CS_MAX_COLS,
// x 16-byte aligned.
template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
k_colsum_partial(const T* __restrict__ x, long long rows, int cols, long long rows_per_cta, float* __restrict__ partial) {
  extern __shared__ float cs_sm[];      // (row groups) x cols
  const int chunks = cols >> 3;                       // threads per row
  const int groups = CS_THREADS / chunks;             // rows in flight per pass
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  if (rr < groups) {
    const T* p = x + (size_t)(r0 + rr) * cols + 8 * cc;
    const size_t step = (size_t)groups * cols;
    long long row = r0 + rr;
    // four rows per thread in flight
    for (; row + 3LL * groups < r1; row += 4LL * groups, p += 4 * step) {
      Chunk8<T>::add(p, acc);
      Chunk8<T>::add(p + step, acc);
      Chunk8<T>::add(p + 2 * step, acc);
      Chunk8<T>::add(p + 3 * step, acc);
    }
    for (; row < r1; row += groups, p += step) Chunk8<T>::add(p, acc);
#pragma unroll
    for (int i = 0; i < 8; ++i) cs_sm[rr * cols + 8 * cc + i] = acc[i];
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += CS_THREADS) {
    float s = 0.f;
    for (int g = 0; g < groups; ++g) s += cs_sm[g * cols + c];      // fixed order
    partial[(size_t)blockIdx.x * cols + c] = s;
  }
}

// Second stage: a CTA of CF_THREADS threads adds up the partial rows of CF_COLS columns.  Thread (slice, col)
// sums every CF_SLICES-th partial row with eight loads in flight, the slices are then added in slice order:
// the order of the additions is fixed, and no thread walks more than nparts / CF_SLICES values.
constexpr int CF_COLS = 32, CF_SLICES = 8, CF_THREADS = CF_COLS * CF_SLICES;
__device__ __forceinline__ float cf_combine(const float* __restrict__ partial, int nparts, size_t part_stride, int c,
                                            int cols, float* sm /* CF_THREADS floats */) {
  const int col_l = threadIdx.x % CF_COLS, slice = threadIdx.x / CF_COLS;
  float s = 0.f;
  if (c < cols) {
    int p = slice;
    for (; p + 7 * CF_SLICES < nparts; p += 8 * CF_SLICES) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = partial[(size_t)(p + u * CF_SLICES) * part_stride + c];
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; p < nparts; p += CF_SLICES) s += partial[(size_t)p * part_stride + c];
  }
  __syncthreads();      // the scratch may still be in use by a previous call
  sm[slice * CF_COLS + col_l] = s;
  __syncthreads();
  float total = 0.f;
#pragma unroll
  for (int u = 0; u < CF_SLICES; ++u) total += sm[u * CF_COLS + col_l];
  return total;      // the same value in every slice of a column
}

__global__ void __launch_bounds__(CF_THREADS)
k_colsum_final(const float* __restrict__ partial, int nparts, int cols, float* __restrict__ out) {
  __shared__ float sm[CF_THREADS];
  const int c = blockIdx.x * CF_COLS + threadIdx.x % CF_COLS;
  const float s = cf_combine(partial, nparts, (size_t)cols, c, cols, sm);
  if (c < cols && threadIdx.x < CF_COLS) out[c] = s;
}

template <typename T>
static int launch_colsum(const void* x, long long rows, int cols, float* partial, int nparts, float* out,
                         cudaStream_t stream) {
  const long long rows_per_cta = (rows + nparts - 1) / nparts;
  const int groups = CS_THREADS / (cols >> 3);
  const size_t smem = (size_t)groups * cols * sizeof(float);
  static size_t configured[64] = {};
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
    CONEF_CUDA(cudaFuncSetAttribute(k_colsum_partial<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = smem;
  }
  k_colsum_partial<T><<<nparts, CS_THREADS, smem, stream>>>((const T*)x, rows, cols, rows_per_cta, partial);
  CONEF_CHECK_LAUNCH("k_colsum_partial");
  k_colsum_final<<<(cols + CF_COLS - 1) / CF_COLS, CF_THREADS, 0, stream>>>(partial, nparts, cols, out);
  CONEF_CHECK_LAUNCH("k_colsum_final");
  return 0;
}

// dtype: 0 fp32, 1 bf16, 2 fp16.  partial: scratch of nparts * cols floats.  Returns 2 for shapes it does not
// take (cols not a multiple of 8, more than 2048 columns, unaligned x): the caller then uses a library sum.
extern "C" int conef_colsum(const void* x, int dtype, long long rows, int cols, float* partial, int nparts, float* out,
                            cudaStream_t stream) {
  if (rows <= 0 || cols <= 0 || nparts <= 0) { conef_set_error("colsum: empty input"); return 1; }
  if ((cols & 7) != 0 || cols > CS_MAX_COLS || (reinterpret_cast<uintptr_t>(x) & 15) != 0) {
    conef_set_error("colsum: needs cols %% 8 == 0, cols <= %d and a 16-byte aligned input", CS_MAX_COLS);
    return 2;
  }
  if (dtype == 0) return launch_colsum<float>(x, rows, cols, partial, nparts, out, stream);
  if (dtype == 1) return launch_colsum<__nv_bfloat16>(x, rows, cols, partial, nparts, out, stream);
  if (dtype == 2) return launch_colsum<__half>(x, rows, cols, partial, nparts, out, stream);
  conef_set_error("colsum: dtype %d", dtype);
  return 1;
}

// ---------------------------------------------------------------------------
// Batch-norm statistics over a channels-last activation: per column the sums of (x - pivot) and (x - pivot)^2
// with pivot = x[0, c] (shifted sums: the variance does not cancel when |mean| >> std), then mean, 1 / std and
// the running statistics in a small second kernel.  Same slab / row-group layout as k_colsum_partial.
template <typename T> struct Load8;
template <> struct Load8<__nv_bfloat16> {
  static __device__ __forceinline__ void get(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
};
template <> struct Load8<__half> {
  static __device__ __forceinline__ void get(const __half* p, float (&v)[8]) {
    const uint4 u = __ldcs(reinterpret_cast<const uint4*>(p));
    const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
  }
};
template <> struct Load8<float> {
  static __device__ __forceinline__ void get(const float* p, float (&v)[8]) {
    const float4 a = __ldcs(reinterpret_cast<const float4*>(p)), b = __ldcs(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
};

// per-channel scale = invstd * weight and shift = bias - mean * scale for the eight columns of a thread
__device__ __forceinline__ void bn_coeffs(const float* mean, const float* invstd, const float* weight, const float* bias,
                                          int c0, float (&scale)[8], float (&shift)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    scale[i] = invstd[c0 + i] * (weight ? weight[c0 + i] : 1.f);
    shift[i] = (bias ? bias[c0 + i] : 0.f) - mean[c0 + i] * scale[i];
  }
}

// MODE 0: s1 = sum (x - pivot), s2 = sum (x - pivot)^2, pivot = x[0, c] (`y` unused).
// MODE 1: s1 = sum y, s2 = sum y (x - center[c]): the two sums of the batch-norm backward pass (y = dL/dout).
// MODE 2: as MODE 1 with y masked by the ReLU that follows the batch norm: y counts where
//         (x - mean) invstd weight + bias > 0 (center = mean; invstd, weight, bias given).
// partial[blockIdx.x][0 | 1][0..cols).
template <typename T, int MODE>
__global__ void __launch_bounds__(CS_THREADS)
k_colpair_partial(const T* __restrict__ x, const T* __restrict__ y, const float* __restrict__ center, long long rows,
                  int cols, long long rows_per_cta, float* __restrict__ partial, const float* __restrict__ invstd,
                  const float* __restrict__ weight, const float* __restrict__ bias) {
  extern __shared__ float cs_sm[];      // (row groups) x 2 x cols
  const int chunks = cols >> 3;
  const int groups = CS_THREADS / chunks;
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float s1[8], s2[8], ctr[8], scale[8], shift[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { s1[i] = 0.f; s2[i] = 0.f; scale[i] = 0.f; shift[i] = 0.f; }
  if (rr < groups) {
    if (MODE == 0) {
      Load8<T>::get(x + 8 * cc, ctr);
    } else {
#pragma unroll
      for (int i = 0; i < 8; ++i) ctr[i] = center[8 * cc + i];
      if (MODE == 2) bn_coeffs(center, invstd, weight, bias, 8 * cc, scale, shift);
    }
    const size_t step = (size_t)groups * cols;
    size_t off = (size_t)(r0 + rr) * cols + 8 * cc;
    long long row = r0 + rr;
    for (; row + groups < r1; row += 2LL * groups, off += 2 * step) {      // two rows (times two arrays) in flight
      float a[8], b[8], ya[8], yb[8];
      Load8<T>::get(x + off, a);
      Load8<T>::get(x + off + step, b);
      if (MODE >= 1) { Load8<T>::get(y + off, ya); Load8<T>::get(y + off + step, yb); }
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (MODE == 2) {
          if (!(fmaf(a[i], scale[i], shift[i]) > 0.f)) ya[i] = 0.f;
          if (!(fmaf(b[i], scale[i], shift[i]) > 0.f)) yb[i] = 0.f;
        }
        const float da = a[i] - ctr[i], db = b[i] - ctr[i];
        if (MODE == 0) { s1[i] += da + db; s2[i] = fmaf(da, da, fmaf(db, db, s2[i])); }
        else { s1[i] += ya[i] + yb[i]; s2[i] = fmaf(ya[i], da, fmaf(yb[i], db, s2[i])); }
      }
    }
    for (; row < r1; row += groups, off += step) {
      float a[8], ya[8];
      Load8<T>::get(x + off, a);
      if (MODE >= 1) Load8<T>::get(y + off, ya);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        if (MODE == 2 && !(fmaf(a[i], scale[i], shift[i]) > 0.f)) ya[i] = 0.f;
        const float da = a[i] - ctr[i];
        if (MODE == 0) { s1[i] += da; s2[i] = fmaf(da, da, s2[i]); }
        else { s1[i] += ya[i]; s2[i] = fmaf(ya[i], da, s2[i]); }
      }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      cs_sm[(rr * 2 + 0) * cols + 8 * cc + i] = s1[i];
      cs_sm[(rr * 2 + 1) * cols + 8 * cc + i] = s2[i];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * cols; c += CS_THREADS) {
    const int which = c / cols, col = c - which * cols;
    float s = 0.f;
    for (int g = 0; g < groups; ++g) s += cs_sm[(g * 2 + which) * cols + col];      // fixed order
    partial[((size_t)blockIdx.x * 2 + which) * cols + col] = s;
  }
}

// mean, 1 / sqrt(var + eps) (biased variance) and, when given, the running statistics
// (running = (1 - momentum) running + momentum new; the running variance takes the unbiased estimate).
template <typename T>
__global__ void __launch_bounds__(CF_THREADS) k_colstats_final(const float* __restrict__ partial, int nparts, const T* __restrict__ x, long long rows,
                                 int cols, float eps, float momentum, float* __restrict__ mean,
                                 float* __restrict__ invstd, float* __restrict__ running_mean,
                                 float* __restrict__ running_var) {
  __shared__ float sm[CF_THREADS];
  const int c = blockIdx.x * CF_COLS + threadIdx.x % CF_COLS;
  const float s1 = cf_combine(partial, nparts, (size_t)2 * cols, c, cols, sm);
  const float s2 = cf_combine(partial + cols, nparts, (size_t)2 * cols, c, cols, sm);
  if (c >= cols || threadIdx.x >= CF_COLS) return;
  const float n = (float)rows;
  const float pivot = (float)x[c];
  const float m1 = s1 / n;
  const float var = fmaxf(s2 / n - m1 * m1, 0.f);
  const float mu = pivot + m1;
  mean[c] = mu;
  invstd[c] = rsqrtf(var + eps);
  if (running_mean != nullptr) running_mean[c] = (1.f - momentum) * running_mean[c] + momentum * mu;
  if (running_var != nullptr)
    running_var[c] = (1.f - momentum) * running_var[c] + momentum * var * (rows > 1 ? n / (n - 1.f) : 1.f);
}

// sum_dy, sum_dy_xmu and, when given, grad_weight = sum_dy_xmu * invstd and grad_bias = sum_dy
__global__ void __launch_bounds__(CF_THREADS) k_coldot_final(const float* __restrict__ partial, int nparts, int cols,
                               const float* __restrict__ invstd, float* __restrict__ sum_dy,
                               float* __restrict__ sum_dy_xmu, float* __restrict__ grad_weight,
                               float* __restrict__ grad_bias) {
  __shared__ float sm[CF_THREADS];
  const int c = blockIdx.x * CF_COLS + threadIdx.x % CF_COLS;
  const float s1 = cf_combine(partial, nparts, (size_t)2 * cols, c, cols, sm);
  const float s2 = cf_combine(partial + cols, nparts, (size_t)2 * cols, c, cols, sm);
  if (c >= cols || threadIdx.x >= CF_COLS) return;
  sum_dy[c] = s1;
  sum_dy_xmu[c] = s2;
  if (grad_weight != nullptr) grad_weight[c] = s2 * invstd[c];
  if (grad_bias != nullptr) grad_bias[c] = s1;
}

static bool colpair_ok(const void* x, const void* y, long long rows, int cols, int nparts) {
  if (rows <= 0 || cols <= 0 || nparts <= 0) return false;
  if ((cols & 7) != 0 || cols > CS_MAX_COLS) return false;
  if ((reinterpret_cast<uintptr_t>(x) & 15) != 0 || (reinterpret_cast<uintptr_t>(y) & 15) != 0) return false;
  return true;
}

template <typename T, int MODE>
static int launch_colpair(const void* x, const void* y, const float* center, long long rows, int cols, float* partial,
                          int nparts, cudaStream_t stream, const float* invstd = nullptr, const float* weight = nullptr,
                          const float* bias = nullptr) {
  const long long rows_per_cta = (rows + nparts - 1) / nparts;
  const int groups = CS_THREADS / (cols >> 3);
  const size_t smem = (size_t)groups * 2 * cols * sizeof(float);
  static size_t configured[64] = {};
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (smem > 48 * 1024 && (dev < 0 || dev >= 64 || smem > configured[dev])) {
    CONEF_CUDA(cudaFuncSetAttribute(k_colpair_partial<T, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    if (dev >= 0 && dev < 64) configured[dev] = smem;
  }
  k_colpair_partial<T, MODE><<<nparts, CS_THREADS, smem, stream>>>((const T*)x, (const T*)y, center, rows, cols,
                                                                  rows_per_cta, partial, invstd, weight, bias);
  CONEF_CHECK_LAUNCH("k_colpair_partial");
  return 0;
}

template <typename T>
static int colstats_t(const void* x, long long rows, int cols, float eps, float momentum, float* partial, int nparts,
                      float* mean, float* invstd, float* running_mean, float* running_var, cudaStream_t stream) {
  const int rc = launch_colpair<T, 0>(x, x, nullptr, rows, cols, partial, nparts, stream);
  if (rc != 0) return rc;
  k_colstats_final<T><<<(cols + CF_COLS - 1) / CF_COLS, CF_THREADS, 0, stream>>>(partial, nparts, (const T*)x, rows, cols, eps, momentum,
                                                             mean, invstd, running_mean, running_var);
  CONEF_CHECK_LAUNCH("k_colstats_final");
  return 0;
}

// Batch statistics of a row-major (rows x cols) activation (channels-last: rows = N H W).  partial: scratch of
// nparts * 2 * cols floats.  running_mean / running_var may be NULL.  Returns 2 for inputs it does not take.
extern "C" int conef_colstats(const void* x, int dtype, long long rows, int cols, float eps, float momentum,
                              float* partial, int nparts, float* mean, float* invstd, float* running_mean,
                              float* running_var, cudaStream_t stream) {
  if (!colpair_ok(x, x, rows, cols, nparts)) { conef_set_error("colstats: shape or alignment not supported"); return 2; }
  if (dtype == 0) return colstats_t<float>(x, rows, cols, eps, momentum, partial, nparts, mean, invstd, running_mean, running_var, stream);
  if (dtype == 1) return colstats_t<__nv_bfloat16>(x, rows, cols, eps, momentum, partial, nparts, mean, invstd, running_mean, running_var, stream);
  if (dtype == 2) return colstats_t<__half>(x, rows, cols, eps, momentum, partial, nparts, mean, invstd, running_mean, running_var, stream);
  conef_set_error("colstats: dtype %d", dtype);
  return 1;
}

// The two sums of the batch-norm backward pass: sum_dy[c] = sum dy, sum_dy_xmu[c] = sum dy (x - mean[c]);
// grad_weight (= sum_dy_xmu * invstd) and grad_bias (= sum_dy) when given.  dy and x have the same dtype.
extern "C" int conef_coldot(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                            const float* invstd, float* partial, int nparts, float* sum_dy, float* sum_dy_xmu,
                            float* grad_weight, float* grad_bias, cudaStream_t stream) {
  if (!colpair_ok(x, dy, rows, cols, nparts)) { conef_set_error("coldot: shape or alignment not supported"); return 2; }
  int rc;
  if (dtype == 0) rc = launch_colpair<float, 1>(x, dy, mean, rows, cols, partial, nparts, stream);
  else if (dtype == 1) rc = launch_colpair<__nv_bfloat16, 1>(x, dy, mean, rows, cols, partial, nparts, stream);
  else if (dtype == 2) rc = launch_colpair<__half, 1>(x, dy, mean, rows, cols, partial, nparts, stream);
  else { conef_set_error("coldot: dtype %d", dtype); return 1; }
  if (rc != 0) return rc;
  k_coldot_final<<<(cols + CF_COLS - 1) / CF_COLS, CF_THREADS, 0, stream>>>(partial, nparts, cols, invstd, sum_dy, sum_dy_xmu, grad_weight,
                                                        grad_bias);
  CONEF_CHECK_LAUNCH("k_coldot_final");
  return 0;
}

// ---------------------------------------------------------------------------
// Elementwise passes of batch norm fused with the ReLU that follows it (pre-activation blocks:
// relu(bn(x))).  PyTorch runs batch_norm_elemt and relu as two passes over the activation in each
// direction; fused, the activation is read once and written once.
template <typename T> struct Store8;
template <> struct Store8<__nv_bfloat16> {
  static __device__ __forceinline__ void put(__nv_bfloat16* p, const float (&v)[8]) {
    uint4 u;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Store8<__half> {
  static __device__ __forceinline__ void put(__half* p, const float (&v)[8]) {
    uint4 u;
    __half2* h = reinterpret_cast<__half2*>(&u);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = u;
  }
};
template <> struct Store8<float> {
  static __device__ __forceinline__ void put(float* p, const float (&v)[8]) {
    reinterpret_cast<float4*>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
};

// y = x * scale + shift, then max(0, .) with RELU.  Thread (rr, cc): columns 8 cc .. 8 cc + 7, rows rr, rr + groups, ...
template <typename T, bool RELU>
__global__ void __launch_bounds__(CS_THREADS)
k_bn_apply(const T* __restrict__ x, T* __restrict__ y, long long rows, int cols, long long rows_per_cta,
           const float* __restrict__ mean, const float* __restrict__ invstd, const float* __restrict__ weight,
           const float* __restrict__ bias) {
  const int chunks = cols >> 3, groups = CS_THREADS / chunks;
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  if (rr >= groups) return;
  float scale[8], shift[8];
  bn_coeffs(mean, invstd, weight, bias, 8 * cc, scale, shift);
  const long long r0 = (long long)blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  const size_t step = (size_t)groups * cols;
  size_t off = (size_t)(r0 + rr) * cols + 8 * cc;
  long long row = r0 + rr;
  for (; row + groups < r1; row += 2LL * groups, off += 2 * step) {
    float a[8], b[8];
    Load8<T>::get(x + off, a);
    Load8<T>::get(x + off + step, b);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      a[i] = fmaf(a[i], scale[i], shift[i]);
      b[i] = fmaf(b[i], scale[i], shift[i]);
      if (RELU) { a[i] = fmaxf(a[i], 0.f); b[i] = fmaxf(b[i], 0.f); }
    }
    Store8<T>::put(y + off, a);
    Store8<T>::put(y + off + step, b);
  }
  for (; row < r1; row += groups, off += step) {
    float a[8];
    Load8<T>::get(x + off, a);
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = fmaf(a[i], scale[i], shift[i]); if (RELU) a[i] = fmaxf(a[i], 0.f); }
    Store8<T>::put(y + off, a);
  }
}

// gx = (gy - sum_dy / n - (x - mean) invstd^2 sum_dy_xmu / n) invstd weight, with gy masked by the ReLU
// ((x - mean) invstd weight + bias > 0) when RELU.
template <typename T, bool RELU>
__global__ void __launch_bounds__(CS_THREADS)
k_bn_backward_apply(const T* __restrict__ gy, const T* __restrict__ x, T* __restrict__ gx, long long rows, int cols,
                    long long rows_per_cta, const float* __restrict__ mean, const float* __restrict__ invstd,
                    const float* __restrict__ weight, const float* __restrict__ bias,
                    const float* __restrict__ sum_dy, const float* __restrict__ sum_dy_xmu) {
  const int chunks = cols >> 3, groups = CS_THREADS / chunks;
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  if (rr >= groups) return;
  float scale[8], shift[8], mu[8], k0[8], k1[8], k2[8];
  bn_coeffs(mean, invstd, weight, bias, 8 * cc, scale, shift);
  const float inv_n = 1.f / (float)rows;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int c = 8 * cc + i;
    const float is = invstd[c], w = weight ? weight[c] : 1.f;
    mu[i] = mean[c];
    k0[i] = is * w;                                  // gx = (gy - k1 - (x - mu) k2) k0
    k1[i] = sum_dy[c] * inv_n;
    k2[i] = is * is * sum_dy_xmu[c] * inv_n;
  }
  const long long r0 = (long long)blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  const size_t step = (size_t)groups * cols;
  size_t off = (size_t)(r0 + rr) * cols + 8 * cc;
  long long row = r0 + rr;      // one row (two loads) per pass: two rows in flight cost occupancy and measured slower
  for (; row < r1; row += groups, off += step) {
    float g[8], a[8];
    Load8<T>::get(gy + off, g);
    Load8<T>::get(x + off, a);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (RELU && !(fmaf(a[i], scale[i], shift[i]) > 0.f)) g[i] = 0.f;
      g[i] = (g[i] - k1[i] - (a[i] - mu[i]) * k2[i]) * k0[i];
    }
    Store8<T>::put(gx + off, g);
  }
}

#define CONEF_BY_DTYPE(dtype, ...)                                             \
  do {                                                                         \
    if ((dtype) == 0) { using T = float; __VA_ARGS__; }                        \
    else if ((dtype) == 1) { using T = __nv_bfloat16; __VA_ARGS__; }           \
    else if ((dtype) == 2) { using T = __half; __VA_ARGS__; }                  \
    else { conef_set_error("unknown dtype %d", (int)(dtype)); return 1; }      \
  } while (0)

// y = relu?((x - mean) invstd weight + bias) over a row-major (rows x cols) activation; weight / bias may be NULL.
extern "C" int conef_bn_apply(const void* x, void* y, int dtype, long long rows, int cols, const float* mean,
                              const float* invstd, const float* weight, const float* bias, int relu, int nparts,
                              cudaStream_t stream) {
  if (!colpair_ok(x, y, rows, cols, nparts)) { conef_set_error("bn_apply: shape or alignment not supported"); return 2; }
  const long long rpc = (rows + nparts - 1) / nparts;
  CONEF_BY_DTYPE(dtype, {
    if (relu) k_bn_apply<T, true><<<nparts, CS_THREADS, 0, stream>>>((const T*)x, (T*)y, rows, cols, rpc, mean, invstd, weight, bias);
    else k_bn_apply<T, false><<<nparts, CS_THREADS, 0, stream>>>((const T*)x, (T*)y, rows, cols, rpc, mean, invstd, weight, bias);
  });
  CONEF_CHECK_LAUNCH("k_bn_apply");
  return 0;
}

// The backward sums with dy masked by the ReLU behind the batch norm (see k_colpair_partial, MODE 2).
extern "C" int conef_coldot_relu(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                                 const float* invstd, const float* weight, const float* bias, float* partial,
                                 int nparts, float* sum_dy, float* sum_dy_xmu, float* grad_weight, float* grad_bias,
                                 cudaStream_t stream) {
  if (!colpair_ok(x, dy, rows, cols, nparts)) { conef_set_error("coldot_relu: shape or alignment not supported"); return 2; }
  int rc = 0;
  CONEF_BY_DTYPE(dtype, { rc = launch_colpair<T, 2>(x, dy, mean, rows, cols, partial, nparts, stream, invstd, weight, bias); });
  if (rc != 0) return rc;
  k_coldot_final<<<(cols + CF_COLS - 1) / CF_COLS, CF_THREADS, 0, stream>>>(partial, nparts, cols, invstd, sum_dy,
                                                                          sum_dy_xmu, grad_weight, grad_bias);
  CONEF_CHECK_LAUNCH("k_coldot_final");
  return 0;
}

extern "C" int conef_bn_backward_apply(const void* gy, const void* x, void* gx, int dtype, long long rows, int cols,
                                       const float* mean, const float* invstd, const float* weight, const float* bias,
                                       const float* sum_dy, const float* sum_dy_xmu, int relu, int nparts,
                                       cudaStream_t stream) {
  if (!colpair_ok(x, gy, rows, cols, nparts) || (reinterpret_cast<uintptr_t>(gx) & 15) != 0) {
    conef_set_error("bn_backward_apply: shape or alignment not supported");
    return 2;
  }
  const long long rpc = (rows + nparts - 1) / nparts;
  CONEF_BY_DTYPE(dtype, {
    if (relu) k_bn_backward_apply<T, true><<<nparts, CS_THREADS, 0, stream>>>((const T*)gy, (const T*)x, (T*)gx, rows, cols, rpc, mean, invstd, weight, bias, sum_dy, sum_dy_xmu);
    else k_bn_backward_apply<T, false><<<nparts, CS_THREADS, 0, stream>>>((const T*)gy, (const T*)x, (T*)gx, rows, cols, rpc, mean, invstd, weight, bias, sum_dy, sum_dy_xmu);
  });
  CONEF_CHECK_LAUNCH("k_bn_backward_apply");
  return 0;
}

// y[row, c] += bias[c] in place over a row-major (rows x cols) activation: the bias of a convolution whose
// output lies in channels-last memory.  PyTorch adds it with a broadcasting elementwise kernel that is not
// vectorised for this layout (27 us per convolution of WRN-28-10).
template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
k_bias_add(T* __restrict__ y, long long rows, int cols, long long rows_per_cta, const float* __restrict__ bias) {
  const int chunks = cols >> 3, groups = CS_THREADS / chunks;
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  if (rr >= groups) return;
  float b[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) b[i] = bias[8 * cc + i];
  const long long r0 = (long long)blockIdx.x * rows_per_cta, r1 = min(rows, r0 + rows_per_cta);
  const size_t step = (size_t)groups * cols;
  size_t off = (size_t)(r0 + rr) * cols + 8 * cc;
  long long row = r0 + rr;
  for (; row + groups < r1; row += 2LL * groups, off += 2 * step) {
    float a[8], c[8];
    Load8<T>::get(y + off, a);
    Load8<T>::get(y + off + step, c);
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] += b[i]; c[i] += b[i]; }
    Store8<T>::put(y + off, a);
    Store8<T>::put(y + off + step, c);
  }
  for (; row < r1; row += groups, off += step) {
    float a[8];
    Load8<T>::get(y + off, a);
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] += b[i];
    Store8<T>::put(y + off, a);
  }
}

extern "C" int conef_bias_add(void* y, int dtype, long long rows, int cols, const float* bias, int nparts,
                              cudaStream_t stream) {
  if (!colpair_ok(y, y, rows, cols, nparts)) { conef_set_error("bias_add: shape or alignment not supported"); return 2; }
  const long long rpc = (rows + nparts - 1) / nparts;
  CONEF_BY_DTYPE(dtype, { k_bias_add<T><<<nparts, CS_THREADS, 0, stream>>>((T*)y, rows, cols, rpc, bias); });
  CONEF_CHECK_LAUNCH("k_bias_add");
  return 0;
}

// ---------------------------------------------------------------------------
// Weight and bias gradients of layer norm over a (rows x cols) activation normalised along its rows:
//   dgamma[c] = sum_rows dy[row, c] (x[row, c] - mean[row]) rstd[row],   dbeta[c] = sum_rows dy[row, c].
// PyTorch's kernel for this pair takes 65 us per 8192 x 1024 fp32 activation of BERT-large (50 of them per
// step); the slab layout of k_colpair_partial streams dy and x once.  partial[blockIdx.x][0 | 1][0..cols):
// 0 = dbeta, 1 = dgamma.
template <typename T>
__global__ void __launch_bounds__(CS_THREADS)
k_ln_wgrad_partial(const T* __restrict__ dy, const T* __restrict__ x, const float* __restrict__ mean,
                   const float* __restrict__ rstd, long long rows, int cols, long long rows_per_cta,
                   float* __restrict__ partial) {
  extern __shared__ float cs_sm[];      // (row groups) x 2 x cols
  const int chunks = cols >> 3;
  const int groups = CS_THREADS / chunks;
  const int cc = threadIdx.x % chunks, rr = threadIdx.x / chunks;
  const long long r0 = (long long)blockIdx.x * rows_per_cta;
  const long long r1 = min(rows, r0 + rows_per_cta);
  float s1[8], s2[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) { s1[i] = 0.f; s2[i] = 0.f; }
  if (rr < groups) {
    const size_t step = (size_t)groups * cols;
    size_t off = (size_t)(r0 + rr) * cols + 8 * cc;
    long long row = r0 + rr;
    for (; row + groups < r1; row += 2LL * groups, off += 2 * step) {      // two rows in flight
      float a[8], b[8], ya[8], yb[8];
      Load8<T>::get(x + off, a);
      Load8<T>::get(x + off + step, b);
      Load8<T>::get(dy + off, ya);
      Load8<T>::get(dy + off + step, yb);
      const float ma = mean[row], ra = rstd[row], mb = mean[row + groups], rb = rstd[row + groups];
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        s1[i] += ya[i] + yb[i];
        s2[i] = fmaf(ya[i], (a[i] - ma) * ra, fmaf(yb[i], (b[i] - mb) * rb, s2[i]));
      }
    }
    for (; row < r1; row += groups, off += step) {
      float a[8], ya[8];
      Load8<T>::get(x + off, a);
      Load8<T>::get(dy + off, ya);
      const float ma = mean[row], ra = rstd[row];
#pragma unroll
      for (int i = 0; i < 8; ++i) { s1[i] += ya[i]; s2[i] = fmaf(ya[i], (a[i] - ma) * ra, s2[i]); }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      cs_sm[(rr * 2 + 0) * cols + 8 * cc + i] = s1[i];
      cs_sm[(rr * 2 + 1) * cols + 8 * cc + i] = s2[i];
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < 2 * cols; c += CS_THREADS) {
    const int which = c / cols, col = c - which * cols;
    float s = 0.f;
    for (int g = 0; g < groups; ++g) s += cs_sm[(g * 2 + which) * cols + col];      // fixed order
    partial[((size_t)blockIdx.x * 2 + which) * cols + col] = s;
  }
}

__global__ void __launch_bounds__(CF_THREADS)
k_ln_wgrad_final(const float* __restrict__ partial, int nparts, int cols, float* __restrict__ dgamma,
                 float* __restrict__ dbeta) {
  __shared__ float sm[CF_THREADS];
  const int c = blockIdx.x * CF_COLS + threadIdx.x % CF_COLS;
  const float s1 = cf_combine(partial, nparts, (size_t)2 * cols, c, cols, sm);
  const float s2 = cf_combine(partial + cols, nparts, (size_t)2 * cols, c, cols, sm);
  if (c >= cols || threadIdx.x >= CF_COLS) return;
  dbeta[c] = s1;
  dgamma[c] = s2;
}

// mean / rstd: one fp32 value per row (what the forward pass of layer norm saves).  partial: nparts * 2 * cols.
extern "C" int conef_ln_wgrad(const void* dy, const void* x, int dtype, long long rows, int cols, const float* mean,
                              const float* rstd, float* partial, int nparts, float* dgamma, float* dbeta,
                              cudaStream_t stream) {
  if (!colpair_ok(x, dy, rows, cols, nparts)) { conef_set_error("ln_wgrad: shape or alignment not supported"); return 2; }
  const long long rpc = (rows + nparts - 1) / nparts;
  const int groups = CS_THREADS / (cols >> 3);
  const size_t smem = (size_t)groups * 2 * cols * sizeof(float);
  if (smem > 48 * 1024) { conef_set_error("ln_wgrad: %d columns need too much shared memory", cols); return 2; }
  CONEF_BY_DTYPE(dtype, {
    k_ln_wgrad_partial<T><<<nparts, CS_THREADS, smem, stream>>>((const T*)dy, (const T*)x, mean, rstd, rows, cols, rpc, partial);
  });
  CONEF_CHECK_LAUNCH("k_ln_wgrad_partial");
  k_ln_wgrad_final<<<(cols + CF_COLS - 1) / CF_COLS, CF_THREADS, 0, stream>>>(partial, nparts, cols, dgamma, dbeta);
  CONEF_CHECK_LAUNCH("k_ln_wgrad_final");
  return 0;
}

// ---------------------------------------------------------------------------
// fp32 -> bf16 copy (the per-step casts of weights and activations under bf16 autocast).  PyTorch's copy kernel
// for this pair of types is not vectorised and runs at 0.5 TB/s (5 ms of a BERT-large step); here a thread moves
// eight values per pass with two 16-byte loads and one 16-byte store.
__global__ void __launch_bounds__(256)
k_cast_f32_bf16(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long n8 = n >> 3;
  const long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
    float v[8];
    Load8<float>::get(src + 8 * i, v);
    Store8<__nv_bfloat16>::put(dst + 8 * i, v);
  }
  if (blockIdx.x == 0 && threadIdx.x < (int)(n & 7)) {
    const long long i = (n8 << 3) + threadIdx.x;
    dst[i] = __float2bfloat16_rn(src[i]);
  }
}

extern "C" int conef_cast_f32_bf16(const float* src, void* dst, long long n, cudaStream_t stream) {
  if (n <= 0) return 0;
  if ((reinterpret_cast<uintptr_t>(src) & 15) != 0 || (reinterpret_cast<uintptr_t>(dst) & 15) != 0) {
    conef_set_error("cast: pointers must be 16-byte aligned");
    return 2;
  }
  long long blocks = ((n >> 3) + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks < 1) blocks = 1;
  k_cast_f32_bf16<<<(int)blocks, 256, 0, stream>>>(src, (__nv_bfloat16*)dst, n);
  CONEF_CHECK_LAUNCH("k_cast_f32_bf16");
  return 0;
}
