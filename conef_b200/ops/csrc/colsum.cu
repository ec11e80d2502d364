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

__global__ void k_colsum_final(const float* __restrict__ partial, int nparts, int cols, float* __restrict__ out) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= cols) return;
  float s = 0.f;
  int p = 0;
  for (; p + 8 <= nparts; p += 8) {      // eight loads in flight, fixed order of the additions
    float v[8];
#pragma unroll
    for (int u = 0; u < 8; ++u) v[u] = partial[(size_t)(p + u) * cols + c];
#pragma unroll
    for (int u = 0; u < 8; ++u) s += v[u];
  }
  for (; p < nparts; ++p) s += partial[(size_t)p * cols + c];
  out[c] = s;
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
  k_colsum_final<<<(cols + 127) / 128, 128, 0, stream>>>(partial, nparts, cols, out);
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
