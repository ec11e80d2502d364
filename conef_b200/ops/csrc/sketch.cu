// Count-sketch error compressor kernels: column hash table, query and update
// for the single-row sketch (fp32 or fp16 storage) and the three-row median
// sketch.  Behaviour follows the reference's NVRTC kernels
// (communication/compressors/CountSketch.py:27-98, CountSketchHash3.py:27-147,
// halfCountSketch.py:27-106) with these differences: the hash is evaluated
// once per column into a table instead of once per element, a CTA owns whole
// sketch rows so accumulation happens with shared-memory atomics followed by
// one plain global store per sketch cell, and fp16 sketches are read and
// written directly instead of being up-cast around every launch.
#include <cuda_fp16.h>
#include <stdarg.h>
#include <string.h>
#include "common.cuh"

static thread_local char g_err[512] = "";
void conef_set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
extern "C" const char* conef_last_error(void) { return g_err; }
extern "C" int conef_version(void) { return 100; }

// ---------------------------------------------------------------------------
__global__ void k_hash_table(int32_t* __restrict__ table, int32_t* __restrict__ counts, int D, int W,
                             int a, int b, int sa, int sb, int layout) {
  int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= D) return;
  int h = conef_cell(j, W, a, b, layout);
  int sign_bit = conef_hash(j, W, a + sa, b + sb) & 1;
  table[j] = (int32_t)((uint32_t)h | ((uint32_t)sign_bit << 31));
  if (counts) atomicAdd(&counts[h], 1);
}

extern "C" int conef_build_hash_table(int32_t* table, int32_t* counts, int D, int W, int a, int b,
                                      int sa, int sb, int layout, cudaStream_t stream) {
  if (D <= 0 || W <= 0) { conef_set_error("hash table: bad D=%d W=%d", D, W); return 1; }
  if (counts) CONEF_CUDA(cudaMemsetAsync(counts, 0, sizeof(int32_t) * (size_t)W, stream));
  k_hash_table<<<(D + 255) / 256, 256, 0, stream>>>(table, counts, D, W, a, b, sa, sb, layout);
  CONEF_CHECK_LAUNCH("k_hash_table");
  return 0;
}

// ---------------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float ld_cs(const T* p);
template <> __device__ __forceinline__ float ld_cs<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld_cs<__half>(const __half* p) { return __half2float(*p); }
template <typename T> __device__ __forceinline__ void st_cs(T* p, float v);
template <> __device__ __forceinline__ void st_cs<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void st_cs<__half>(__half* p, float v) { *p = __float2half_rn(v); }

constexpr int SK_ROWS = 4;  // rows per CTA in the query kernel

template <typename T>
__global__ void k_sketch_query(float* __restrict__ mat, const T* __restrict__ cs,
                               const int32_t* __restrict__ table, int N, int D, int W, float alpha) {
  const int row0 = blockIdx.x * SK_ROWS;
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const int e = table[j];
    const int h = unpack_bucket(e);
    const float s = unpack_sign(e) * alpha;
#pragma unroll
    for (int ii = 0; ii < SK_ROWS; ++ii) {
      const int row = row0 + ii;
      if (row < N) mat[(size_t)row * D + j] += s * ld_cs<T>(cs + (size_t)row * W + h);
    }
  }
}

extern "C" int conef_sketch_query(float* mat, const void* cs, int cs_is_half, const int32_t* table,
                                  int N, int D, int W, float alpha, cudaStream_t stream) {
  if (N <= 0 || D <= 0) return 0;
  const int grid = (N + SK_ROWS - 1) / SK_ROWS;
  if (cs_is_half)
    k_sketch_query<__half><<<grid, 256, 0, stream>>>(mat, (const __half*)cs, table, N, D, W, alpha);
  else
    k_sketch_query<float><<<grid, 256, 0, stream>>>(mat, (const float*)cs, table, N, D, W, alpha);
  CONEF_CHECK_LAUNCH("k_sketch_query");
  return 0;
}

// cs[row, h] <- cs[row, h] * (1 - (1-beta) * count[h]) + sum_{j -> h} s_j vec[row, j]
template <typename T>
__global__ void k_sketch_update(const float* __restrict__ vec, T* __restrict__ cs,
                                const int32_t* __restrict__ table, const int32_t* __restrict__ counts,
                                int N, int D, int W, float beta, int rows_per_cta) {
  extern __shared__ float acc[];  // rows_per_cta * W
  const int row0 = blockIdx.x * rows_per_cta;
  const int rows = min(rows_per_cta, N - row0);
  for (int i = threadIdx.x; i < rows * W; i += blockDim.x) acc[i] = 0.f;
  __syncthreads();
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const int e = table[j];
    const int h = unpack_bucket(e);
    const float s = unpack_sign(e);
    for (int ii = 0; ii < rows; ++ii)
      atomicAdd(&acc[ii * W + h], s * vec[(size_t)(row0 + ii) * D + j]);
  }
  __syncthreads();
  const float omb = 1.f - beta;
  for (int i = threadIdx.x; i < rows * W; i += blockDim.x) {
    const int ii = i / W, h = i - ii * W;
    T* cell = cs + (size_t)(row0 + ii) * W + h;
    st_cs<T>(cell, ld_cs<T>(cell) * (1.f - omb * (float)counts[h]) + acc[i]);
  }
}

static int pick_rows_per_cta(int W, int words_per_row_cell, int max_rows, size_t* smem_out) {
  // Shared memory needed is rows * W * words * 4 bytes; stay below 200 KB.
  const size_t budget = 200 * 1024;
  size_t per_row = (size_t)W * words_per_row_cell * sizeof(float);
  if (per_row > budget) return 0;
  int rows = (int)(budget / per_row);
  if (rows > max_rows) rows = max_rows;
  *smem_out = per_row * rows;
  return rows;
}

extern "C" int conef_sketch_update(const float* vec, void* cs, int cs_is_half, const int32_t* table,
                                   const int32_t* counts, int N, int D, int W, float beta,
                                   cudaStream_t stream) {
  if (N <= 0 || D <= 0) return 0;
  size_t smem = 0;
  const int rows = pick_rows_per_cta(W, 1, 8, &smem);
  if (rows == 0) { conef_set_error("sketch_update: W=%d does not fit in shared memory", W); return 2; }
  const int grid = (N + rows - 1) / rows;
  if (cs_is_half) {
    CONEF_CUDA(cudaFuncSetAttribute(k_sketch_update<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_sketch_update<__half><<<grid, 256, smem, stream>>>(vec, (__half*)cs, table, counts, N, D, W, beta, rows);
  } else {
    CONEF_CUDA(cudaFuncSetAttribute(k_sketch_update<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    k_sketch_update<float><<<grid, 256, smem, stream>>>(vec, (float*)cs, table, counts, N, D, W, beta, rows);
  }
  CONEF_CHECK_LAUNCH("k_sketch_update");
  return 0;
}

// ---------------------------------------------------------------------------
// three hash rows, median-of-three estimator
__device__ __forceinline__ float median3(float a, float b, float c) {
  return fmaxf(fminf(a, b), fminf(fmaxf(a, b), c));
}

__global__ void k_sketch3_query(float* __restrict__ mat, const float* __restrict__ cs0,
                                const float* __restrict__ cs1, const float* __restrict__ cs2,
                                const int32_t* __restrict__ t0, const int32_t* __restrict__ t1,
                                const int32_t* __restrict__ t2, int N, int D, int W, float alpha) {
  const int row0 = blockIdx.x * SK_ROWS;
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const int e0 = t0[j], e1 = t1[j], e2 = t2[j];
#pragma unroll
    for (int ii = 0; ii < SK_ROWS; ++ii) {
      const int row = row0 + ii;
      if (row >= N) break;
      const size_t base = (size_t)row * W;
      const float a = alpha * unpack_sign(e0) * cs0[base + unpack_bucket(e0)];
      const float b = alpha * unpack_sign(e1) * cs1[base + unpack_bucket(e1)];
      const float c = alpha * unpack_sign(e2) * cs2[base + unpack_bucket(e2)];
      mat[(size_t)row * D + j] += median3(a, b, c);
    }
  }
}

extern "C" int conef_sketch3_query(float* mat, const float* cs0, const float* cs1, const float* cs2,
                                   const int32_t* t0, const int32_t* t1, const int32_t* t2, int N,
                                   int D, int W, float alpha, cudaStream_t stream) {
  if (N <= 0 || D <= 0) return 0;
  k_sketch3_query<<<(N + SK_ROWS - 1) / SK_ROWS, 256, 0, stream>>>(mat, cs0, cs1, cs2, t0, t1, t2, N, D, W, alpha);
  CONEF_CHECK_LAUNCH("k_sketch3_query");
  return 0;
}

// One CTA per matrix row.  Shared memory: old[3][W] then acc[3][W].
__global__ void k_sketch3_update(const float* __restrict__ vec, float* __restrict__ cs0,
                                 float* __restrict__ cs1, float* __restrict__ cs2,
                                 const int32_t* __restrict__ t0, const int32_t* __restrict__ t1,
                                 const int32_t* __restrict__ t2, int N, int D, int W, float beta) {
  extern __shared__ float sm[];
  float* old = sm;
  float* acc = sm + 3 * (size_t)W;
  const int row = blockIdx.x;
  const size_t base = (size_t)row * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    old[i] = cs0[base + i];
    old[W + i] = cs1[base + i];
    old[2 * W + i] = cs2[base + i];
    acc[i] = 0.f; acc[W + i] = 0.f; acc[2 * W + i] = 0.f;
  }
  __syncthreads();
  const float k = -(1.f - beta);
  for (int j = threadIdx.x; j < D; j += blockDim.x) {
    const int e0 = t0[j], e1 = t1[j], e2 = t2[j];
    const int h0 = unpack_bucket(e0), h1 = unpack_bucket(e1), h2 = unpack_bucket(e2);
    const float s0 = unpack_sign(e0), s1 = unpack_sign(e1), s2 = unpack_sign(e2);
    const float u = median3(k * s0 * old[h0], k * s1 * old[W + h1], k * s2 * old[2 * W + h2]) +
                    vec[(size_t)row * D + j];
    atomicAdd(&acc[h0], s0 * u);
    atomicAdd(&acc[W + h1], s1 * u);
    atomicAdd(&acc[2 * W + h2], s2 * u);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    cs0[base + i] = old[i] + acc[i];
    cs1[base + i] = old[W + i] + acc[W + i];
    cs2[base + i] = old[2 * W + i] + acc[2 * W + i];
  }
}

extern "C" int conef_sketch3_update(const float* vec, float* cs0, float* cs1, float* cs2,
                                    const int32_t* t0, const int32_t* t1, const int32_t* t2, int N,
                                    int D, int W, float beta, cudaStream_t stream) {
  if (N <= 0 || D <= 0) return 0;
  const size_t smem = (size_t)W * 6 * sizeof(float);
  if (smem > 200 * 1024) { conef_set_error("sketch3_update: W=%d does not fit in shared memory", W); return 2; }
  CONEF_CUDA(cudaFuncSetAttribute(k_sketch3_update, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  k_sketch3_update<<<N, 256, smem, stream>>>(vec, cs0, cs1, cs2, t0, t1, t2, N, D, W, beta);
  CONEF_CHECK_LAUNCH("k_sketch3_update");
  return 0;
}

// ---------------------------------------------------------------------------
// The sparse sign matrix H (m x W, one entry per row: H[j, h_j] = s_j) applied to the
// small PowerSGD factors, grouped over the matrices of a bucket.  With the sketch S,
//   unsketch(S) Q   = S (H^T Q)      -> k_sketch_project   : Z[h, :] += scale * s_j * Q[j, :]
//   unsketch(S)^T P = H (S^T P)      -> k_sketch_unproject : Q[j, :] += scale * s_j * Y[h_j, :]
// Z and Y are (W x r) blocks stored behind the Q blocks of the same flat buffer: record
// nmats + i of the table describes the sketch of matrix i and its q_off points there.
__global__ void k_sketch_project(const ConefMat* __restrict__ mats, int nmats, const int32_t* __restrict__ tables,
                                 float* __restrict__ qz, float scale) {
  const ConefMat M = mats[blockIdx.y];
  const ConefMat E = mats[nmats + blockIdx.y];
  const int r = M.r;
  const int32_t* tab = tables + M.tab_off;
  const float* q = qz + M.q_off;
  float* z = qz + E.q_off;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < M.m; j += gridDim.x * blockDim.x) {
    const int e = tab[j];
    const float s = unpack_sign(e) * scale;
    float* zr = z + (size_t)unpack_bucket(e) * r;
    for (int c = 0; c < r; ++c) atomicAdd(zr + c, s * q[(size_t)j * r + c]);
  }
}

__global__ void k_sketch_unproject(const ConefMat* __restrict__ mats, int nmats, const int32_t* __restrict__ tables,
                                   float* __restrict__ qy, float scale) {
  const ConefMat M = mats[blockIdx.y];
  const ConefMat E = mats[nmats + blockIdx.y];
  const int r = M.r;
  const int32_t* tab = tables + M.tab_off;
  float* q = qy + M.q_off;
  const float* y = qy + E.q_off;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < M.m; j += gridDim.x * blockDim.x) {
    const int e = tab[j];
    const float s = unpack_sign(e) * scale;
    const float* yr = y + (size_t)unpack_bucket(e) * r;
    for (int c = 0; c < r; ++c) q[(size_t)j * r + c] += s * yr[c];
  }
}

// All-reduce of Q fused with the un-projection of the sketch term:
//   Q[j, :] = scale * sum over peers p of ( Q_p[j, :] + alpha s_j Y_p[h_j, :] )
// where every peer buffer holds [Q blocks | Y blocks] as its Q = M^T P pass left them
// (Y_p = S_p^T P, record nmats + i).  The peers' values come over NVLink as plain loads, summed in
// rank order (bit-identical on every rank), after a bounded wait for the epoch their Q pass
// published.  tables == NULL: plain sum of the Q blocks.  world == 1: peer_bufs[0] is this GPU's own
// buffer and nothing is waited for.
__global__ void __launch_bounds__(256)
k_reduce_q(const ConefMat* __restrict__ mats, int nmats, const int32_t* __restrict__ tables, float* __restrict__ out,
           const float* const* __restrict__ peer_bufs, const uint32_t* __restrict__ my_flags, int world,
           uint32_t epoch, float alpha, float scale, int* __restrict__ status, long long spin_limit,
           const uint32_t* __restrict__ epoch_base) {
  __shared__ int ok;
  if (world > 1) {
    if (threadIdx.x == 0) {
      if (epoch_base != nullptr) epoch += *epoch_base;
      ok = wait_flags_bounded(my_flags, world, epoch, spin_limit) ? 1 : 0;
      if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
    }
    __syncthreads();
    if (!ok) return;
  }
  const ConefMat M = mats[blockIdx.y];
  const int r = M.r;
  const bool sk = tables != nullptr && M.tab_off >= 0;
  const int32_t* tab = sk ? tables + M.tab_off : nullptr;
  const long long y_off = sk ? mats[nmats + blockIdx.y].q_off : 0;
  const bool vec = (r & 3) == 0 && ((M.q_off | y_off) & 3) == 0;
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < M.m; j += gridDim.x * blockDim.x) {
    float s = 0.f;
    long long h = 0;
    if (sk) { const int e = tab[j]; s = unpack_sign(e) * alpha; h = unpack_bucket(e); }
    const long long qo = M.q_off + (long long)j * r, yo = y_off + h * r;
    if (vec) {
      for (int c = 0; c < r; c += 4) {
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int p = 0; p < world; ++p) {
          float4 v;
          asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                       : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(peer_bufs[p] + qo + c) : "memory");
          if (sk) {
            float4 y;
            asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                         : "=f"(y.x), "=f"(y.y), "=f"(y.z), "=f"(y.w) : "l"(peer_bufs[p] + yo + c) : "memory");
            v.x = fmaf(s, y.x, v.x); v.y = fmaf(s, y.y, v.y); v.z = fmaf(s, y.z, v.z); v.w = fmaf(s, y.w, v.w);
          }
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        *reinterpret_cast<float4*>(out + qo + c) = make_float4(acc.x * scale, acc.y * scale, acc.z * scale, acc.w * scale);
      }
    } else {
      for (int c = 0; c < r; ++c) {
        float acc = 0.f;
        for (int p = 0; p < world; ++p) {
          float v = ld_relaxed_sys_f32(peer_bufs[p] + qo + c);
          if (sk) v = fmaf(s, ld_relaxed_sys_f32(peer_bufs[p] + yo + c), v);
          acc += v;
        }
        out[qo + c] = acc * scale;
      }
    }
  }
}

extern "C" int conef_reduce_q(const ConefMat* mats, int nmats, int max_cols, const int32_t* tables, float* out,
                              const float* const* peer_bufs, const uint32_t* my_flags, int world, uint32_t epoch,
                              float alpha, float scale, int* status, long long spin_limit,
                              const uint32_t* epoch_base, cudaStream_t stream) {
  if (nmats <= 0) return 0;
  if (((uintptr_t)out & 15) != 0) { conef_set_error("reduce_q: output must be 16-byte aligned"); return 2; }
  int bx = (max_cols + 255) / 256;
  if (bx < 1) bx = 1;
  if (bx > 32) bx = 32;
  dim3 grid(bx, nmats);
  k_reduce_q<<<grid, 256, 0, stream>>>(mats, nmats, tables, out, peer_bufs, my_flags, world, epoch, alpha, scale,
                                      status, spin_limit, epoch_base);
  CONEF_CHECK_LAUNCH("k_reduce_q");
  return 0;
}

extern "C" int conef_sketch_project(const ConefMat* mats, int nmats, int max_cols, const int32_t* tables,
                                    float* qz, float scale, int unproject, cudaStream_t stream) {
  if (nmats <= 0) return 0;
  int bx = (max_cols + 255) / 256;
  if (bx < 1) bx = 1;
  if (bx > 32) bx = 32;
  dim3 grid(bx, nmats);
  if (unproject) k_sketch_unproject<<<grid, 256, 0, stream>>>(mats, nmats, tables, qz, scale);
  else k_sketch_project<<<grid, 256, 0, stream>>>(mats, nmats, tables, qz, scale);
  CONEF_CHECK_LAUNCH("k_sketch_project");
  return 0;
}
