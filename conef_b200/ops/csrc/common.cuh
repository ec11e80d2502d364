// Shared device / host helpers for the conef_b200 kernels.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "conef.h"

void conef_set_error(const char* fmt, ...);

#define CONEF_CHECK_LAUNCH(name)                                              \
  do {                                                                        \
    cudaError_t e__ = cudaGetLastError();                                     \
    if (e__ != cudaSuccess) {                                                 \
      conef_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
      return 1;                                                               \
    }                                                                         \
  } while (0)

#define CONEF_CUDA(call)                                                      \
  do {                                                                        \
    cudaError_t e__ = (call);                                                 \
    if (e__ != cudaSuccess) {                                                 \
      conef_set_error("%s failed: %s", #call, cudaGetErrorString(e__));       \
      return 1;                                                               \
    }                                                                         \
  } while (0)

// Error codes written into the device status word by kernels whose waits ran out.
enum {
  CONEF_STATUS_OK = 0,
  CONEF_STATUS_FLAG_TIMEOUT = 1,      // a peer never published the expected epoch
  CONEF_STATUS_MBAR_TIMEOUT = 2,      // an mbarrier phase never completed
  CONEF_STATUS_BAD_ARG = 3,
};

// Reference hash on signed 32-bit ints, done in uint32 so nothing overflows in
// C++: wrapping multiply, explicit arithmetic shift, non-negative remainder.
__host__ __device__ __forceinline__ uint32_t conef_sar(uint32_t h, int s) {
  return (uint32_t)(((int32_t)h) >> s);  // arithmetic shift on every supported compiler
}
__host__ __device__ __forceinline__ int conef_hash(int value, int range, int a, int b) {
  uint32_t h = (uint32_t)a * (uint32_t)value + (uint32_t)b;
  h ^= conef_sar(h, 16);
  h *= 0x85ebca6bu;
  h ^= conef_sar(h, 13);
  h *= 0xc2b2ae35u;
  h ^= conef_sar(h, 16);   // sign bit is cleared here (x ^ (x >>arith 16) has a zero top bit)
  return (int)(h % (uint32_t)range);
}

// Cell of column j.  layout 0: the reference's per-element hash.  layout 1 (sketch rows of at least
// CONEF_BLOCK_MIN_WIDTH cells): columns are hashed in aligned groups of 32 and the groups in windows of
// nb = W / 32 consecutive groups.  Inside a window a pseudo-random permutation (the rank of
// hash(g, 2^30) among the window's nb group numbers, ties by group number) gives every group a cell
// block of its own, u_g; column 32 g + k goes to cell 32 u_g + (k xor x_g), x_g = hash(g, 32).  The 32
// columns a warp handles together then fall into 32 different shared-memory banks, every cell block
// receives exactly one group per window, and a warp that walks the groups of one cell block keeps
// the block's 32 sums in registers.  O(nb) per call: meant for building tables.
#define CONEF_BLOCK_MIN_WIDTH 64
__host__ __device__ __forceinline__ int conef_cell(int j, int W, int a, int b, int layout) {
  if (layout == 1 && W >= CONEF_BLOCK_MIN_WIDTH) {
    const int nb = W >> 5, g = j >> 5;
    const int g0 = (g / nb) * nb;
    const int key = conef_hash(g, 1 << 30, a, b);
    int u = 0;
    for (int k = 0; k < nb; ++k) {
      const int other = conef_hash(g0 + k, 1 << 30, a, b);
      u += (other < key || (other == key && g0 + k < g)) ? 1 : 0;
    }
    return 32 * u + ((j & 31) ^ conef_hash(g, 32, a + 11, b + 13));
  }
  return conef_hash(j, W, a, b);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum of `v`; every thread gets the result.  `scratch` holds 33 floats.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarps = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarps ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

__device__ __forceinline__ float unpack_sign(int e) { return e < 0 ? 1.f : -1.f; }
__device__ __forceinline__ int unpack_bucket(int e) { return e & 0x7fffffff; }

// System-scope acquire load / release store for flags other GPUs write.
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_acquire_gpu(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ float ld_relaxed_sys_f32(const float* p) {
  float v;
  asm volatile("ld.relaxed.sys.global.f32 %0, [%1];" : "=f"(v) : "l"(p) : "memory");
  return v;
}

// Wait until flags[0..world) have all reached `epoch` (wrap-safe compare), at
// most `limit` polls per flag.  Returns false when a wait ran out; the caller
// records the failure and carries on without touching peer data.
__device__ __forceinline__ bool wait_flags_bounded(const uint32_t* flags, int world, uint32_t epoch,
                                                   long long limit) {
  for (int p = 0; p < world; ++p) {
    long long n = 0;
    while ((int32_t)(ld_acquire_sys(flags + p) - epoch) < 0) {
      if (++n > limit) return false;
      __nanosleep(64);
    }
  }
  return true;
}

// Offset (in floats) of element (k, n) of a small operand inside its packed copy: per K step
// of 8 rows, NP/8 groups of 8 columns, each two 8x4 core matrices (k%8 < 4, k%8 >= 4) of
// 32 floats: K-major, no swizzle, exactly what tcgen05.mma reads for a K=8 tf32 step.
__host__ __device__ __forceinline__ long long conef_packed_offset(long long k, int n, int np) {
  return (k >> 3) * (np * 8) + (n >> 3) * 64 + ((k & 7) >> 2) * 32 + (n & 7) * 4 + (k & 3);
}

// Store element (row, c) of a small factor (which = 0: P block, 1: Q block) into the packed copies the
// tensor-core kernel reads, including the folded ones (see ConefMat::fold).
__device__ __forceinline__ void conef_pack_store(float* __restrict__ packed, const ConefMat& M, int which,
                                                 long long row, int c, float v, int np) {
  if (which == 1) {
    if (M.fold > 1) {
      for (int b = 0; b < M.fold; ++b)
        packed[M.qpk_off + conef_packed_offset((long long)b * M.m + row, b * M.r + c, np)] = v;
    } else {
      packed[M.qpk_off + conef_packed_offset(row, c, np)] = v;
    }
  } else {
    packed[M.ppk_off + conef_packed_offset(row, c, np)] = v;
    if (M.fold > 1)
      packed[M.ppk_fold_off + conef_packed_offset(row / M.fold, (int)(row % M.fold) * M.r + c, np)] = v;
  }
}

// "The CTA that finishes last tells the peers": a kernel whose output a peer-memory reduction
// consumes publishes the epoch itself instead of leaving that to a launch of its own.  `done`
// counts finished CTAs and is zero between launches.  Call from every CTA, all threads, after the
// CTA's last global write.  All-zero struct: nothing is published.
struct ConefPublish {
  uint32_t* done;
  uint32_t* const* peer_flags;
  const uint32_t* epoch_base;     // nullable device word added to `epoch` (replayed launches)
  uint32_t epoch;
  int world, rank;
};
__device__ __forceinline__ void conef_publish_if_last(const ConefPublish& s, unsigned ncta) {
  if (s.done == nullptr) return;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();                                   // this CTA's results, then the counter
    if (atomicAdd(s.done, 1u) == ncta - 1) {
      atomicExch(s.done, 0u);
      __threadfence_system();                          // everything counted above, then the flags
      const uint32_t epoch = s.epoch + (s.epoch_base != nullptr ? *s.epoch_base : 0u);
      for (int p = 0; p < s.world; ++p) st_release_sys(s.peer_flags[p] + s.rank, epoch);
    }
  }
}

// cp.async into / loads from shared memory at a shared-space address plus an immediate offset
template <int OFF>
__device__ __forceinline__ void cp_async_f32(uint32_t dst, const void* gmem_src) {
  asm volatile("cp.async.ca.shared.global [%0+%2], [%1], 4;" ::"r"(dst), "l"(gmem_src), "n"(OFF) : "memory");
}
template <int OFF>
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* gmem_src) {
  asm volatile("cp.async.cg.shared.global [%0+%2], [%1], 16;" ::"r"(dst), "l"(gmem_src), "n"(OFF) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
template <int OFF>
__device__ __forceinline__ float lds_f32(uint32_t src) {
  float v;
  asm volatile("ld.shared.f32 %0, [%1+%2];" : "=f"(v) : "r"(src), "n"(OFF) : "memory");
  return v;
}
template <int OFF>
__device__ __forceinline__ float4 lds_f32x4(uint32_t src) {
  float4 v;
  asm volatile("ld.shared.v4.f32 {%0, %1, %2, %3}, [%4+%5];"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(src), "n"(OFF) : "memory");
  return v;
}

// Philox-4x32-10 keyed by `seed` at counter `ctr`, turned into four standard normal values by
// Box-Muller: a pure function of (seed, ctr), so every rank draws the same numbers.
__device__ __forceinline__ void conef_philox_round(uint32_t& c0, uint32_t& c1, uint32_t& c2, uint32_t& c3,
                                                   uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u;
  const uint32_t hi0 = __umulhi(M0, c0), lo0 = M0 * c0;
  const uint32_t hi1 = __umulhi(M1, c2), lo1 = M1 * c2;
  const uint32_t n0 = hi1 ^ c1 ^ k0, n1 = lo1, n2 = hi0 ^ c3 ^ k1, n3 = lo0;
  c0 = n0; c1 = n1; c2 = n2; c3 = n3;
}
__device__ __forceinline__ void conef_philox_normal4(uint64_t seed, uint64_t ctr, float (&out)[4]) {
  uint32_t c0 = (uint32_t)ctr, c1 = (uint32_t)(ctr >> 32), c2 = 0u, c3 = 0u;
  uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
#pragma unroll
  for (int i = 0; i < 10; ++i) {
    conef_philox_round(c0, c1, c2, c3, k0, k1);
    k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
  }
  const float two_pi = 6.283185307179586f;
  const float u0 = ((float)c0 + 1.f) * 2.3283064365386963e-10f;  // (0, 1]
  const float u1 = (float)c1 * 2.3283064365386963e-10f;
  const float u2 = ((float)c2 + 1.f) * 2.3283064365386963e-10f;
  const float u3 = (float)c3 * 2.3283064365386963e-10f;
  const float r0 = sqrtf(-2.f * logf(u0)), r1 = sqrtf(-2.f * logf(u2));
  out[0] = r0 * cosf(two_pi * u1); out[1] = r0 * sinf(two_pi * u1);
  out[2] = r1 * cosf(two_pi * u3); out[3] = r1 * sinf(two_pi * u3);
}

