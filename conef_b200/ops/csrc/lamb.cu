// Multi-tensor LAMB: every parameter tensor of the model in three launches.
// Stands in for apex.optimizers.FusedLAMB, which the reference's BERT driver
// imports (examples/BertPretraining/run_pretraining_conef.py:42,449-450) and
// which is not available without apex.
//   launch 1: squared global gradient norm (for clipping)
//   launch 2: moments, update direction u = m_hat / (sqrt(v_hat) + eps) + wd * p,
//             written over the gradient; squared norms of p and u per tensor
//   launch 3: p -= lr * trust * u with trust = |p| / |u| (1 when either is 0)
#include "common.cuh"

constexpr int L_THREADS = 512;

__global__ void __launch_bounds__(L_THREADS)
k_lamb_gnorm(const ConefLambTensor* __restrict__ tensors, const int2* __restrict__ chunks, int chunk_elems,
             float* __restrict__ norms) {
  __shared__ float scratch[33];
  const int2 c = chunks[blockIdx.x];
  const ConefLambTensor T = tensors[c.x];
  const long long lo = (long long)c.y * chunk_elems;
  const long long hi = min(lo + (long long)chunk_elems, T.numel);
  float s = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += L_THREADS) { const float g = T.g[i]; s = fmaf(g, g, s); }
  s = block_sum(s, scratch);
  if (threadIdx.x == 0) atomicAdd(&norms[0], s);
}

__global__ void __launch_bounds__(L_THREADS)
k_lamb_stage1(const ConefLambTensor* __restrict__ tensors, const int2* __restrict__ chunks, int chunk_elems,
              float* __restrict__ norms, float beta1, float beta2, float eps, float bc1, float bc2,
              float grad_scale, float max_grad_norm) {
  __shared__ float scratch[33];
  const int2 c = chunks[blockIdx.x];
  const ConefLambTensor T = tensors[c.x];
  const long long lo = (long long)c.y * chunk_elems;
  const long long hi = min(lo + (long long)chunk_elems, T.numel);
  // gradient un-scaling and global-norm clipping folded into one factor
  float gmul = 1.f / grad_scale;
  if (max_grad_norm > 0.f) {
    const float gn = sqrtf(norms[0]) * gmul;
    if (gn > max_grad_norm) gmul *= max_grad_norm / gn;
  }
  float pn = 0.f, un = 0.f;
  for (long long i = lo + threadIdx.x; i < hi; i += L_THREADS) {
    const float g = T.g[i] * gmul;
    const float p = T.p[i];
    const float m = beta1 * T.m[i] + (1.f - beta1) * g;
    const float v = beta2 * T.v[i] + (1.f - beta2) * g * g;
    T.m[i] = m;
    T.v[i] = v;
    const float u = (m / bc1) / (sqrtf(v / bc2) + eps) + T.weight_decay * p;
    T.g[i] = u;
    pn = fmaf(p, p, pn);
    un = fmaf(u, u, un);
  }
  pn = block_sum(pn, scratch);
  un = block_sum(un, scratch);
  if (threadIdx.x == 0) {
    atomicAdd(&norms[1 + 2 * c.x], pn);
    atomicAdd(&norms[2 + 2 * c.x], un);
  }
}

__global__ void __launch_bounds__(L_THREADS)
k_lamb_stage2(const ConefLambTensor* __restrict__ tensors, const int2* __restrict__ chunks, int chunk_elems,
              const float* __restrict__ norms, float lr) {
  const int2 c = chunks[blockIdx.x];
  const ConefLambTensor T = tensors[c.x];
  const long long lo = (long long)c.y * chunk_elems;
  const long long hi = min(lo + (long long)chunk_elems, T.numel);
  const float pn = sqrtf(norms[1 + 2 * c.x]), un = sqrtf(norms[2 + 2 * c.x]);
  const float trust = (pn > 0.f && un > 0.f) ? pn / un : 1.f;
  const float step = lr * trust;
  for (long long i = lo + threadIdx.x; i < hi; i += L_THREADS) T.p[i] -= step * T.g[i];
}

extern "C" int conef_lamb_step(const ConefLambTensor* tensors, int ntensors, const int2* chunks, int nchunks,
                               int chunk_elems, float* norms, float lr, float beta1, float beta2, float eps,
                               int step, int bias_correction, float grad_scale, float max_grad_norm,
                               cudaStream_t stream) {
  if (ntensors <= 0 || nchunks <= 0) return 0;
  CONEF_CUDA(cudaMemsetAsync(norms, 0, sizeof(float) * (size_t)(1 + 2 * ntensors), stream));
  if (max_grad_norm > 0.f) {
    k_lamb_gnorm<<<nchunks, L_THREADS, 0, stream>>>(tensors, chunks, chunk_elems, norms);
    CONEF_CHECK_LAUNCH("k_lamb_gnorm");
  }
  float bc1 = 1.f, bc2 = 1.f;
  if (bias_correction) {
    bc1 = 1.f - powf(beta1, (float)step);
    bc2 = 1.f - powf(beta2, (float)step);
  }
  k_lamb_stage1<<<nchunks, L_THREADS, 0, stream>>>(tensors, chunks, chunk_elems, norms, beta1, beta2, eps, bc1, bc2,
                                                 grad_scale, max_grad_norm);
  CONEF_CHECK_LAUNCH("k_lamb_stage1");
  k_lamb_stage2<<<nchunks, L_THREADS, 0, stream>>>(tensors, chunks, chunk_elems, norms, lr);
  CONEF_CHECK_LAUNCH("k_lamb_stage2");
  return 0;
}

// ---------------------------------------------------------------------------
// Allocation-free variant (declared in conef_noalloc.h): the norm scratch lives in
// static device memory instead of a caller-provided buffer.
#include "conef_noalloc.h"

static __device__ __align__(256) float g_lamb_scratch[1 + 2 * CONEF_NOALLOC_MAX_TENSORS];

// In host code the array's name is only a handle; kernels need its device address,
// looked up once per device with that device current.
static float* g_lamb_scratch_addr[64] = {nullptr};

extern "C" int conef_lamb_step_noalloc(const ConefLambTensor* tensors, int ntensors, const int2* chunks,
                                       int nchunks, int chunk_elems, float lr, float beta1, float beta2,
                                       float eps, int step, int bias_correction, float grad_scale,
                                       float max_grad_norm, cudaStream_t stream) {
  if (ntensors <= 0 || nchunks <= 0) return 0;
  if (ntensors > CONEF_NOALLOC_MAX_TENSORS) {
    conef_set_error("conef_lamb_step_noalloc: %d tensors exceed the built-in scratch of %d tensors; "
                    "use conef_lamb_step with a caller-provided buffer", ntensors, CONEF_NOALLOC_MAX_TENSORS);
    return 2;
  }
  int dev = -1;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) { conef_set_error("conef_lamb_step_noalloc: unsupported device index %d", dev); return 2; }
  if (g_lamb_scratch_addr[dev] == nullptr) {
    float* addr = nullptr;
    CONEF_CUDA(cudaGetSymbolAddress((void**)&addr, g_lamb_scratch));
    g_lamb_scratch_addr[dev] = addr;
  }
  // the same memset and kernels as the entry point with a caller-provided buffer: the accumulators
  // this call uses are cleared first, the rest of the array keeps old values
  return conef_lamb_step(tensors, ntensors, chunks, nchunks, chunk_elems, g_lamb_scratch_addr[dev], lr, beta1, beta2,
                         eps, step, bias_correction, grad_scale, max_grad_norm, stream);
}

// ---------------------------------------------------------------------------
// Multi-tensor SGD with momentum: one launch over all tensors (the same tensor / chunk tables as LAMB; `v` is
// unused).  torch.optim.SGD semantics: g += weight_decay p; buf = first ? g : momentum buf + (1 - dampening) g;
// update = nesterov ? g + momentum buf : buf; p -= lr update.  PyTorch's foreach path is about fifteen launches
// and three passes over parameters, gradients and buffers; this is one pass (read p, g, buf; write p, buf).
__global__ void __launch_bounds__(L_THREADS)
k_sgd_step(const ConefLambTensor* __restrict__ tensors, const int2* __restrict__ chunks, int chunk_elems, float lr,
           float momentum, float dampening, int nesterov, int first) {
  const int2 c = chunks[blockIdx.x];
  const ConefLambTensor T = tensors[c.x];
  const long long lo = (long long)c.y * chunk_elems;
  const long long hi = min(lo + (long long)chunk_elems, T.numel);
  const float wd = T.weight_decay;
  const bool vec = ((reinterpret_cast<uintptr_t>(T.p) | reinterpret_cast<uintptr_t>(T.g) |
                     reinterpret_cast<uintptr_t>(T.m)) & 15) == 0 && (lo & 3) == 0;
  long long i = lo;
  if (vec) {
    const long long hi4 = lo + ((hi - lo) & ~3LL);
    for (i = lo + 4LL * threadIdx.x; i < hi4; i += 4LL * L_THREADS) {
      float4 p = *reinterpret_cast<const float4*>(T.p + i);
      const float4 g4 = *reinterpret_cast<const float4*>(T.g + i);
      float4 b = momentum != 0.f && !first ? *reinterpret_cast<const float4*>(T.m + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      float* pp = reinterpret_cast<float*>(&p);
      const float* gp = reinterpret_cast<const float*>(&g4);
      float* bp = reinterpret_cast<float*>(&b);
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float g = fmaf(wd, pp[k], gp[k]);
        float u = g;
        if (momentum != 0.f) {
          bp[k] = first ? g : fmaf(momentum, bp[k], (1.f - dampening) * g);
          u = nesterov ? fmaf(momentum, bp[k], g) : bp[k];
        }
        pp[k] = fmaf(-lr, u, pp[k]);
      }
      *reinterpret_cast<float4*>(T.p + i) = p;
      if (momentum != 0.f) *reinterpret_cast<float4*>(T.m + i) = b;
    }
    i = hi4;
  }
  for (i += threadIdx.x; i < hi; i += L_THREADS) {
    const float g = fmaf(wd, T.p[i], T.g[i]);
    float u = g;
    if (momentum != 0.f) {
      const float b = first ? g : fmaf(momentum, T.m[i], (1.f - dampening) * g);
      T.m[i] = b;
      u = nesterov ? fmaf(momentum, b, g) : b;
    }
    T.p[i] = fmaf(-lr, u, T.p[i]);
  }
}

extern "C" int conef_sgd_step(const ConefLambTensor* tensors, int ntensors, const int2* chunks, int nchunks,
                              int chunk_elems, float lr, float momentum, float dampening, int nesterov, int first,
                              cudaStream_t stream) {
  if (ntensors <= 0 || nchunks <= 0) return 0;
  k_sgd_step<<<nchunks, L_THREADS, 0, stream>>>(tensors, chunks, chunk_elems, lr, momentum, dampening, nesterov, first);
  CONEF_CHECK_LAUNCH("k_sgd_step");
  return 0;
}
