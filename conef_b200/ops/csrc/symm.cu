// Collectives issued from inside our own kernels over NVLink peer memory.
//
// Every rank owns one buffer of a symmetric allocation (same size and layout
// on every GPU) and can address every peer's buffer directly.  A reduction is
// "one shot": a rank publishes an epoch number into slot `rank` of every
// peer's flag array once its data is written, waits (bounded) until all slots
// of its own flag array reached that epoch, then loads the peers' values in
// rank order and sums them, so every rank obtains bit-identical results.
// Epochs only grow, so flags are never reset; buffers are double-buffered by
// the caller (a rank can be at most one phase ahead of its slowest peer).
//
// These replace the reference's dist.all_reduce calls on the P / Q / staging
// buffers (communication/powerSGD_hook.py:503-505,517-523,539-545;
// communication/RandomBlock_hook.py:250-252,263-269).  Plain peer loads and
// stores only: no TMA, no cluster multicast.
#include <string.h>
#include "common.cuh"

// epoch_base (nullable): a device word added to `epoch`, so that a captured launch can be
// replayed with an epoch that advances on the device.
__global__ void k_signal_peers(uint32_t* const* __restrict__ peer_flags, int world, int rank, uint32_t epoch,
                               const uint32_t* __restrict__ epoch_base) {
  if (epoch_base != nullptr) epoch += *epoch_base;
  // Everything the preceding kernels of this stream wrote must be visible to
  // the peers before the flag: fence at system scope, then release-store.
  __threadfence_system();
  const int p = threadIdx.x;
  if (p < world) st_release_sys(peer_flags[p] + rank, epoch);
}

extern "C" int conef_signal_peers_ex(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                                     const uint32_t* epoch_base, cudaStream_t stream) {
  if (world <= 1) return 0;
  k_signal_peers<<<1, 32, 0, stream>>>(peer_flags, world, rank, epoch, epoch_base);
  CONEF_CHECK_LAUNCH("k_signal_peers");
  return 0;
}

extern "C" int conef_signal_peers(uint32_t* const* peer_flags, int world, int rank, uint32_t epoch,
                                  cudaStream_t stream) {
  return conef_signal_peers_ex(peer_flags, world, rank, epoch, nullptr, stream);
}

__global__ void k_wait_flags(const uint32_t* __restrict__ my_flags, int world, uint32_t epoch,
                             int* __restrict__ status, long long spin_limit,
                             const uint32_t* __restrict__ epoch_base) {
  if (epoch_base != nullptr) epoch += *epoch_base;
  if (threadIdx.x == 0 && !wait_flags_bounded(my_flags, world, epoch, spin_limit))
    atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
}

extern "C" int conef_wait_flags_ex(const uint32_t* my_flags, int world, uint32_t epoch, int* status,
                                   long long spin_limit, const uint32_t* epoch_base, cudaStream_t stream) {
  k_wait_flags<<<1, 32, 0, stream>>>(my_flags, world, epoch, status, spin_limit, epoch_base);
  CONEF_CHECK_LAUNCH("k_wait_flags");
  return 0;
}

extern "C" int conef_wait_flags(const uint32_t* my_flags, int world, uint32_t epoch, int* status,
                                long long spin_limit, cudaStream_t stream) {
  return conef_wait_flags_ex(my_flags, world, epoch, status, spin_limit, nullptr, stream);
}

// signal + wait + reduce in one kernel.  Block 0 publishes the epoch; every
// block waits on the local flag array before touching peer data.
__global__ void __launch_bounds__(256)
k_allreduce_oneshot(float* __restrict__ out, const float* const* __restrict__ peer_bufs,
                    uint32_t* const* __restrict__ peer_flags, const uint32_t* __restrict__ my_flags,
                    int world, int rank, uint32_t epoch, long long numel, float scale,
                    int* __restrict__ status, long long spin_limit, const uint32_t* __restrict__ epoch_base) {
  __shared__ int ok;
  if (epoch_base != nullptr) epoch += *epoch_base;
  if (blockIdx.x == 0 && threadIdx.x < world && peer_flags != nullptr) {
    __threadfence_system();
    st_release_sys(peer_flags[threadIdx.x] + rank, epoch);
  }
  if (threadIdx.x == 0) {
    ok = wait_flags_bounded(my_flags, world, epoch, spin_limit) ? 1 : 0;
    if (!ok) atomicExch(status, CONEF_STATUS_FLAG_TIMEOUT);
  }
  __syncthreads();
  if (!ok) return;
  const long long stride = (long long)gridDim.x * blockDim.x;
  const long long n4 = numel >> 2;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int p = 0; p < world; ++p) {
      float4 v;
      asm volatile("ld.relaxed.sys.global.v4.f32 {%0,%1,%2,%3}, [%4];"
                   : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                   : "l"(reinterpret_cast<const float4*>(peer_bufs[p]) + i) : "memory");
      s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    s.x *= scale; s.y *= scale; s.z *= scale; s.w *= scale;
    reinterpret_cast<float4*>(out)[i] = s;
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < numel; i += stride) {
    float s = 0.f;
    for (int p = 0; p < world; ++p) s += ld_relaxed_sys_f32(peer_bufs[p] + i);
    out[i] = s * scale;
  }
}

extern "C" int conef_allreduce_oneshot_ex(float* out, const float* const* peer_bufs,
                                          uint32_t* const* peer_flags, const uint32_t* my_flags, int world,
                                          int rank, uint32_t epoch, long long numel, float scale, int* status,
                                          long long spin_limit, const uint32_t* epoch_base, cudaStream_t stream) {
  if (numel <= 0) return 0;
  if (((uintptr_t)out & 15) != 0) { conef_set_error("allreduce_oneshot: output must be 16-byte aligned"); return 2; }
  long long blocks = (numel / 4 + 255) / 256;
  if (blocks < 1) blocks = 1;
  if (blocks > 296) blocks = 296;  // all blocks must be able to wait at once: 2 per SM
  k_allreduce_oneshot<<<(unsigned)blocks, 256, 0, stream>>>(out, peer_bufs, peer_flags, my_flags, world, rank,
                                                          epoch, numel, scale, status, spin_limit, epoch_base);
  CONEF_CHECK_LAUNCH("k_allreduce_oneshot");
  return 0;
}

extern "C" int conef_allreduce_oneshot(float* out, const float* const* peer_bufs,
                                       uint32_t* const* peer_flags, const uint32_t* my_flags, int world,
                                       int rank, uint32_t epoch, long long numel, float scale,
                                       int* status, long long spin_limit, cudaStream_t stream) {
  return conef_allreduce_oneshot_ex(out, peer_bufs, peer_flags, my_flags, world, rank, epoch, numel, scale,
                                    status, spin_limit, nullptr, stream);
}

// The device-side epoch word of captured launches: set it, or advance it by `delta`.
__global__ void k_epoch_word(uint32_t* word, uint32_t value, int add) {
  if (threadIdx.x == 0) *word = add ? *word + value : value;
}

extern "C" int conef_epoch_word(uint32_t* word, uint32_t value, int add, cudaStream_t stream) {
  k_epoch_word<<<1, 32, 0, stream>>>(word, value, add);
  CONEF_CHECK_LAUNCH("k_epoch_word");
  return 0;
}

// Legacy CUDA IPC fall-back for platforms where the framework's symmetric
// memory allocator is unavailable: export / import a cudaMalloc'd buffer.
extern "C" int conef_ipc_get_handle(void* dev_ptr, void* handle_out_64B) {
  cudaIpcMemHandle_t h;
  CONEF_CUDA(cudaIpcGetMemHandle(&h, dev_ptr));
  memcpy(handle_out_64B, &h, sizeof(h));
  return 0;
}
extern "C" int conef_ipc_open_handle(const void* handle_64B, void** dev_ptr_out) {
  cudaIpcMemHandle_t h;
  memcpy(&h, handle_64B, sizeof(h));
  CONEF_CUDA(cudaIpcOpenMemHandle(dev_ptr_out, h, cudaIpcMemLazyEnablePeerAccess));
  return 0;
}
extern "C" int conef_ipc_close_handle(void* dev_ptr) {
  CONEF_CUDA(cudaIpcCloseMemHandle(dev_ptr));
  return 0;
}
