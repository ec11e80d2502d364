// Tall-skinny GEMM tiles of PowerSGD on the 5th-generation tensor cores:
//   P = M Q      (n x m)(m x r)      "P mode": A = M tile, K-major (128-byte swizzle), K runs over columns
//   Q = M^T P    (m x n)(n x r)      "Q mode": A = M^T tile, MN-major, K runs over rows.  tf32 accepts an
//                                     MN-major operand only in the "128-byte swizzle, 32-byte atom" layout,
//                                     which TMA produces with CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B.
// for every TMA-addressable matrix of a bucket in one launch (grouped, split-K).
//
// One CTA computes a 128 x NP accumulator tile (NP = r padded to 16 or 32) in
// tensor memory:
//   warp 4, one lane : TMA producer - per stage four 32x32 fp32 boxes of M
//                      (cp.async.bulk.tensor.2d, 128-byte swizzle) and one bulk copy of the
//                      matching 32 x NP slice of the small operand, which the host side keeps
//                      pre-packed in the K-major core-matrix layout; local memory only
//   warps 0-3        : epilogue
//   warp 5, one lane : tcgen05.mma.kind::tf32 (4 x K=8 per stage), tcgen05.commit frees the stage
//   epilogue         : tcgen05.ld 32 lanes x NP columns per warp -> r floats per output row,
//                      plain store or fp32 atomics when K is split across CTAs
//   tail             : the CTA that finishes last (a device counter) publishes the bucket's epoch
//                      in every peer's flag array (release at system scope), so the all-reduce
//                      that consumes the product starts from this kernel, not from a launch of
//                      its own.  Peer memory is only written here (one flag word per peer),
//                      never read, and never the source of a bulk or tensor copy.
// Every mbarrier wait is bounded; when one gives up the CTA records
// CONEF_STATUS_MBAR_TIMEOUT, waits (bounded) for the copies it has in flight, frees its tensor
// memory and returns.
//
// Replaces torch.matmul(tensor, q, out=p) and torch.matmul(tensor.t(), p, out=q) of the
// reference (communication/powerSGD_hook.py:497-498,531-532), which are cuBLAS calls.
#include <cuda.h>
#include <string.h>
#include "common.cuh"

namespace {

constexpr int TC_BM = 128;
constexpr int TC_BK = 32;                    // fp32 elements per stage along K = one 128-byte row
constexpr int TC_STAGES = 6;
constexpr int TC_THREADS = 192;
constexpr int A_STAGE_BYTES = TC_BM * TC_BK * 4;   // 16 KB
constexpr int BOX_BYTES = 32 * 32 * 4;             // one TMA box
constexpr long long MBAR_SPIN_LIMIT = 4LL * 1000 * 1000;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait.  Returns false (and raises the CTA-wide abort flag) when the phase
// never completes or when another role has already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  for (long long it = 0; it < MBAR_SPIN_LIMIT; ++it) {
    if (mbar_try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
  }
  *abort_flag = 1;
  return false;
}

// plain (untiled) bulk copy global -> shared, 16-byte aligned on both sides, size a multiple of 16
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const void* tmap, int x, int y, uint32_t bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(tmap), "r"(x), "r"(y), "r"(bar) : "memory");
}

// 64-bit shared-memory matrix descriptor (sm_100 format, version 1).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes,
                                                   uint32_t layout_type) {
  uint64_t d = 0;
  d |= (uint64_t)((addr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                       // descriptor version
  d |= (uint64_t)(layout_type & 7) << 61;       // 0 = no swizzle, 1 = 128 B swizzle / 32 B atom, 2 = 128 B swizzle
  return d;
}

// Instruction descriptor: tf32 x tf32 -> fp32, M = 128, N = NP.
__host__ __device__ constexpr uint32_t make_idesc(int np, int a_mn_major, int b_mn_major) {
  return (1u << 4)                       // accumulator format fp32
         | (2u << 7) | (2u << 10)        // A, B = tf32
         | ((uint32_t)a_mn_major << 15) | ((uint32_t)b_mn_major << 16)
         | ((uint32_t)(np >> 3) << 17) | ((uint32_t)(TC_BM >> 4) << 24);
}

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                          uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

struct TcSignal {           // all zero: nothing is published
  uint32_t* done;           // counter of finished CTAs; zero between launches (the last CTA resets it)
  uint32_t* const* peer_flags;
  const uint32_t* epoch_base;   // nullable device word added to `epoch` (replayed launches)
  uint32_t epoch;
  int world, rank;
};

struct TcTile {      // one CTA's work
  int mat_flags;     // matrix index | (atomic accumulate << 30)
  int mn0;           // first output row of the 128-row tile (row of M in P mode, column of M in Q mode)
  int k0;            // first K index
  int klen;          // K extent of this CTA
};

template <int NP> struct BStage { static constexpr int BYTES = NP * TC_BK * 4; };

template <int NP>
constexpr int tc_smem_bytes() {
  return 1024 /* alignment slack */ + TC_STAGES * (A_STAGE_BYTES + BStage<NP>::BYTES) + 256;   // barriers, tmem slot, two flags
}

// Q_MODE = 0: out = P, A K-major, small operand = Q (m x r).   Q_MODE = 1: out = Q, A MN-major, small operand = P.
template <int NP, int Q_MODE>
__global__ void __launch_bounds__(TC_THREADS, 1)
k_tc_skinny(const ConefMat* __restrict__ mats, const CUtensorMap* __restrict__ maps,
            const TcTile* __restrict__ tiles, const float* __restrict__ small_packed, float* __restrict__ out_base,
            int* __restrict__ status, const TcSignal sig) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint8_t* a_st = smem;
  uint8_t* b_st = smem + TC_STAGES * A_STAGE_BYTES;
  uint64_t* bars = (uint64_t*)(b_st + TC_STAGES * BStage<NP>::BYTES);
  uint64_t* full = bars;                   // [TC_STAGES]
  uint64_t* empty = bars + TC_STAGES;      // [TC_STAGES]
  uint64_t* accum = bars + 2 * TC_STAGES;  // [1]
  uint32_t* tmem_slot = (uint32_t*)(bars + 2 * TC_STAGES + 1);
  volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
  volatile int* issued = abort_flag + 1;      // stages the producer has put in flight

  const TcTile T = tiles[blockIdx.x];
  const int mat = T.mat_flags & 0x3FFFFFFF;
  const bool atomic_out = (T.mat_flags >> 30) & 1;
  const ConefMat M = mats[mat];
  const int r = M.r;
  const int fold = M.fold > 1 ? M.fold : 1;          // folded view: (n / fold) x (fold * m), see ConefMat
  const int mn_total = Q_MODE ? M.m * fold : M.n / fold;
  const int k_total = Q_MODE ? M.n / fold : M.m * fold;
  const int k_end = min(k_total, T.k0 + T.klen);
  const int iters = (k_end - T.k0 + TC_BK - 1) / TC_BK;
  // small operand, packed: per K step of 8 rows NP * 8 floats (see conef_packed_offset)
  const float* small = small_packed + (Q_MODE ? (fold > 1 ? M.ppk_fold_off : M.ppk_off) : M.qpk_off);
  float* out = out_base + (Q_MODE ? M.q_off : M.p_off);              // (mn_total x r), row-major
  const CUtensorMap* tmap = maps + 2 * mat + Q_MODE;   // [2*mat] K-major view, [2*mat+1] MN-major view

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    *abort_flag = 0;
    *issued = 0;
    for (int s = 0; s < TC_STAGES; ++s) {
      mbar_init(smem_u32(full + s), 1);       // the producer's arrive.expect_tx
      mbar_init(smem_u32(empty + s), 1);      // tcgen05.commit
    }
    mbar_init(smem_u32(accum), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (warp == 0) {
    // 32 columns of tensor memory: 128 lanes x NP fp32 accumulators
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 32;" ::"r"(smem_u32(tmem_slot)) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 4) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      asm volatile("fence.proxy.tensormap::generic.acquire.gpu [%0], 128;" ::"l"(tmap) : "memory");
      for (int it = 0; it < iters; ++it) {
        const int s = it % TC_STAGES;
        if (!mbar_wait(smem_u32(empty + s), ((it / TC_STAGES) & 1) ^ 1, abort_flag)) break;
        const uint32_t bar = smem_u32(full + s);
        mbar_arrive_expect_tx(bar, A_STAGE_BYTES + BStage<NP>::BYTES);
        const uint32_t dst = smem_u32(a_st + s * A_STAGE_BYTES);
        const int k = T.k0 + it * TC_BK;
        bulk_load(smem_u32(b_st + s * BStage<NP>::BYTES), small + (size_t)k * NP, BStage<NP>::BYTES, bar);
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          // the tensor map is (columns, rows) of M with a 32 x 32 box; x is a multiple of 32 elements
          if (Q_MODE) tma_load_2d(dst + a * BOX_BYTES, tmap, T.mn0 + 32 * a, k, bar);
          else        tma_load_2d(dst + a * BOX_BYTES, tmap, k, T.mn0 + 32 * a, bar);
        }
        *issued = it + 1;
      }
    }
  } else if (warp == 5) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc(NP, Q_MODE ? 1 : 0, 0);
      constexpr uint32_t B_STEP = (NP / 8) * 256;     // bytes of the small operand per K step of 8
      bool ok = true;
      for (int it = 0; it < iters && ok; ++it) {
        const int s = it % TC_STAGES;
        ok = mbar_wait(smem_u32(full + s), (it / TC_STAGES) & 1, abort_flag);
        if (!ok) break;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t a_addr = smem_u32(a_st + s * A_STAGE_BYTES);
        const uint32_t b_addr = smem_u32(b_st + s * BStage<NP>::BYTES);
#pragma unroll
        for (int ks = 0; ks < TC_BK / 8; ++ks) {
          uint64_t da, db;
          if (Q_MODE)   // MN-major, 32-byte-atom swizzle: 32-column atoms 4096 B apart, 4-row K groups 512 B apart
            da = make_smem_desc(a_addr + ks * 1024, 4096, 512, 1);
          else          // K-major: 8-row groups 1024 B apart; a K step of 8 floats is 32 B inside the swizzle row
            da = make_smem_desc(a_addr + ks * 32, 16, 1024, 2);
          // small operand, K-major without swizzle: K-adjacent cores 128 B apart, 8-row N groups 256 B apart
          db = make_smem_desc(b_addr + ks * B_STEP, 128, 256, 0);
          umma_tf32(tmem_base, da, db, idesc, (it > 0 || ks > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(empty + s));     // stage reusable once these MMAs have read it
      }
      if (ok) umma_commit(smem_u32(accum));   // accumulator complete
    }
  } else {
    // ---------------- epilogue (warps 0-3) ----------------
    bool ok = true;
    if (ok) ok = mbar_wait(smem_u32(accum), 0, abort_flag);
    if (ok) {
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      uint32_t v[NP];
      const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
      if (NP == 16) {
        asm volatile(
            "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
            : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
              "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
            : "r"(taddr) : "memory");
      } else {
#pragma unroll
        for (int half = 0; half < NP / 16; ++half) {
          asm volatile(
              "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
              : "=r"(v[16 * half + 0]), "=r"(v[16 * half + 1]), "=r"(v[16 * half + 2]), "=r"(v[16 * half + 3]),
                "=r"(v[16 * half + 4]), "=r"(v[16 * half + 5]), "=r"(v[16 * half + 6]), "=r"(v[16 * half + 7]),
                "=r"(v[16 * half + 8]), "=r"(v[16 * half + 9]), "=r"(v[16 * half + 10]), "=r"(v[16 * half + 11]),
                "=r"(v[16 * half + 12]), "=r"(v[16 * half + 13]), "=r"(v[16 * half + 14]), "=r"(v[16 * half + 15])
              : "r"(taddr + 16 * half) : "memory");
        }
      }
      asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
      const int row = T.mn0 + warp * 32 + lane;
      if (row < mn_total) {
        if (!Q_MODE || fold == 1) {
          // P of a folded view: (n / fold) rows of fold * r values, which is the (n x r) block itself
          const int re = r * fold;
          float* o = out + (size_t)row * re;
#pragma unroll
          for (int c = 0; c < NP; ++c) {
            if (c < re) {
              if (atomic_out) atomicAdd(o + c, __uint_as_float(v[c]));
              else o[c] = __uint_as_float(v[c]);
            }
          }
        } else {
          // Q of a folded view: output row b * m + j carries its part of Q[j, :] in columns [b r, (b+1) r)
          const int b = row / M.m, j = row - b * M.m;
          float* o = out + (size_t)j * r;
#pragma unroll
          for (int c = 0; c < NP; ++c)
            if (c >= b * r && c < (b + 1) * r) atomicAdd(o + (c - b * r), __uint_as_float(v[c]));
        }
      }
    }
  }

  // ---------------- teardown (every role gets here: all loops are bounded) ----------------
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  if (*abort_flag) {
    if (threadIdx.x == 0) {
      atomicExch(status, CONEF_STATUS_MBAR_TIMEOUT);
      // Copies still in flight must land before this CTA's shared memory passes to the next one:
      // wait (bounded) for the `full` phase of every stage issued and not yet seen complete.
      const int n_issued = *issued;
      for (int it = max(0, n_issued - TC_STAGES); it < n_issued; ++it) {
        const uint32_t bar = smem_u32(full + it % TC_STAGES), parity = (it / TC_STAGES) & 1;
        for (long long spin = 0; spin < MBAR_SPIN_LIMIT && !mbar_try_wait(bar, parity); ++spin) {}
      }
    }
    __syncthreads();
  }
  if (warp == 0) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 32;" ::"r"(tmem_base) : "memory");
  }
  // ---------------- publish: the last CTA tells the peers that this GPU's product is complete ----------------
  if (sig.done != nullptr && threadIdx.x == 0) {
    __threadfence();                                   // this CTA's results, then the counter
    const unsigned prev = atomicAdd(sig.done, 1u);
    if (prev == gridDim.x - 1) {
      atomicExch(sig.done, 0u);                        // ready for the next launch
      __threadfence_system();                          // everything counted above, then the flags
      const uint32_t epoch = sig.epoch + (sig.epoch_base != nullptr ? *sig.epoch_base : 0u);
      for (int p = 0; p < sig.world; ++p) st_release_sys(sig.peer_flags[p] + sig.rank, epoch);
    }
  }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static bool tried = false;
  if (!tried) {
    tried = true;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = (EncodeTiledFn)p;
  }
  return fn;
}

template <int NP, int Q_MODE>
int launch_tc(const ConefMat* mats, const void* maps, const void* tiles, int ntiles, const float* small_base,
              float* out_base, int* status, const TcSignal& sig, cudaStream_t stream) {
  constexpr int smem = tc_smem_bytes<NP>();
  static bool configured[64] = {};      // the attribute is per device
  int dev = 0;
  CONEF_CUDA(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64 || !configured[dev]) {
    CONEF_CUDA(cudaFuncSetAttribute(k_tc_skinny<NP, Q_MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    if (dev >= 0 && dev < 64) configured[dev] = true;
  }
  k_tc_skinny<NP, Q_MODE><<<ntiles, TC_THREADS, smem, stream>>>(mats, (const CUtensorMap*)maps, (const TcTile*)tiles,
                                                               small_base, out_base, status, sig);
  CONEF_CHECK_LAUNCH("k_tc_skinny");
  return 0;
}

}  // namespace

extern "C" int conef_tc_supported(void) { return get_encode_fn() != nullptr ? 1 : 0; }

// Encode two tensor maps per matrix (host side): [2i] 128-byte swizzle for the K-major
// reads of P = M Q, [2i+1] 128-byte swizzle with 32-byte atoms for the MN-major reads of
// Q = M^T P.  A matrix can be addressed by TMA when its first element is 16-byte aligned
// and its row pitch is a multiple of 16 bytes; ok[i] = 0 marks the others, which the
// caller routes to the SIMT kernels.
extern "C" int conef_tc_encode_maps(const ConefMat* host_mats, int nmats, const float* bucket_dev,
                                    const float* aux_dev, void* maps_out_256B_each, unsigned char* ok) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) { conef_set_error("cuTensorMapEncodeTiled is not available"); return 1; }
  CUtensorMap* out = (CUtensorMap*)maps_out_256B_each;
  for (int i = 0; i < nmats; ++i) {
    const ConefMat& M = host_mats[i];
    const uintptr_t base = (uintptr_t)((M.src ? aux_dev : bucket_dev) + M.g_off);
    ok[i] = 0;
    memset(&out[2 * i], 0, 2 * sizeof(CUtensorMap));
    const int fold = M.fold > 1 ? M.fold : 1;
    const long long vm = (long long)M.m * fold;          // the (n / fold) x (fold * m) view
    if ((base & 15) != 0 || (vm % 4) != 0 || vm < 4 || (M.n % fold) != 0 || (M.src && aux_dev == nullptr)) continue;
    cuuint64_t dims[2] = {(cuuint64_t)vm, (cuuint64_t)(M.n / fold)};
    cuuint64_t strides[1] = {(cuuint64_t)vm * sizeof(float)};
    cuuint32_t box[2] = {32, 32};
    cuuint32_t estr[2] = {1, 1};
    CUresult rc0 = enc(&out[2 * i], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    CUresult rc1 = enc(&out[2 * i + 1], CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc0 == CUDA_SUCCESS && rc1 == CUDA_SUCCESS) ok[i] = 1;
  }
  return 0;
}

// mode 0: P = M Q (small operand Q, output P); mode 1: Q = M^T P (small operand P, output Q).
// With done != NULL the CTA that finishes last stores epoch (+ *epoch_base) into
// peer_flags[p][rank] for every p < world.
extern "C" int conef_psgd_tc_signal(int mode, const ConefMat* mats, const void* maps, const void* tiles, int ntiles,
                                    const float* small_base, float* out_base, int max_rank, int* status,
                                    uint32_t* done, uint32_t* const* peer_flags, int world, int rank,
                                    uint32_t epoch, const uint32_t* epoch_base,
                                    cudaStream_t stream) {   // small_base: packed small operands
  if (ntiles <= 0) return 0;
  if (max_rank > 32) { conef_set_error("tcgen05 path supports rank <= 32"); return 2; }
  TcSignal sig;
  memset(&sig, 0, sizeof(sig));
  if (done != nullptr && peer_flags != nullptr && world > 1) {
    sig.done = done; sig.peer_flags = peer_flags; sig.epoch_base = epoch_base;
    sig.epoch = epoch; sig.world = world; sig.rank = rank;
  }
  if (max_rank <= 16) {
    return mode == 0 ? launch_tc<16, 0>(mats, maps, tiles, ntiles, small_base, out_base, status, sig, stream)
                     : launch_tc<16, 1>(mats, maps, tiles, ntiles, small_base, out_base, status, sig, stream);
  }
  return mode == 0 ? launch_tc<32, 0>(mats, maps, tiles, ntiles, small_base, out_base, status, sig, stream)
                   : launch_tc<32, 1>(mats, maps, tiles, ntiles, small_base, out_base, status, sig, stream);
}

extern "C" int conef_psgd_tc(int mode, const ConefMat* mats, const void* maps, const void* tiles, int ntiles,
                             const float* small_base, float* out_base, int max_rank, int* status,
                             cudaStream_t stream) {
  return conef_psgd_tc_signal(mode, mats, maps, tiles, ntiles, small_base, out_base, max_rank, status, nullptr,
                              nullptr, 1, 0, 0, nullptr, stream);
}
