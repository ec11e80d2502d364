// Grouped magnitude top-k of the error matrices of a bucket (hPowerSGD's error store).
//
// The reference keeps the k largest-magnitude entries of every residual matrix with one
// torch.topk + gather + zero + scatter per matrix (communication/hPowerSGD_hook.py:90-97), i.e. a
// sort per matrix.  Here all matrices of a bucket go through one radix select: three histogram
// passes over the 31 magnitude bits (11 + 10 + 10), each followed by a tiny per-matrix scan that
// fixes the next digits of the k-th largest magnitude, then one pass that zeroes what is smaller.
// Entries that tie with the threshold are all kept (a sort would keep an arbitrary subset of them).
#include "common.cuh"

namespace {

constexpr int TK_THREADS = 256;
constexpr int TK_CHUNK = 16384;          // elements per CTA
constexpr int TK_BINS = 2048;            // bins of the first pass; later passes use 1024

struct TopkState {                       // one per matrix, in the scratch buffer
  uint32_t prefix;                       // digits of the threshold found so far
  uint32_t remaining;                    // how many entries are still wanted among the candidates
};

__device__ __forceinline__ uint32_t mag_bits(float x) { return __float_as_uint(x) & 0x7fffffffu; }

// pass 0: digit = bits >> 20 (all entries); pass 1: digit = (bits >> 10) & 1023 where bits >> 20 == prefix;
// pass 2: digit = bits & 1023 where bits >> 10 == prefix.
template <int PASS>
__global__ void __launch_bounds__(TK_THREADS)
k_topk_hist(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, const float* __restrict__ err,
            const TopkState* __restrict__ st, uint32_t* __restrict__ hist) {
  __shared__ uint32_t h[TK_BINS];
  constexpr int BINS = PASS == 0 ? TK_BINS : 1024;
  for (int i = threadIdx.x; i < BINS; i += TK_THREADS) h[i] = 0;
  __syncthreads();
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const long long numel = (long long)M.n * M.m;
  const long long lo = (long long)t.y * TK_CHUNK;
  const int len = (int)min((long long)TK_CHUNK, numel - lo);
  const float* x = err + M.g_off + lo;
  const uint32_t prefix = PASS == 0 ? 0u : st[t.x].prefix;
  auto count = [&](float v) {
    const uint32_t b = mag_bits(v);
    if (PASS == 0) atomicAdd(&h[b >> 20], 1u);
    else if (PASS == 1) { if ((b >> 20) == prefix) atomicAdd(&h[(b >> 10) & 1023u], 1u); }
    else { if ((b >> 10) == prefix) atomicAdd(&h[b & 1023u], 1u); }
  };
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {        // 16-byte loads where the chunk starts aligned
    const int len4 = len >> 2;
    const float4* x4 = reinterpret_cast<const float4*>(x);
    for (int i = threadIdx.x; i < len4; i += TK_THREADS) {
      const float4 v = __ldg(x4 + i);
      count(v.x); count(v.y); count(v.z); count(v.w);
    }
    for (int i = (len4 << 2) + threadIdx.x; i < len; i += TK_THREADS) count(__ldg(x + i));
  } else {
    for (int i = threadIdx.x; i < len; i += TK_THREADS) count(__ldg(x + i));
  }
  __syncthreads();
  uint32_t* g = hist + (size_t)t.x * TK_BINS;
  for (int i = threadIdx.x; i < BINS; i += TK_THREADS)
    if (h[i]) atomicAdd(g + i, h[i]);
}

// One CTA (one warp) per matrix: find the bin, counted from the top, in which the cumulative count
// reaches `remaining`; append it to the prefix, keep what is still wanted inside that bin, and clear
// the histogram for the next pass.
__global__ void k_topk_scan(const ConefMat* __restrict__ mats, TopkState* __restrict__ st, uint32_t* __restrict__ hist,
                            int pass, float ratio) {
  const int k = blockIdx.x, lane = threadIdx.x;
  const int bins = pass == 0 ? TK_BINS : 1024, shift = pass == 0 ? 11 : 10;
  uint32_t* g = hist + (size_t)k * TK_BINS;
  TopkState s = st[k];
  if (pass == 0) {
    const long long numel = (long long)mats[k].n * mats[k].m;
    long long want = (long long)(0.5 * (double)ratio * (double)numel);
    if (want < 1) want = 1;
    if (want > numel) want = numel;
    s.prefix = 0;
    s.remaining = (uint32_t)want;
  }
  const int per = bins / 32;               // lane 0 owns the top bins
  const int top = bins - 1 - lane * per;   // highest bin of this lane
  uint32_t mine = 0;
  for (int i = 0; i < per; ++i) mine += g[top - i];
  uint32_t incl = mine;                     // inclusive scan over lanes (top lanes first)
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t v = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += v;
  }
  const uint32_t before = incl - mine;
  const bool here = before < s.remaining && incl >= s.remaining;
  const unsigned who = __ballot_sync(0xffffffffu, here);
  uint32_t digit = 0, rem = s.remaining;
  if (who == 0) {                           // fewer candidates than wanted (cannot happen for pass 0): keep all
    digit = 0;
    rem = 0;
  } else {
    const int src = __ffs(who) - 1;
    if (lane == src) {
      uint32_t acc = before;
      for (int i = 0; i < per; ++i) {
        const uint32_t c = g[top - i];
        if (acc + c >= s.remaining) { digit = (uint32_t)(top - i); rem = s.remaining - acc; break; }
        acc += c;
      }
    }
    digit = __shfl_sync(0xffffffffu, digit, src);
    rem = __shfl_sync(0xffffffffu, rem, src);
  }
  __syncwarp();
  for (int i = lane; i < bins; i += 32) g[i] = 0;
  if (lane == 0) {
    s.prefix = (s.prefix << shift) | digit;
    s.remaining = rem;
    st[k] = s;
  }
}

__global__ void __launch_bounds__(TK_THREADS)
k_topk_apply(const ConefMat* __restrict__ mats, const int2* __restrict__ tiles, float* __restrict__ err,
             const TopkState* __restrict__ st) {
  const int2 t = tiles[blockIdx.x];
  const ConefMat M = mats[t.x];
  const long long numel = (long long)M.n * M.m;
  const long long lo = (long long)t.y * TK_CHUNK;
  const int len = (int)min((long long)TK_CHUNK, numel - lo);
  float* x = err + M.g_off + lo;
  const uint32_t thr = st[t.x].prefix;      // the 31 magnitude bits of the k-th largest entry
  if ((reinterpret_cast<uintptr_t>(x) & 15) == 0) {
    const int len4 = len >> 2;
    float4* x4 = reinterpret_cast<float4*>(x);
    for (int i = threadIdx.x; i < len4; i += TK_THREADS) {
      float4 v = x4[i];
      const bool cx = mag_bits(v.x) < thr, cy = mag_bits(v.y) < thr, cz = mag_bits(v.z) < thr, cw = mag_bits(v.w) < thr;
      if (cx | cy | cz | cw) {
        if (cx) v.x = 0.f;
        if (cy) v.y = 0.f;
        if (cz) v.z = 0.f;
        if (cw) v.w = 0.f;
        x4[i] = v;
      }
    }
    for (int i = (len4 << 2) + threadIdx.x; i < len; i += TK_THREADS)
      if (mag_bits(x[i]) < thr) x[i] = 0.f;
  } else {
    for (int i = threadIdx.x; i < len; i += TK_THREADS) {
      const float v = x[i];
      if (mag_bits(v) < thr) x[i] = 0.f;
    }
  }
}

}  // namespace

// scratch: nmats * (2048 + 2) 32-bit words, zero before the first call (every call leaves the
// histograms zero again).  tiles: int2 {matrix, chunk of 16384 elements} over the first nmats records.
extern "C" int conef_topk_keep(const ConefMat* mats, int nmats, const int2* tiles, int ntiles, float* err,
                               float ratio, uint32_t* scratch, cudaStream_t stream) {
  if (nmats <= 0 || ntiles <= 0) return 0;
  uint32_t* hist = scratch;
  TopkState* st = reinterpret_cast<TopkState*>(scratch + (size_t)nmats * TK_BINS);
  k_topk_hist<0><<<ntiles, TK_THREADS, 0, stream>>>(mats, tiles, err, st, hist);
  CONEF_CHECK_LAUNCH("k_topk_hist<0>");
  k_topk_scan<<<nmats, 32, 0, stream>>>(mats, st, hist, 0, ratio);
  CONEF_CHECK_LAUNCH("k_topk_scan");
  k_topk_hist<1><<<ntiles, TK_THREADS, 0, stream>>>(mats, tiles, err, st, hist);
  CONEF_CHECK_LAUNCH("k_topk_hist<1>");
  k_topk_scan<<<nmats, 32, 0, stream>>>(mats, st, hist, 1, ratio);
  CONEF_CHECK_LAUNCH("k_topk_scan");
  k_topk_hist<2><<<ntiles, TK_THREADS, 0, stream>>>(mats, tiles, err, st, hist);
  CONEF_CHECK_LAUNCH("k_topk_hist<2>");
  k_topk_scan<<<nmats, 32, 0, stream>>>(mats, st, hist, 2, ratio);
  CONEF_CHECK_LAUNCH("k_topk_scan");
  k_topk_apply<<<ntiles, TK_THREADS, 0, stream>>>(mats, tiles, err, st);
  CONEF_CHECK_LAUNCH("k_topk_apply");
  return 0;
}

extern "C" int conef_topk_chunk(void) { return TK_CHUNK; }
