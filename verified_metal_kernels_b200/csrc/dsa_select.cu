// `dsa` stage 2: exact top-2048 selection per request.
//
// One CTA of 1024 threads per request.  Scores are mapped to order-preserving 32-bit keys (NaN ranks
// last); a three-pass radix select (11 + 11 + 10 bits, shared-memory histograms) finds the exact key T
// of the 2048-th largest score and how many entries equal to T belong to the result; an ordered
// compaction then writes the positions in ascending order, taking ties at T from the lowest positions.
// The result is therefore deterministic: the same scores always give the same index list.
#include "common.cuh"

namespace vmk {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kSelThreads = 1024;

__device__ __forceinline__ uint32_t score_key(float x) {
  if (x != x) return 0u;                       // NaN: never preferred
  const uint32_t u = __float_as_uint(x + 0.0f);   // -0.0 and +0.0 compare equal, so they share a key
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Finds, scanning bins from the top, the bin where the running count reaches `need`.
// hist has NB bins; returns the bin and the count strictly above it.  All threads call it.
template <int NB>
__device__ __forceinline__ void find_bin(const uint32_t* hist, uint32_t need, uint32_t* s_scan, uint32_t* s_res) {
  // Each thread owns NB / 1024 consecutive bins counted from the top.
  constexpr int PER = NB / kSelThreads;
  static_assert(PER >= 1, "bins per thread");
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t own = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) own += hist[NB - 1 - (tid * PER + i)];
  // inclusive scan over threads (descending bins)
  uint32_t v = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  if (lane == 31) s_scan[warp] = v;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = s_scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    s_scan[lane] = w;
  }
  __syncthreads();
  const uint32_t incl = v + (warp > 0 ? s_scan[warp - 1] : 0u);
  const uint32_t excl = incl - own;
  if (excl < need && need <= incl) {           // exactly one thread
    uint32_t above = excl;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int bin = NB - 1 - (tid * PER + i);
      const uint32_t c = hist[bin];
      if (above < need && need <= above + c) {
        s_res[0] = (uint32_t)bin;
        s_res[1] = above;
        s_res[2] = c;
      }
      above += c;
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(kSelThreads) select_kernel(const float* __restrict__ scores,
                                                             const int32_t* __restrict__ lens,
                                                             int32_t* __restrict__ idx, int32_t* __restrict__ cnt,
                                                             int L) {
  __shared__ uint32_t hist[2048];
  __shared__ uint32_t s_scan[32];
  __shared__ uint32_t s_res[3];
  __shared__ uint32_t w_eq[32], w_sel[32];

  const int b = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int n = L;
  if (lens != nullptr) n = max(0, min(lens[b], L));
  const float* s = scores + (size_t)b * L;
  int32_t* out = idx + (size_t)b * kTopK;

  if (n <= kTopK) {
    for (int i = tid; i < kTopK; i += kSelThreads) out[i] = i < n ? i : 0;
    if (tid == 0) cnt[b] = n;
    return;
  }

  // ---- radix select of the 2048-th largest key ---------------------------------------------------
  uint32_t prefix = 0, mask = 0, need = kTopK, tie_total = 0;
#pragma unroll 1
  for (int pass = 0; pass < 3; ++pass) {
    const int shift = pass == 0 ? 21 : (pass == 1 ? 10 : 0);
    const uint32_t nb = pass == 2 ? 1024u : 2048u;
    for (int i = tid; i < 2048; i += kSelThreads) hist[i] = 0;
    __syncthreads();
#pragma unroll 4
    for (int i = tid; i < n; i += kSelThreads) {
      const uint32_t k = score_key(s[i]);
      if ((k & mask) == prefix) atomicAdd(&hist[(k >> shift) & (nb - 1)], 1u);
    }
    __syncthreads();
    find_bin<2048>(hist, need, s_scan, s_res);   // bins beyond nb are empty
    const uint32_t bin = s_res[0];
    need -= s_res[1];
    tie_total = s_res[2];
    prefix |= bin << shift;
    mask |= (nb - 1) << shift;
    __syncthreads();
  }
  const uint32_t T = prefix;            // key of the 2048-th largest score
  const bool partial_tie = tie_total != need;   // more entries equal T than fit

  // ---- ordered compaction: warp w walks [w*span, (w+1)*span) ----------------------------------------
  const int span = (n + 31) / 32;
  const int beg = min(n, warp * span), end = min(n, beg + span);
  const int iters = (span + 31) / 32;

  // Walks the warp's range 128 positions at a time (four independent loads in flight per lane).
  auto walk = [&](auto&& body) {
    for (int it = 0; it < iters; it += 4) {
      uint32_t k[4];
      bool v[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = beg + (it + u) * 32 + lane;
        v[u] = i < end;
        k[u] = v[u] ? score_key(s[i]) : 0u;
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) body(beg + (it + u) * 32 + lane, v[u], k[u]);
    }
  };

  uint32_t eq_base = 0;
  if (partial_tie) {
    uint32_t c = 0;
    walk([&](int, bool v, uint32_t k) { c += __popc(__ballot_sync(0xffffffffu, v && k == T)); });
    if (lane == 0) w_eq[warp] = c;
    __syncthreads();
    for (int w = 0; w < warp; ++w) eq_base += w_eq[w];
  }
  const uint32_t below = (1u << lane) - 1u;
  {
    uint32_t c = 0, eqs = eq_base;
    walk([&](int, bool v, uint32_t k) {
      const uint32_t eqm = __ballot_sync(0xffffffffu, v && k == T);
      const uint32_t rank = eqs + __popc(eqm & below);
      const bool sel = v && (k > T || (k == T && (!partial_tie || rank < need)));
      c += __popc(__ballot_sync(0xffffffffu, sel));
      eqs += __popc(eqm);
    });
    if (lane == 0) w_sel[warp] = c;
  }
  __syncthreads();
  uint32_t pos = 0;
  for (int w = 0; w < warp; ++w) pos += w_sel[w];
  {
    uint32_t eqs = eq_base;
    walk([&](int i, bool v, uint32_t k) {
      const uint32_t eqm = __ballot_sync(0xffffffffu, v && k == T);
      const uint32_t rank = eqs + __popc(eqm & below);
      const bool sel = v && (k > T || (k == T && (!partial_tie || rank < need)));
      const uint32_t sm = __ballot_sync(0xffffffffu, sel);
      if (sel) {
        const uint32_t p = pos + __popc(sm & below);
        if (p < (uint32_t)kTopK) out[p] = i;
      }
      pos += __popc(sm);
      eqs += __popc(eqm);
    });
  }
  if (tid == 0) cnt[b] = kTopK;
}

}  // namespace vmk

extern "C" int vmk_dsa_select(const float* scores, const int32_t* lens, int32_t* idx, int32_t* cnt, int B, int L,
                              void* stream) {
  using namespace vmk;
  if (!scores || !idx || !cnt || B <= 0 || L <= 0) return VMK_E_BADARG;
  select_kernel<<<B, kSelThreads, 0, static_cast<cudaStream_t>(stream)>>>(scores, lens, idx, cnt, L);
  return check_launch(cudaGetLastError());
}
