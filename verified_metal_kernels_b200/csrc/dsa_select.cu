// `dsa` stage 2: exact top-2048 selection per request.
//
// One CTA of 1024 threads per request.  Scores are mapped to order-preserving 32-bit keys (NaN ranks
// last) and the 2048-th largest key T is found by a radix select over 11 + 11 + 10 bits:
//   level 1  a 2048-bin histogram of the top 11 bits -- taken from the indexer, which accumulates it in
//            its epilogue, or built here in one pass when absent;
//   fast path (the boundary bin holds at most 8192 entries; entries equal to T that do not all fit in the
//            result are told apart by position): ONE pass over the scores stages the boundary bin's (key,
//            position) pairs in shared memory and, per warp span, counts the entries above the bin and keeps their positions while they
//            fit; levels 2 and 3 then run on the staged pairs only; a warp whose selected entries were all kept
//            (the usual case) ranks them by counting and writes them out, any other warp makes ONE more pass over
//            its span that writes the positions in ascending order;
//   general path (a boundary bin of more than 8192 entries, more than twice a warp's share of it inside one warp's
//            span, or more than 256 entries equal to T): levels 2 and 3 over the scores, then an ordered compaction
//            that takes the ties at T from the lowest positions.
// The result is deterministic: the same scores always give the same ascending index list.  Passes read
// the scores as float4 when the row length allows (four independent 16-byte loads in flight per lane).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace vmk {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kSelThreads = 1024;
constexpr int kCandBin = 8192;              // largest boundary bin the fast path takes
constexpr int kCandCap = 2 * kCandBin;      // room for staged pairs: each warp stages into a region of its own (no
constexpr int kCandWarp = kCandCap / 32;    // atomics) that holds twice its share of the largest bin.  With regions of
                                            // exactly the share, a bin of 7738 entries (242 per warp on average) had a
                                            // warp with 283 and sent its request down the general path: 0.137 ms for
                                            // the kernel instead of 0.035, on about one batch of 128 in four
constexpr int kAboveWarp = 160;             // per warp: positions of the entries above the boundary bin (staged too,
                                            // so that a warp whose selected entries fit here needs no second pass)
constexpr int kRankMax = 96;                // ... and are few enough to be ranked by counting
constexpr int kRankSpan = 1024;             // shortest warp span for which that is done
constexpr int kTieCap = 256;                // most entries equal to the threshold key the fast path sorts out itself
constexpr int kSelSmem = kCandCap * 8 + 32 * kAboveWarp * 4;      // (key, position) pairs, then the positions above

#ifdef VMK_SEL_TIMING
// Debug build only: cycles per phase of CTA 0, thread 0.
__device__ long long g_sel_timing[8];
#define SEL_T(slot) do { if (blockIdx.x == 0 && threadIdx.x == 0) { long long _t1 = clock64(); g_sel_timing[slot] += _t1 - _t0; _t0 = _t1; } } while (0)
#else
#define SEL_T(slot) do {} while (0)
#endif

struct SelShared {
  uint32_t hist[kSelBins];
  uint32_t scan[32];
  uint32_t res[3];
  uint32_t w_a[32], w_b[32];
  uint32_t w_n[32];          // staged pairs per warp
  uint32_t overflow;
  uint32_t total;            // entries this CTA contributes to the result
  uint32_t tie_n;            // rank 0 only: entries with key == T gathered so far (peers add theirs remotely)
  uint32_t tie_cut;          // entries with key == T belong to the result up to this position
  uint32_t tie_pos[kTieCap]; // rank 0: their positions, in no order; every rank: a local copy
  uint32_t sum[kSelBins];    // histogram summed over the cluster (level 1, or a local copy of acc*)
  uint32_t acc2[kSelBins];   // rank 0 only: level-2 histogram, peers add their staged entries remotely
  uint32_t acc3[kSelBins];   // rank 0 only: level-3 histogram
};

// Scanning bins from the top, finds the bin where the running count reaches `need`; returns the bin, the
// count strictly above it and the bin's own count through sh.res.  Called by all threads.
__device__ __forceinline__ void find_bin(SelShared& sh, const uint32_t* hist, uint32_t need) {
  constexpr int PER = kSelBins / kSelThreads;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t own = 0;
#pragma unroll
  for (int i = 0; i < PER; ++i) own += hist[kSelBins - 1 - (tid * PER + i)];
  uint32_t v = own;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
    if (lane >= o) v += t;
  }
  if (lane == 31) sh.scan[warp] = v;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = sh.scan[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
      if (lane >= o) w += t;
    }
    sh.scan[lane] = w;
  }
  __syncthreads();
  const uint32_t incl = v + (warp > 0 ? sh.scan[warp - 1] : 0u);
  const uint32_t excl = incl - own;
  if (excl < need && need <= incl) {           // exactly one thread
    uint32_t above = excl;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
      const int bin = kSelBins - 1 - (tid * PER + i);
      const uint32_t c = hist[bin];
      if (above < need && need <= above + c) {
        sh.res[0] = (uint32_t)bin;
        sh.res[1] = above;
        sh.res[2] = c;
      }
      above += c;
    }
  }
  __syncthreads();
}

__device__ __forceinline__ void clear_hist(SelShared& sh) {
  for (int i = threadIdx.x; i < kSelBins; i += kSelThreads) sh.hist[i] = 0u;
  __syncthreads();
}

// One step of a warp's walk over its span: lane l loads the EPL consecutive scores at
// beg + (step * 32 + l) * EPL and returns their keys (0 beyond `end`).
template <int EPL>
__device__ __forceinline__ void load_keys(const float* __restrict__ s, int i0, int end, uint32_t (&k)[EPL]) {
  if (EPL == 4) {
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i0 < end) v = *reinterpret_cast<const float4*>(s + i0);   // the row length is a multiple of 4
    k[0] = score_key(v.x);
    k[1 % EPL] = score_key(v.y);
    k[2 % EPL] = score_key(v.z);
    k[3 % EPL] = score_key(v.w);
  } else {
    k[0] = i0 < end ? score_key(s[i0]) : 0u;
  }
}

// Inverse of score_key for non-NaN keys: the float whose key is k.
__device__ __forceinline__ float key_to_float(uint32_t k) {
  return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

// Raw scores of one step (NaN beyond `end`, so that every ordered comparison is false there).
template <int EPL>
__device__ __forceinline__ void load_vals(const float* __restrict__ s, int i0, int end, float (&x)[EPL]) {
  const float nanv = __uint_as_float(0x7fc00000u);
  if (EPL == 4) {
    float4 v = make_float4(nanv, nanv, nanv, nanv);
    if (i0 < end) v = *reinterpret_cast<const float4*>(s + i0);
    x[0] = v.x;
    x[1 % EPL] = i0 + 1 < end ? v.y : nanv;
    x[2 % EPL] = i0 + 2 < end ? v.z : nanv;
    x[3 % EPL] = i0 + 3 < end ? v.w : nanv;
  } else {
    x[0] = i0 < end ? s[i0] : nanv;
  }
}

// Warp walk over [beg, end) with U independent loads in flight per lane.  body(i, valid, key) sees each
// lane's positions in ascending order.
template <int EPL, int U, class Body>
__device__ __forceinline__ void walk(const float* __restrict__ s, int beg, int end, int lane, Body&& body) {
  const int per_step = 32 * EPL;
  const int steps = (end - beg + per_step - 1) / per_step;
  for (int t = 0; t < steps; t += U) {
    uint32_t k[U][EPL];
#pragma unroll
    for (int u = 0; u < U; ++u) load_keys<EPL>(s, beg + ((t + u) * 32 + lane) * EPL, end, k[u]);
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int i0 = beg + ((t + u) * 32 + lane) * EPL;
#pragma unroll
      for (int e = 0; e < EPL; ++e) body(i0 + e, i0 + e < end, k[u][e]);
    }
  }
}

// General path: levels 2 and 3 over the scores themselves, then an ordered compaction with the ties at
// T taken from the lowest positions.
template <int EPL>
__device__ void general_path(SelShared& sh, const float* __restrict__ s, int beg, int end, uint32_t b1,
                             uint32_t above1, int32_t* __restrict__ out) {
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  uint32_t prefix = b1 << kSelShift, mask = (uint32_t)(kSelBins - 1) << kSelShift;
  uint32_t need = kTopK - above1, tie_total = 0;
#pragma unroll 1
  for (int pass = 1; pass < 3; ++pass) {
    const int shift = pass == 1 ? 10 : 0;
    const uint32_t nb = pass == 2 ? 1024u : 2048u;
    clear_hist(sh);
    walk<EPL, 4>(s, beg, end, lane, [&](int, bool v, uint32_t k) {
      if (v && (k & mask) == prefix) atomicAdd(&sh.hist[(k >> shift) & (nb - 1)], 1u);
    });
    __syncthreads();
    find_bin(sh, sh.hist, need);
    need -= sh.res[1];
    tie_total = sh.res[2];
    prefix |= sh.res[0] << shift;
    mask |= (nb - 1) << shift;
    __syncthreads();
  }
  const uint32_t T = prefix;
  const bool partial_tie = tie_total != need;
  const uint32_t below = (1u << lane) - 1u;
  uint32_t eq_base = 0;
  if (partial_tie) {
    uint32_t c = 0;
    walk<1, 4>(s, beg, end, lane, [&](int, bool v, uint32_t k) { c += __popc(__ballot_sync(0xffffffffu, v && k == T)); });
    if (lane == 0) sh.w_a[warp] = c;
    __syncthreads();
    for (int w = 0; w < warp; ++w) eq_base += sh.w_a[w];
  }
  {
    uint32_t c = 0, eqs = eq_base;
    walk<1, 4>(s, beg, end, lane, [&](int, bool v, uint32_t k) {
      const uint32_t eqm = __ballot_sync(0xffffffffu, v && k == T);
      const uint32_t rank = eqs + __popc(eqm & below);
      const bool sel = v && (k > T || (k == T && (!partial_tie || rank < need)));
      c += __popc(__ballot_sync(0xffffffffu, sel));
      eqs += __popc(eqm);
    });
    if (lane == 0) sh.w_b[warp] = c;
  }
  __syncthreads();
  uint32_t pos = 0;
  for (int w = 0; w < warp; ++w) pos += sh.w_b[w];
  {
    uint32_t eqs = eq_base;
    walk<1, 4>(s, beg, end, lane, [&](int i, bool v, uint32_t k) {
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
}

// Sum of the per-CTA histograms of a cluster into sh.sum (all ranks end up with the same totals), and the
// OR of the ranks' overflow flags.  With a single CTA it is a plain copy.
template <bool CLUSTER>
__device__ __forceinline__ bool reduce_hist(SelShared& sh) {
  const int tid = threadIdx.x;
  bool any_overflow = sh.overflow != 0u;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                   // every rank's histogram is complete
    const unsigned nr = cluster.num_blocks();
    for (int i = tid; i < kSelBins; i += kSelThreads) {
      uint32_t acc = 0;
      for (unsigned r = 0; r < nr; ++r) acc += *cluster.map_shared_rank(&sh.hist[i], r);
      sh.sum[i] = acc;
    }
    for (unsigned r = 0; r < nr; ++r) any_overflow |= *cluster.map_shared_rank(&sh.overflow, r) != 0u;
    cluster.sync();                                   // nobody clears a histogram that is still being read
  } else {
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.sum[i] = sh.hist[i];
    __syncthreads();
  }
  return any_overflow;
}

// Histogram of one radix digit of the staged entries of the whole cluster.  The entries are few (at most
// 8192 per cluster), so every rank adds its own directly into rank 0's `acc` array with distributed
// shared-memory atomics; after one cluster barrier every rank copies the 2048 totals into its local
// sh.sum.  `acc` was cleared before the first cluster barrier of the kernel.  Returns the OR of the
// overflow flags, gathered the same way.
template <bool CLUSTER, class Digit>
__device__ __forceinline__ bool staged_hist(SelShared& sh, uint32_t* acc_local, const uint32_t* ckey, Digit&& digit) {
  const int tid = threadIdx.x;
  if (CLUSTER) {
    cg::cluster_group cluster = cg::this_cluster();
    uint32_t* acc0 = cluster.map_shared_rank(acc_local, 0);
    uint32_t* ovf0 = cluster.map_shared_rank(&sh.overflow, 0);
    for (int j = tid; j < kCandCap; j += kSelThreads) {
      if ((uint32_t)(j % kCandWarp) < sh.w_n[j / kCandWarp]) {
        const int d = digit(ckey[j]);
        if (d >= 0) atomicAdd(&acc0[d], 1u);
      }
    }
    if (tid == 0 && sh.overflow != 0u) atomicOr(ovf0, 1u);
    cluster.sync();
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.sum[i] = acc0[i];
    const bool ovf = *ovf0 != 0u;
    __syncthreads();
    return ovf;
  } else {
    for (int j = tid; j < kCandCap; j += kSelThreads) {
      if ((uint32_t)(j % kCandWarp) < sh.w_n[j / kCandWarp]) {
        const int d = digit(ckey[j]);
        if (d >= 0) atomicAdd(&acc_local[d], 1u);
      }
    }
    __syncthreads();
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.sum[i] = acc_local[i];
    const bool ovf = sh.overflow != 0u;
    __syncthreads();
    return ovf;
  }
}

// One request per CTA, or per cluster of CTAs that split the positions between them (a single SM reads its
// scores at well under 100 GB/s, so a long row is spread over several SMs; histograms, flags and counts
// are exchanged through distributed shared memory).
template <int EPL, bool CLUSTER>
__global__ void __launch_bounds__(kSelThreads, 1) select_kernel(const float* __restrict__ scores,
                                                             const uint32_t* __restrict__ hist_in,
                                                             const int32_t* __restrict__ lens,
                                                             int32_t* __restrict__ idx, int32_t* __restrict__ cnt,
                                                             int L, int csize) {
  // the kernel after this one (the sparse attention, in the fused call) may set itself up while this one runs;
  // it waits for this grid to finish before it reads the lists written here
  asm volatile("griddepcontrol.launch_dependents;");
  __shared__ SelShared sh;
  extern __shared__ uint32_t cand[];          // [kCandCap] keys, then [kCandCap] positions
  uint32_t* ckey = cand;
  uint32_t* cidx = cand + kCandCap;
  uint32_t* cpos = cand + 2 * kCandCap;       // [32 warps][kAboveWarp]

  const int b = CLUSTER ? blockIdx.x / csize : blockIdx.x;
  const int crank = CLUSTER ? blockIdx.x % csize : 0;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  // Set-up that reads nothing the indexer writes: this kernel is itself a programmatic dependent of it, so the
  // shared-memory clearing and the first cluster barrier overlap the indexer's tail.
  if (tid == 0) {
    sh.overflow = 0u;
    sh.total = 0u;
    sh.tie_n = 0u;
    sh.tie_cut = 0xffffffffu;
  }
  for (int i = tid; i < kSelBins; i += kSelThreads) sh.acc2[i] = sh.acc3[i] = 0u;
  __syncthreads();
  if (CLUSTER) cg::this_cluster().sync();         // rank 0's accumulators are clear before any peer adds to them
  pdl_wait();                                     // scores, histogram and lengths are read below this line

  int n = L;
  if (lens != nullptr) n = max(0, min(lens[b], L));
  const float* s = scores + (size_t)b * L;
  int32_t* out = idx + (size_t)b * kTopK;

  if (n <= kTopK) {                            // uniform across the cluster: nobody reaches a later cluster barrier
    if (crank == 0) {
      for (int i = tid; i < kTopK; i += kSelThreads) out[i] = i < n ? i : 0;
      if (tid == 0) cnt[b] = n;
    }
    return;
  }
  // this CTA's part of the row, and its warps' spans: contiguous, multiples of 4 long (float4 alignment)
  const int part = CLUSTER ? (((n + csize - 1) / csize + 127) & ~127) : n;
  const int pbeg = min(n, crank * part), pend = min(n, pbeg + part);
  const int span = ((pend - pbeg + 31) / 32 + 3) & ~3;
  const int beg = min(pend, pbeg + warp * span);
  int end = min(pend, beg + span);

#ifdef VMK_SEL_TIMING
  long long _t0 = clock64();
#endif
  // ---- level 1 ------------------------------------------------------------------------------------------
  if (hist_in != nullptr) {
    for (int i = tid; i < kSelBins; i += kSelThreads) sh.sum[i] = hist_in[(size_t)b * kSelBins + i];
    __syncthreads();
  } else {
    clear_hist(sh);
    walk<EPL, 4>(s, beg, end, lane, [&](int, bool v, uint32_t k) {
      if (v) atomicAdd(&sh.hist[k >> kSelShift], 1u);
    });
    __syncthreads();
    reduce_hist<CLUSTER>(sh);
  }
  SEL_T(0);
  find_bin(sh, sh.sum, kTopK);
  const uint32_t b1 = sh.res[0], above1 = sh.res[1], c1 = sh.res[2];
  __syncthreads();
  SEL_T(1);

  // cluster-uniform; the lowest bin (NaN lives there) and the empty top bins take the general path
  bool fast = c1 <= (uint32_t)kCandBin && b1 >= 1u && b1 <= 2043u;
  uint32_t T = 0;
  // entries above the boundary bin in this warp's span (warp-uniform).  Their positions are kept only for a span
  // long enough that ranking the kept entries beats a second pass over it (measured: 4096 positions per warp
  // 41 -> 35.5 us, 1024: 19.7 -> 18.6; a span of 256 lost 2-4 us): a short span starts "full".
  uint32_t bstaged = (end - beg) >= kRankSpan ? 0u : (uint32_t)kAboveWarp + 1u;
  if (fast) {
    // ---- one pass: every warp stages the boundary-bin entries of its span, in position order, into its
    //      own region, and counts what lies above the bin.  Membership in the bin is an interval test on
    //      the raw score (keys are monotonic in the score); NaN fails both tests. -------------------------
    const float lo = key_to_float(b1 << kSelShift), hi = key_to_float((b1 + 1u) << kSelShift);
    uint32_t above = 0, staged = 0;             // staged is warp-uniform
    uint32_t* wkey = ckey + warp * kCandWarp;
    uint32_t* widx = cidx + warp * kCandWarp;
    uint32_t* wpos = cpos + warp * kAboveWarp;  // positions of the entries above the bin, kept while they fit
    {
      constexpr int U = 8;
      const int per_step = 32 * EPL;
      const int steps = (end - beg + per_step - 1) / per_step;
      for (int t = 0; t < steps; t += U) {
        float x[U][EPL];
#pragma unroll
        for (int u = 0; u < U; ++u) load_vals<EPL>(s, beg + ((t + u) * 32 + lane) * EPL, end, x[u]);
        uint32_t cf = 0, af = 0;
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
          for (int e = 0; e < EPL; ++e) {
            af |= x[u][e] >= hi ? (1u << (u * EPL + e)) : 0u;
            cf |= (x[u][e] >= lo && x[u][e] < hi) ? (1u << (u * EPL + e)) : 0u;
          }
        }
        above += __popc(af);
        if (bstaged <= (uint32_t)kAboveWarp && __any_sync(0xffffffffu, af != 0u)) {
          const uint32_t c = __popc(af);
          uint32_t incl = c;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
          }
          uint32_t slot = bstaged + incl - c;
          while (af != 0u) {                      // about one element in sixty
            const int bit = __ffs(af) - 1;
            af &= af - 1u;
            if (slot < (uint32_t)kAboveWarp) wpos[slot] = (uint32_t)(beg + ((t + bit / EPL) * 32 + lane) * EPL + bit % EPL);
            ++slot;
          }
          bstaged += __shfl_sync(0xffffffffu, incl, 31);
        }
        if (__any_sync(0xffffffffu, cf != 0u)) {
          const uint32_t c = __popc(cf);
          uint32_t incl = c;
#pragma unroll
          for (int o = 1; o < 32; o <<= 1) {
            const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += y;
          }
          uint32_t slot = staged + incl - c;
          while (cf != 0u) {                      // candidates are rare: walk the set bits only
            const int bit = __ffs(cf) - 1;
            cf &= cf - 1u;
            const int u = bit / EPL, e = bit % EPL;
            if (slot < (uint32_t)kCandWarp) {
              float xv = x[0][0];
#pragma unroll
              for (int uu = 0; uu < U; ++uu)
#pragma unroll
                for (int ee = 0; ee < EPL; ++ee) xv = (uu * EPL + ee == bit) ? x[uu][ee] : xv;
              wkey[slot] = score_key(xv);
              widx[slot] = (uint32_t)(beg + ((t + u) * 32 + lane) * EPL + e);
            }
            ++slot;
          }
          staged += __shfl_sync(0xffffffffu, incl, 31);
        }
      }
    }
    above = (uint32_t)__reduce_add_sync(0xffffffffu, above);
    if (lane == 0) {
      sh.w_a[warp] = above;
      sh.w_n[warp] = min(staged, (uint32_t)kCandWarp);
      if (staged > (uint32_t)kCandWarp) sh.overflow = 1u;
    }
    __syncthreads();
    SEL_T(2);
    // ---- levels 2 and 3 on the staged pairs -----------------------------------------------------------
    uint32_t need = kTopK - above1;
    const bool overflow = staged_hist<CLUSTER>(sh, sh.acc2, ckey, [](uint32_t k) { return (int)((k >> 10) & 2047u); });
    uint32_t tie_total = 0;
    if (!overflow) {
      find_bin(sh, sh.sum, need);
      const uint32_t b2 = sh.res[0];
      need -= sh.res[1];
      __syncthreads();
      staged_hist<CLUSTER>(sh, sh.acc3, ckey,
                           [b2](uint32_t k) { return ((k >> 10) & 2047u) == b2 ? (int)(k & 1023u) : -1; });
      find_bin(sh, sh.sum, need);
      T = (b1 << kSelShift) | (b2 << 10) | sh.res[0];
      need -= sh.res[1];
      tie_total = sh.res[2];
      __syncthreads();
    }
    // Entries equal to T: all of them belong to the result (the usual case), or only the `need` of them at the lowest
    // positions.  With scores summed from 16-bit products a tie at the threshold is not rare (about one request in a
    // thousand at L = 131072), and the general path costs a request 0.13 ms instead of 0.035: the tied entries are
    // staged ones, so they are gathered (positions only, on rank 0 of a cluster) and the cut position is the need-th
    // smallest of them.
    bool ties_ok = tie_total == need;
    if (!overflow && !ties_ok && tie_total <= (uint32_t)kTieCap) {
      uint32_t* n0 = &sh.tie_n;
      uint32_t* pos0 = sh.tie_pos;
      if (CLUSTER) {
        cg::cluster_group cluster = cg::this_cluster();
        n0 = cluster.map_shared_rank(&sh.tie_n, 0);
        pos0 = cluster.map_shared_rank(sh.tie_pos, 0);
      }
      for (int j = tid; j < kCandCap; j += kSelThreads) {
        if ((uint32_t)(j % kCandWarp) < sh.w_n[j / kCandWarp] && ckey[j] == T) {
          const uint32_t slot = atomicAdd(n0, 1u);
          if (slot < (uint32_t)kTieCap) pos0[slot] = cidx[j];
        }
      }
      if (CLUSTER) cg::this_cluster().sync(); else __syncthreads();
      uint32_t mine = 0xffffffffu;
      if ((uint32_t)tid < tie_total) mine = pos0[tid];      // (rank 0's list; every rank takes its own copy)
      __syncthreads();
      if ((uint32_t)tid < tie_total) sh.tie_pos[tid] = mine;
      __syncthreads();
      if ((uint32_t)tid < tie_total) {
        uint32_t r = 0;
        for (uint32_t j = 0; j < tie_total; ++j) r += sh.tie_pos[j] < mine ? 1u : 0u;
        if (r + 1u == need) sh.tie_cut = mine;              // positions are distinct: exactly one thread
      }
      __syncthreads();
      ties_ok = true;
    }
    fast = !overflow && ties_ok;
  }
  const uint32_t tie_cut = sh.tie_cut;          // 0xffffffff when every entry equal to T is taken
  // a staged or scanned entry belongs to the result
  auto taken = [&](uint32_t key, uint32_t position) { return key > T || (key == T && position <= tie_cut); };
  uint32_t pos = 0;
  if (fast) {
    // selected entries of this warp's span = those above the boundary bin + its staged ones with key >= T
    uint32_t c = 0;
    for (uint32_t j = lane; j < sh.w_n[warp]; j += 32)
      c += taken(ckey[warp * kCandWarp + j], cidx[warp * kCandWarp + j]) ? 1u : 0u;
    c = (uint32_t)__reduce_add_sync(0xffffffffu, c);
    if (lane == 0) {
      sh.w_a[warp] += c;
      atomicAdd(&sh.total, sh.w_a[warp]);
    }
    __syncthreads();
    if (CLUSTER) {
      cg::cluster_group cluster = cg::this_cluster();
      cluster.sync();                            // every rank's total is final
      for (int r = 0; r < crank; ++r) pos += *cluster.map_shared_rank(&sh.total, r);
    }
  }
  if (!fast) {
    // cluster-uniform decision.  The general path runs on one CTA over the whole row.
    if (CLUSTER) {
      if (crank != 0) return;
      const int gspan = ((n + 31) / 32 + 3) & ~3;
      const int gbeg = min(n, warp * gspan), gend = min(n, gbeg + gspan);
      general_path<EPL>(sh, s, gbeg, gend, b1, above1, out);
    } else {
      general_path<EPL>(sh, s, beg, end, b1, above1, out);
    }
    if (tid == 0) cnt[b] = kTopK;
    return;
  }

  SEL_T(3);
  // ---- ordered emission: positions with score >= the threshold, ascending -------------------------------
  for (int w = 0; w < warp; ++w) pos += sh.w_a[w];
  {
    // A warp whose selected entries were all staged (those above the bin in the first pass, those of the bin with
    // key >= T now) and are few ranks them by counting and writes them out: no second pass over its span.
    uint32_t n = bstaged;
    bool staged_all = bstaged <= (uint32_t)kAboveWarp;
    if (staged_all) {
      uint32_t* wpos = cpos + warp * kAboveWarp;
      const uint32_t* wkey = ckey + warp * kCandWarp;
      const uint32_t* widx = cidx + warp * kCandWarp;
      const uint32_t nA = sh.w_n[warp];
      for (uint32_t j0 = 0; j0 < nA; j0 += 32) {
        const uint32_t j = j0 + lane;
        const bool f = j < nA && taken(wkey[j], widx[j]);
        const uint32_t mask = __ballot_sync(0xffffffffu, f);
        const uint32_t at = n + __popc(mask & ((1u << lane) - 1u));
        if (f && at < (uint32_t)kAboveWarp) wpos[at] = widx[j];
        n += __popc(mask);
      }
      staged_all = n <= (uint32_t)kRankMax;
      if (staged_all) {
        __syncwarp();
        for (uint32_t i = lane; i < n; i += 32) {
          const uint32_t pi = wpos[i];
          uint32_t r = 0;
          for (uint32_t j = 0; j < n; ++j) r += wpos[j] < pi ? 1u : 0u;
          if (pos + r < (uint32_t)kTopK) out[pos + r] = (int32_t)pi;
        }
      }
    }
    if (staged_all) end = beg;                  // nothing left for the second pass
  }
  const int per_step = 32 * EPL;
  const int steps = (end - beg + per_step - 1) / per_step;
  const float Tf = key_to_float(T);             // score >= Tf  <=>  key >= T (NaN: false)
  constexpr int UE = 8;                           // loads in flight per lane
  for (int t = 0; t < steps; t += UE) {
    float x[UE][EPL];
#pragma unroll
    for (int u = 0; u < UE; ++u) load_vals<EPL>(s, beg + ((t + u) * 32 + lane) * EPL, end, x[u]);
#pragma unroll
    for (int u = 0; u < UE; ++u) {
      const int i0 = beg + ((t + u) * 32 + lane) * EPL;
      uint32_t flags = 0;
#pragma unroll
      for (int e = 0; e < EPL; ++e)
        flags |= (x[u][e] > Tf || (x[u][e] == Tf && (uint32_t)(i0 + e) <= tie_cut)) ? (1u << e) : 0u;
      if (!__any_sync(0xffffffffu, flags != 0u)) continue;
      const uint32_t c = __popc(flags);
      uint32_t incl = c;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += y;
      }
      uint32_t p = pos + incl - c;
      while (flags != 0u) {                       // about one element in sixty is selected
        const int e = __ffs(flags) - 1;
        flags &= flags - 1u;
        if (p < (uint32_t)kTopK) out[p] = i0 + e;
        ++p;
      }
      pos += __shfl_sync(0xffffffffu, incl, 31);
    }
  }
  SEL_T(4);
  if (tid == 0 && crank == 0) cnt[b] = kTopK;
  if (CLUSTER) cg::this_cluster().sync();         // peers may still be reading this CTA's shared memory
}

#ifdef VMK_SEL_TIMING
extern "C" VMK_API int vmk_debug_sel_timing(long long* out, int reset) {
  long long zero[8] = {0};
  cudaDeviceSynchronize();
  if (out) cudaMemcpyFromSymbol(out, g_sel_timing, sizeof(zero));
  if (reset) cudaMemcpyToSymbol(g_sel_timing, zero, sizeof(zero));
  return 0;
}
#endif

static int g_select_cluster = 0;       // test hook: 0 = chosen by the batch, else 1, 2, 4 or 8

template <int EPL>
static int launch_select(const float* scores, const uint32_t* hist, const int32_t* lens, int32_t* idx, int32_t* cnt,
                         int B, int L, cudaStream_t stream) {
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(select_kernel<EPL, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelSmem);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(select_kernel<EPL, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSelSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  // Long rows of a small batch are split over a cluster of 8, 4 or 2 CTAs (that many SMs read a row together), at
  // most the size at which all B clusters are resident together.  That is fewer than SMs / size: a cluster lives inside
  // one GPC (16 requests x 8 CTAs are 128 CTAs, but they took two waves: 0.036 ms against 0.020 ms with 4 CTAs each;
  // 32 x 8: 0.055 against 0.021; 37 x 4: 0.043 against 0.028 with 2 each).  With many requests every SM is busy
  // anyway and one CTA per request does the same work with fewer barriers.
  static int resident[4] = {0, 0, 0, 0};       // clusters of 1 << i CTAs that can be resident together (i = 1..3)
  static int resident_dev = -1;
  if (resident_dev != dev) {
    for (int i = 1; i <= 3; ++i) {
      cudaLaunchConfig_t q;
      memset(&q, 0, sizeof(q));
      q.gridDim = dim3((unsigned)(sm_count() / (1 << i)) * (1 << i));
      q.blockDim = dim3(kSelThreads);
      q.dynamicSmemBytes = kSelSmem;
      cudaLaunchAttribute qa[1];
      qa[0].id = cudaLaunchAttributeClusterDimension;
      qa[0].val.clusterDim.x = 1 << i;
      qa[0].val.clusterDim.y = 1;
      qa[0].val.clusterDim.z = 1;
      q.attrs = qa;
      q.numAttrs = 1;
      int n = 0;
      if (cudaOccupancyMaxActiveClusters(&n, select_kernel<EPL, true>, &q) != cudaSuccess) n = 0;
      cudaGetLastError();
      resident[i] = n;
    }
    resident_dev = dev;
  }
  int csize = 1;
  if (g_select_cluster > 0) {
    csize = g_select_cluster;
  } else {
    // measured with 1-8 requests (us, CTAs per request 1 / 2 / 4 / 8): L = 32768: 16.0-16.9 / 15.4-15.9 / 15.5-16.0 /
    // 17.3-17.8; L = 65536: 19.8-22.2 / 15.2-17.2 / 16.1-17.5 / 17.6-19.0; L = 131072: 27.7-31.7 / 19.4-22.0 /
    // 15.0-16.9 / 17.9-20.1 (eight CTAs: the extra barriers cost more than the shorter spans save until the rows are
    // much longer); then no more CTAs per request than are resident together
    csize = L >= 524288 ? 8 : L >= 98304 ? 4 : 2;
    int i = csize == 8 ? 3 : csize == 4 ? 2 : 1;
    while (csize > 1 && B > resident[i]) {
      csize >>= 1;
      --i;
    }
  }
  if (L >= 32768 && csize > 1) {
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)B * csize);
    cfg.blockDim = dim3(kSelThreads);
    cfg.dynamicSmemBytes = kSelSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = csize;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    return check_launch(cudaLaunchKernelEx(&cfg, select_kernel<EPL, true>, scores, hist, lens, idx, cnt, L, csize));
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3((unsigned)B);
  cfg.blockDim = dim3(kSelThreads);
  cfg.dynamicSmemBytes = kSelSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_launch(cudaLaunchKernelEx(&cfg, select_kernel<EPL, false>, scores, hist, lens, idx, cnt, L, 1));
}

int select_launch(const float* scores, const uint32_t* hist, const int32_t* lens, int32_t* idx, int32_t* cnt, int B,
                  int L, cudaStream_t stream) {
  if (!scores || !idx || !cnt || B <= 0 || L <= 0) return VMK_E_BADARG;
  const bool vec = (L % 4 == 0) && ((reinterpret_cast<uintptr_t>(scores) & 15) == 0);
  return vec ? launch_select<4>(scores, hist, lens, idx, cnt, B, L, stream)
             : launch_select<1>(scores, hist, lens, idx, cnt, B, L, stream);
}

}  // namespace vmk

// Test hook: CTAs per request of the top-k selection on long rows (0 = chosen by the batch size, the default).
extern "C" VMK_API int vmk_dsa_set_select_cluster(int csize) {
  if (csize != 0 && csize != 1 && csize != 2 && csize != 4 && csize != 8) return VMK_E_BADARG;
  vmk::g_select_cluster = csize;
  return VMK_OK;
}

extern "C" int vmk_dsa_select(const float* scores, const int32_t* lens, int32_t* idx, int32_t* cnt, int B, int L,
                              void* stream) {
  return vmk::select_launch(scores, nullptr, lens, idx, cnt, B, L, static_cast<cudaStream_t>(stream));
}
