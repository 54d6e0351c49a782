// `dsa` stage 3 on the 5th-generation tensor cores, two SMs per request: absorbed-MLA attention over the
// selected rows by a CLUSTER OF TWO CTAs that share the score product.
//
// What one CTA per (request, value half) costs: a tcgen05.mma of M = 128 and N <= 128 takes about 96 cycles
// whatever N is, and each value half needs the whole S = Q.K^T (36 instructions of K = 16 per 64 keys) for its
// 8 instructions of P.V: 44 x 96 = 4.25 k cycles per 64 keys, 36 of the 44 spent on a product the other half
// computes as well.  Here the two CTAs of a cluster take one request together:
//   * CTA r computes the partial scores over HALF of the 576 contraction elements (r = 0: elements [0,288),
//     r = 1: [288,576); 18 instructions instead of 36).  Four exchange warps take them out of tensor memory into a
//     staging buffer and send them on to the peer with one asynchronous shared-memory-to-shared-memory copy per warp
//     (8 KiB each, completing on a barrier in the peer's shared memory).  Every softmax thread adds the two halves
//     in the same order, so both CTAs hold the same S, P, m and l;
//   * CTA r owns value columns [256 r, 256 r + 256): its P.V is four instructions of N = 256 (138 cycles each) that
//     ACCUMULATE O in tensor memory.  The softmax threads keep a reference maximum that follows the true one lazily
//     (raised only when a block exceeds it by more than 2^8, so that P stays far inside the 16-bit range); only then
//     is O read, rescaled and written back, which after a request's first block is rare.  The result is the same
//     quotient: numerator and denominator carry the same factor;
//   * CTA r therefore gathers only column blocks [4 r, 4 r + 5) of every selected row (its value columns, which
//     are also its share of the contraction; block 4 goes to both): 40 KiB per 64 keys instead of 72.
// Floor of the tensor pipe: 18 x 96.5 + 4 x 138 = 2.3 k cycles per 64 keys.  What sets the period in practice is the
// chain of the softmax threads (3.5-3.8 k cycles per block): the copy of a block's 32 KiB of partial scores takes
// about 2 k cycles to cross, which is why it is issued by warps of its own, a block ahead of the softmax.
// The B requests x 32 block slots form one list, cut into equal contiguous ranges, one per cluster; a request
// cut by a range boundary leaves (m, l, o) partials, at most two per cluster, merged by mla_pair_combine_kernel.
// Shared memory: a ring of three 40 KiB slots (per request two entries of staged queries, then the key blocks:
// five [64 rows][128 B] blocks with the 128-byte swizzle), two 32 KiB staging buffers and the 32 KiB buffer the
// peer's copies land in.  One CTA = 576 threads:
//   warps 0-3   softmax group A, warps 4-7 group B: one thread per head and group.  A takes keys [0,32) of each
//               block and value columns [0,128) of the CTA's half (when O is rescaled or written out), B keys
//               [32,64) and columns [128,256); the two threads of a head exchange block maxima through shared memory
//   warps 8-11  gather by cp.async: warp w fetches rows [16 w, 16 w + 16) of every key block; positions are
//               loaded a block ahead, and the rows of the block three ahead are asked into L2
//   warp 12     issues S = Q.K^T (A = the queries, kept in tensor memory)
//   warp 13     owns tensor memory and issues P.V (A = P from tensor memory)
//   warps 14-17 exchange (above); they also copy a request's queries from the ring into tensor memory, so that the
//               next request's first scores are on their way while the softmax threads still write the last one out
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA winds down through the
// common exit, where both CTAs meet at a cluster barrier (nobody leaves while its peer may still copy into its
// shared memory) and tensor memory is freed.  Nothing here is a multicast: every copy has one destination.
#include "dsa_mla_tc.cuh"
#include "tcgen05.cuh"

namespace vmk {
namespace {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kMH = 128, kDK = 576, kDV = 512;
constexpr int kBK = 64;                               // keys per block
constexpr int kBlkBytes = kBK * 128;                  // one [64 rows][128 B] swizzled block
constexpr int kSlotBlocks = 5;                        // column blocks a CTA holds per key block
constexpr int kSlot = kSlotBlocks * kBlkBytes;        // 40 KiB
constexpr int kStages = 3;
constexpr int kThreads = 576;
constexpr int kGatherWarps = 4, kWarpGather0 = 8;     // warps 8..11
constexpr int kWarpQK = 12, kWarpPV = 13;
constexpr int kWarpExch0 = 14;                        // warps 14..17: partial scores out of tensor memory, to the peer
constexpr int kPrefetch = 3;                          // key blocks the L2 prefetch runs ahead of the gather
constexpr float kLazy = 8.f;                          // how far (log2) a block maximum may exceed the reference maximum
constexpr int kQEntries = 2;                          // ring entries that stage a request's queries
constexpr int kKSteps = 18;                           // K = 16 steps of the contraction per CTA
constexpr int kColQ = 0;                              // 144 columns: this CTA's 288 query elements, packed pairs
constexpr int kColS = 160;                            // 64 columns: partial scores
constexpr int kColT = 224;                            // 256 columns: O, the output accumulator of the CTA's value half
constexpr int kColP = 480;                            // 32 columns: P as packed pairs
constexpr int kCols = 512;
constexpr int kXBytes = 128 * kBK * 4;                // partial scores of a block: [lane quarter][float4 i of 16][lane]
constexpr int kBars = 2 * kStages + 17;
constexpr int kSmem = kStages * kSlot + 3 * kXBytes + kBars * 8 + 16 + 8 * 128 * 4 + 1024;

constexpr int kUnitSlots = kTopK / kBK;               // 32 block slots per request
constexpr int kMinSlotsPerCluster = 2;

__host__ __device__ __forceinline__ int range_start(int c, int total, int n) {
  return (int)(((long long)c * total) / n);
}

// One request's share of a cluster's range.
struct UnitWork {
  int k0, k1, nblk;
  bool whole;
};
__device__ __forceinline__ UnitWork unit_work(const MlaTcParams& p, int b, int slot0, int slot1) {
  UnitWork w;
  const int ja = max(slot0 - b * kUnitSlots, 0), jb = min(slot1 - b * kUnitSlots, kUnitSlots);
  const int nb = max(0, min(p.cnt[b], kTopK));
  w.k0 = ja * kBK;
  w.k1 = min(nb, jb * kBK);
  w.nblk = w.k1 > w.k0 ? (w.k1 - w.k0 + kBK - 1) / kBK : 0;
  w.whole = ja == 0 && jb == kUnitSlots;
  return w;
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// ---- the cluster of two: addresses in the peer's shared memory, stores and barrier arrivals there -----------
__device__ __forceinline__ uint32_t cluster_rank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ uint32_t peer_addr(const void* local, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_u32(local)), "r"(rank));
  return r;
}
// Arrival at a barrier in the peer's shared memory that only says "I have finished READING what you sent": no data
// of ours has to become visible with it, and the values it covers have been used by the time it is issued, so it
// carries no fence (a release at cluster scope was measured at 1-2 k cycles here, in the middle of the softmax).
__device__ __forceinline__ void arrive_peer_relaxed(uint32_t bar_addr) {
  asm volatile("mbarrier.arrive.relaxed.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_addr) : "memory");
}
// Bounded wait for such an arrival from the peer.
__device__ __forceinline__ bool mbar_wait_peer_relaxed(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.relaxed.cluster.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    if (ok) return true;
  }
  return false;
}
// Asynchronous copy of `bytes` (a multiple of 16) from this CTA's shared memory into the peer's; the bytes count
// towards the transaction count of a barrier in the peer's shared memory.  One destination, no multicast.
__device__ __forceinline__ void bulk_copy_to_peer(uint32_t dst_addr, const void* src, uint32_t bytes, uint32_t bar_addr) {
  asm volatile("cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst_addr),
               "r"(smem_u32(src)), "r"(bytes), "r"(bar_addr)
               : "memory");
}
// Asks for `bytes` (a multiple of 16) of global memory to be brought into L2.
__device__ __forceinline__ void l2_prefetch(const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

#ifdef VMK_MLA_TIMING
// Debug build only.  Time stamps of blocks 8..15 of CTA 0: [role][block - 8][event]; roles 0 = issuers,
// 1 = gather warp 0, 2 = softmax group A warp 0, 3 = softmax group B warp 0, 4 = the exchange warp of lane quarter 0.
__device__ long long g_pair_trace[5 * 8 * 16];
#define PAIR_E(role, j, ev) do { if (blockIdx.x == 0 && (j) >= 8 && (j) < 16 && lane == 0) \
    g_pair_trace[((role) * 8 + (j) - 8) * 16 + (ev)] = clock64(); } while (0)
#else
#define PAIR_E(role, j, ev) do {} while (0)
#endif

}  // namespace

__global__ void __launch_bounds__(kThreads, 1) mla_pair_kernel(const __grid_constant__ MlaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                   // [stages][5 blocks][64 rows][128 B]
  float4* xsend = reinterpret_cast<float4*>(sK + kStages * kSlot);          // [2] our partial scores, staged for the copy
  float4* xbuf = xsend + 2 * (kXBytes / 16);                                // the peer's, written by its copy
  uint64_t* full = reinterpret_cast<uint64_t*>(reinterpret_cast<uint8_t*>(xbuf) + kXBytes);   // entry landed
  uint64_t* empty = full + kStages;                     // entry consumed                       (MMA commit)
  uint64_t* q_full = empty + kStages;                   // Q stored to tensor memory            (4 warps)
  uint64_t* s_full = q_full + 1;                        // partial scores ready                 (MMA commit)
  uint64_t* s_free = s_full + 1;                        // partial scores out of tensor memory  (4 warps)
  uint64_t* p_full = s_free + 1;                        // P in tensor memory, O rescaled       (8 warps)
  uint64_t* pv_done = p_full + 1;                       // P.V added to O                       (MMA commit)
  uint64_t* o_free = pv_done + 1;                       // a request's O has been written out   (8 warps)
  uint64_t* x_full = o_free + 1;                        // the peer's partial scores are here   (1 arrival + 32 KiB)
  uint64_t* x_free = x_full + 1;                        // the peer has read what we sent       (8 peer warps)
  uint64_t* xch = x_free + 1;                           // [4] pair of warps that share 32 heads exchanged values
  uint64_t* xs_full = xch + 4;                          // [2] our partial scores are staged    (4 warps)
  uint64_t* xs_free = xs_full + 2;                      // [2] ... and have been read           (8 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xs_free + 2);
  float* smax = reinterpret_cast<float*>(tmem_slot + 4);    // [2 parities][2 groups][128 heads] block maxima
  float* ssum = smax + 4 * 128;                             // [2 parities][2 groups][128 heads] row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rank = (int)cluster_rank();                 // value half, and half of the contraction
  const int cl = blockIdx.x >> 1;                       // the range this cluster works on
  const int total_slots = p.B * kUnitSlots;
  const int slot0 = range_start(cl, total_slots, p.ncta), slot1 = range_start(cl + 1, total_slots, p.ncta);
  const int u_first = slot0 / kUnitSlots, u_last = slot1 > slot0 ? (slot1 - 1) / kUnitSlots : u_first - 1;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(&full[s], kGatherWarps * 32);
      mbar_init(&empty[s], 1);
    }
    mbar_init(q_full, 4);
    mbar_init(s_full, 1);
    mbar_init(s_free, 4);
    for (int i = 0; i < 2; ++i) {
      mbar_init(&xs_full[i], 4);
      mbar_init(&xs_free[i], 8);
    }
    mbar_init(p_full, 8);
    mbar_init(pv_done, 1);
    mbar_init(o_free, 8);
    mbar_init(x_full, 1);
    mbar_init(x_free, 8);
    for (int q = 0; q < 4; ++q) mbar_init(&xch[q], 2);
    fence_mbar_init();
  }
  if (warp == kWarpPV) tmem_alloc(tmem_slot, kCols);
  if (warp == kWarpGather0 && lane == 0) tma_prefetch_desc(&p.tmQ);
  tc_fence_before();
  cluster_sync_all();                                   // both CTAs' barriers exist before either arrives at the other's
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched as a programmatic dependent: everything above overlaps the tail of the kernel before (the top-k
  // selection, in the fused call); the candidate lists and counts are read only below this line.
  pdl_wait();
  int nblk_total = 0;                                   // key blocks of this CTA's whole range
  for (int u = u_first; u <= u_last; ++u) nblk_total += unit_work(p, u, slot0, slot1).nblk;

  bool timed_out = false;
  if (warp < 8) {
    // ------------------------------------------------------------------------------ softmax groups
    // Group A (warps 0-3) owns keys [0,32) of every block and value columns [0,128) of the CTA's half when O is
    // rescaled or written out; group B (warps 4-7) keys [32,64) and columns [128,256).  The two threads of a head
    // exchange their block maxima through shared memory, so both follow the same reference maximum.
    const int grp = warp >> 2;
    const int quarter = warp & 3;
    const int head = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tO = lane_base + kColT + grp * 128, tPw = lane_base + kColP + grp * 16;
    // this thread's 32 partial scores of a block: float4 [16 quarter + 8 grp + i][lane], i < 8, in a staging buffer
    // (ours) and in xbuf (the peer's)
    const int xoff = (quarter * 16 + grp * 8) * 32 + lane;
    const float4* rcv = xbuf + xoff;
    const uint32_t peer_x_free = peer_addr(x_free, (uint32_t)(rank ^ 1));
    if (tid == 0 && nblk_total > 0) mbar_expect_tx(x_full, kXBytes);      // the first block's 32 KiB from the peer
    int base = 0;                                       // blocks of the requests before this one
    uint32_t nx = 0;                                    // exchanges through xch so far
    for (int u = u_first; u <= u_last && !timed_out; ++u) {
      const UnitWork w = unit_work(p, u, slot0, slot1);
      // m is the REFERENCE maximum: P = exp2(s - m) and O, l are sums relative to it.  It follows the true
      // maximum lazily: only when a block's maximum exceeds it by more than kLazy (P then stays below 2^kLazy,
      // far inside the range of a 16-bit float) is it raised and O rescaled, which is rare after a request's first
      // block.  The result is the same sum; only the common factor of numerator and denominator differs.
      float m = -INFINITY, l = 0.f;
      for (int j = 0; j < w.nblk; ++j) {
        const int g = base + j;
        // ---- the two halves of the contraction: ours from the staging buffer, the peer's from its copy
        bool ok = mbar_wait(&xs_full[g & 1], (uint32_t)((g >> 1) & 1));
        if (quarter == 0) PAIR_E(2 + grp, g, 0);
        if (ok) ok = mbar_wait(x_full, (uint32_t)(g & 1));   // the bytes were written into OUR shared memory: as for a TMA load
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (tid == 0 && g + 1 < nblk_total) mbar_expect_tx(x_full, kXBytes);     // the next block's
        if (quarter == 0) PAIR_E(2 + grp, g, 3);
        const float4* own = xsend + (g & 1) * (kXBytes / 16) + xoff;
        const int kb = w.k0 + j * kBK + grp * 32;
        const bool tail = kb + 32 > w.k1;
        float bm = -INFINITY;
        uint32_t s[32];
        {
          // both halves into registers first, so that the two buffers go back at once: the peer's next copy waits
          // for that, and it takes about 2 k cycles to cross
          float4 v[8], o[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            v[i] = rcv[i * 32];
            o[i] = own[i * 32];
          }
          // The arrivals must not be issued before the loads have returned: their address is made to depend on one
          // word of every load (and'ed to zero where the compiler cannot see it).
          uint32_t dep = 0u;
#pragma unroll
          for (int i = 0; i < 8; ++i) dep |= __float_as_uint(v[i].x) | __float_as_uint(o[i].x);
          asm volatile("and.b32 %0, %0, 0;" : "+r"(dep));
          __syncwarp();
          if (lane == 0) {
            arrive_peer_relaxed(peer_x_free + dep);          // the peer's copy for the next block may come
            mbar_arrive(&xs_free[(g & 1) + dep]);            // ... and our staging buffer may be refilled
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            // (rank 0's half first on both sides: the two CTAs then hold the same bits)
            float t0 = (rank == 0 ? o[i].x + v[i].x : v[i].x + o[i].x) * p.sc;
            float t1 = (rank == 0 ? o[i].y + v[i].y : v[i].y + o[i].y) * p.sc;
            float t2 = (rank == 0 ? o[i].z + v[i].z : v[i].z + o[i].z) * p.sc;
            float t3 = (rank == 0 ? o[i].w + v[i].w : v[i].w + o[i].w) * p.sc;
            if (tail) {
              if (kb + 4 * i >= w.k1) t0 = -INFINITY;
              if (kb + 4 * i + 1 >= w.k1) t1 = -INFINITY;
              if (kb + 4 * i + 2 >= w.k1) t2 = -INFINITY;
              if (kb + 4 * i + 3 >= w.k1) t3 = -INFINITY;
            }
            s[4 * i] = __float_as_uint(t0); s[4 * i + 1] = __float_as_uint(t1);
            s[4 * i + 2] = __float_as_uint(t2); s[4 * i + 3] = __float_as_uint(t3);
            bm = fmaxf(bm, fmaxf(fmaxf(t0, t1), fmaxf(t2, t3)));
          }
        }
        if (quarter == 0) PAIR_E(2 + grp, g, 8);
        smax[((g & 1) * 2 + grp) * 128 + head] = bm;
        __syncwarp();
        if (lane == 0) mbar_arrive(&xch[quarter]);
        ok = mbar_wait(&xch[quarter], nx & 1);
        ++nx;
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (quarter == 0) PAIR_E(2 + grp, g, 4);
        bm = fmaxf(bm, smax[((g & 1) * 2 + (grp ^ 1)) * 128 + head]);
        float alpha = 1.f;
        if (bm > m + kLazy || m == -INFINITY) {              // (also true while m is -inf and bm is finite)
          const float m_new = fmaxf(m, bm);
          const float mu = (m_new == -INFINITY) ? 0.f : m_new;
          alpha = ex2(m - mu);                               // 0 for a first block
          m = m_new;
        }
        const float mu = (m == -INFINITY) ? 0.f : m;
        float ps = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float pv = ex2(__uint_as_float(s[e]) - mu);
          ps += pv;
          s[e] = __float_as_uint(pv);
        }
        l = l * alpha + ps;
        if (quarter == 0) PAIR_E(2 + grp, g, 5);
        if (g >= 1) {                                        // P is free, and O complete, once the previous P.V is done
          ok = mbar_wait(pv_done, (uint32_t)((g - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
          tc_fence_after();
        }
        if (quarter == 0) PAIR_E(2 + grp, g, 9);
        // O of this warp's heads, this group's 128 columns, is rescaled when some head's reference moved (warp-uniform)
        if (j > 0 && __any_sync(0xffffffffu, alpha != 1.f)) {
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            uint32_t t[32];
            tmem_ld32(tO + c * 32, t);
            tmem_ld_wait();
#pragma unroll
            for (int e = 0; e < 32; ++e) t[e] = __float_as_uint(__uint_as_float(t[e]) * alpha);
            tmem_st32(tO + c * 32, t);
          }
          tmem_st_wait();
        }
        {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]), p.bf16);
          if (quarter == 0) PAIR_E(2 + grp, g, 10);
          tmem_st16(tPw, pk);
          tmem_st_wait();
          if (quarter == 0) PAIR_E(2 + grp, g, 11);
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full);
        }
        if (quarter == 0) PAIR_E(2 + grp, g, 6);
      }
      if (timed_out) break;
      // row sums of the two key halves
      ssum[((nx & 1) * 2 + grp) * 128 + head] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&xch[quarter]);
      {
        const bool ok = mbar_wait(&xch[quarter], nx & 1);
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      }
      l += ssum[((nx & 1) * 2 + (grp ^ 1)) * 128 + head];
      ++nx;

      // ---- emit: O from tensor memory, 32 columns at a time --------------------------------------------------
      if (w.nblk > 0) {
        const bool ok = mbar_wait(pv_done, (uint32_t)((base + w.nblk - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        tc_fence_after();
      }
      const size_t part = (size_t)cl * 2 + (u == u_first ? 0 : 1);
      const float inv = l > 0.f ? 1.f / l : 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t t[32];
        if (w.nblk > 0) {
          tmem_ld32(tO + c * 32, t);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int e = 0; e < 32; ++e) t[e] = 0u;
        }
        if (w.whole) {
          __half* dst = p.out + ((size_t)u * kMH + head) * kDV + rank * 256 + grp * 128 + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2(__uint_as_float(t[8 * i]) * inv, __uint_as_float(t[8 * i + 1]) * inv, p.bf16);
            v.y = pack2(__uint_as_float(t[8 * i + 2]) * inv, __uint_as_float(t[8 * i + 3]) * inv, p.bf16);
            v.z = pack2(__uint_as_float(t[8 * i + 4]) * inv, __uint_as_float(t[8 * i + 5]) * inv, p.bf16);
            v.w = pack2(__uint_as_float(t[8 * i + 6]) * inv, __uint_as_float(t[8 * i + 7]) * inv, p.bf16);
            reinterpret_cast<uint4*>(dst)[i] = v;
          }
        } else {
          // partial record of all 512 value columns, stored [column group of 4][head][4] so that a warp writes 512
          // contiguous bytes; m and l are the same in both CTAs
          float4* dst = reinterpret_cast<float4*>(p.part_o) + (part * 128 + rank * 64 + grp * 32 + c * 8) * kMH + head;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[(size_t)i * kMH] = make_float4(__uint_as_float(t[4 * i]), __uint_as_float(t[4 * i + 1]),
                                               __uint_as_float(t[4 * i + 2]), __uint_as_float(t[4 * i + 3]));
        }
      }
      if (!w.whole && grp == 0 && rank == 0) {
        p.part_ml[(part * kMH + head) * 2] = m;
        p.part_ml[(part * kMH + head) * 2 + 1] = l;
      }
      if (w.nblk > 0) {
        // O may be overwritten by the next request's first P.V
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(o_free);
        base += w.nblk;
      }
    }
  } else if (warp < kWarpGather0 + kGatherWarps) {
    // ------------------------------------------------------------------------------ gather producers
    const int pw = warp - kWarpGather0;                 // rows [16 pw, 16 pw + 16) of every key block
    const int rsub = lane >> 3, c8 = lane & 7;          // 4 rows per instruction, 8 lanes (128 B) per row
    const int cb0 = rank * 4;                           // first column block of the rows this CTA holds
    int rbase = 0;                                      // ring entries of the requests before this one
    int gb = 0;                                         // key blocks of the requests before this one (trace only)
    for (int u = u_first; u <= u_last && !timed_out; ++u) {
      const UnitWork w = unit_work(p, u, slot0, slot1);
      if (w.nblk == 0) continue;
      const int32_t* idxb = p.idx + (size_t)u * kTopK;
      // position in the request's cache -> row of the tensor (request base or page base); -1 = a row of zeros
      auto row_of = [&](int ridx) -> long long {
        if (ridx < 0) return -1;
        if (p.page_table == nullptr) return (long long)u * p.L + ridx;
        const int pi = ridx / p.page_size;
        const int pg = p.page_table[(size_t)u * p.table_stride + pi];
        return (pg >= 0 && pg < p.pages) ? (long long)pg * p.page_size + (ridx - pi * p.page_size) : -1;   // outside the pool: zeros
      };
      // ---- the request's queries: two entries of 64 rows, five TMA boxes of 64 x 64 each
      for (int e = 0; e < kQEntries && !timed_out; ++e) {
        const int r = rbase + e, s = r % kStages;
        if (r >= kStages) {
          const bool ok = mbar_wait(&empty[s], (uint32_t)(((r / kStages) - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        }
        if (pw == 0 && lane == 0) {
          uint8_t* st = sK + s * kSlot;
          mbar_expect_tx(&full[s], kSlot);              // this lane's arrival, and the bytes to come
#pragma unroll
          for (int c = 0; c < kSlotBlocks; ++c)
            tma_load_3d(st + c * kBlkBytes, &p.tmQ, (cb0 + c) * 64, e * 64, u, &full[s]);
        } else {
          mbar_arrive(&full[s]);
        }
      }
      // ---- its key blocks.  Lanes 0-15 (and their mirrors 16-31) each look up one row of this warp's sixteen: its
      // position in the cache (-1 = a row of zeros), then its row in the tensor.  The positions are loaded one block
      // ahead of their use, so that their latency is off the path; the rows of the block kPrefetch ahead are asked
      // into L2 (lanes 0-15: one row of 640 bytes each): a row comes from HBM in about 2 k cycles, more than the
      // ring's three slots cover at the rate the blocks are consumed.
      auto load_idx = [&](int blk) -> int {
        const int krow = w.k0 + blk * kBK + pw * 16 + (lane & 15);
        return (blk < w.nblk && krow < w.k1) ? idxb[krow] : -1;
      };
      auto prefetch_row = [&](int pidx) {
        if (lane < 16 && pidx >= 0 && pidx < p.L) {
          const long long pc = row_of(pidx);
          if (pc >= 0) l2_prefetch(reinterpret_cast<const uint8_t*>(p.kv + (size_t)pc * kDK) + cb0 * 128, kSlotBlocks * 128);
        }
      };
      int cur = load_idx(0);
      for (int ja = 1; ja < kPrefetch; ++ja) prefetch_row(load_idx(ja));
      int pf = load_idx(kPrefetch);
      for (int j = 0; j < w.nblk && !timed_out; ++j) {
        const int r = rbase + kQEntries + j, s = r % kStages;
        uint8_t* st = sK + s * kSlot;
        const int nxt = load_idx(j + 1), pf_nxt = load_idx(j + 1 + kPrefetch);   // used in the next iteration
        int ridx = cur;
        if (ridx >= p.L) {
          report(p.status, kStatusBadIndex);
          ridx = 0;
        }
        const long long coord = row_of(ridx);
        prefetch_row(pf);
        cur = nxt;
        pf = pf_nxt;
        if (pw == 0) PAIR_E(1, gb + j, 0);
        if (r >= kStages) {
          const bool ok = mbar_wait(&empty[s], (uint32_t)(((r / kStages) - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        }
        if (pw == 0) PAIR_E(1, gb + j, 1);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int lr = 4 * i + rsub;                  // row of this warp's sixteen
          const long long c = __shfl_sync(0xffffffffu, coord, lr);
          const bool valid = c >= 0;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv + (size_t)(valid ? c : 0) * kDK) + cb0 * 128 + c8 * 16;
          const int row = pw * 16 + lr;
          uint8_t* dst = st + row * 128 + ((c8 ^ (row & 7)) << 4);
#pragma unroll
          for (int blk = 0; blk < kSlotBlocks; ++blk)
            cp_async16(dst + blk * kBlkBytes, src + blk * 128, valid ? 16 : 0);
        }
        // this lane's arrival happens when its copies have landed; the warp moves on to the next entry at once.
        // The copies are generic-proxy writes: the issuing threads fence before they read the slot through the
        // tensor core's proxy
        cp_async_arrive_noinc(&full[s]);
        if (pw == 0) PAIR_E(1, gb + j, 2);
      }
      rbase += kQEntries + w.nblk;
      gb += w.nblk;
    }
    // no copy outlives the CTA, on the give-up path either
    cp_async_commit();
    cp_async_wait<0>();
  } else if (warp >= kWarpExch0) {
    // ------------------------------------------------------------------------------ exchange warps
    // Warp w takes the 32 heads of tensor-memory lane quarter w % 4: the block's 64 partial scores of each head go
    // to registers (the score columns are then free for the next Q.K^T), to the staging buffer, where this CTA's
    // softmax threads find them, and from there by one asynchronous 8 KiB copy into the peer's shared memory,
    // completing on the peer's barrier.  The 32 KiB of a block take about 2 k cycles to cross; done here, a block
    // ahead of the softmax, the transfer is off its path.
    const int quarter = warp & 3;
    const uint32_t tS = tmem_base + ((uint32_t)(quarter * 32) << 16) + kColS;
    const uint32_t peer = (uint32_t)(rank ^ 1);
    const uint32_t peer_x = peer_addr(xbuf + (quarter * 16) * 32, peer);
    const uint32_t peer_x_full = peer_addr(x_full, peer);
    const int head = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    int g = 0, rbase = 0;                               // blocks / ring entries of the requests before this one
    for (int u = u_first; u <= u_last && !timed_out; ++u) {
      const UnitWork w = unit_work(p, u, slot0, slot1);
      if (w.nblk == 0) continue;
      {
        // This head's share of the request's queries: from the ring entry that holds its row (rows 0-63 in the
        // request's first entry, 64-127 in its second) to tensor memory, two 16-bit values per column.  The CTA's
        // 288 elements are 36 chunks of 16 bytes, starting 4 rank chunks into the five blocks.  Every Q.K^T of the
        // request before has completed: this warp has taken its last scores out of tensor memory.  Done here, the
        // next request's first scores are on their way while the softmax threads still write the last one out.
        const int rq = rbase + (head >> 6), sq = rq % kStages;
        const bool okq = mbar_wait(&full[sq], (uint32_t)((rq / kStages) & 1));
        if (!__all_sync(0xffffffffu, okq)) { timed_out = true; break; }
        const uint8_t* qs = sK + sq * kSlot;
        const int qrow = head & 63;
#pragma unroll 1
        for (int c = 0; c < 9; ++c) {
          uint32_t rr[16];
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ch = rank * 4 + c * 4 + i;
            const uint4 v = *reinterpret_cast<const uint4*>(qs + (ch >> 3) * kBlkBytes + swz128(qrow, ch & 7));
            rr[4 * i] = v.x; rr[4 * i + 1] = v.y; rr[4 * i + 2] = v.z; rr[4 * i + 3] = v.w;
          }
          tmem_st16(lane_base + kColQ + c * 16, rr);
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_full);
      }
      for (int j = 0; j < w.nblk; ++j, ++g) {
        bool ok = mbar_wait(s_full, (uint32_t)(g & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (quarter == 0) PAIR_E(4, g, 0);
        tc_fence_after();
        uint32_t s0[32], s1[32];
        tmem_ld32(tS, s0);
        tmem_ld32(tS + 32, s1);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);
        if (quarter == 0) PAIR_E(4, g, 1);
        // the staging buffer of two blocks back has been read by our softmax threads; the peer has read the block
        // before (so its buffer is free, and our copy out of this staging buffer, older still, is complete)
        if (g >= 2) ok = mbar_wait(&xs_free[g & 1], (uint32_t)(((g >> 1) - 1) & 1));
        if (ok && g >= 1) ok = mbar_wait_peer_relaxed(x_free, (uint32_t)((g - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (quarter == 0) PAIR_E(4, g, 2);
        float4* snd = xsend + (g & 1) * (kXBytes / 16) + (quarter * 16) * 32 + lane;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          snd[i * 32] = make_float4(__uint_as_float(s0[4 * i]), __uint_as_float(s0[4 * i + 1]), __uint_as_float(s0[4 * i + 2]),
                                    __uint_as_float(s0[4 * i + 3]));
          snd[(8 + i) * 32] = make_float4(__uint_as_float(s1[4 * i]), __uint_as_float(s1[4 * i + 1]),
                                          __uint_as_float(s1[4 * i + 2]), __uint_as_float(s1[4 * i + 3]));
        }
        fence_proxy_async();                                   // the copy reads what these threads just wrote
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(&xs_full[g & 1]);
          bulk_copy_to_peer(peer_x, snd - lane, kXBytes / 4, peer_x_full);
        }
        if (quarter == 0) PAIR_E(4, g, 3);
      }
      rbase += kQEntries + w.nblk;
    }
  } else if (warp == kWarpQK) {
    // ------------------------------------------------------------------------------ Q.K^T issuer
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_16(128, kBK, 0, p.bf16);
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      // (the address field is 14 bits: inside a cluster a CTA's shared-memory addresses carry higher bits, which
      // must not spill into the descriptor's other fields)
      const uint32_t k_lo = (uint32_t)umma_desc_sw128(0) + ((smem_u32(sK) >> 4) & 0x3FFF);
      const uint32_t tQ = tmem_base + kColQ, tS = tmem_base + kColS;
      int base = 0, rbase = 0, units = 0;               // blocks / ring entries / non-empty requests before this one
      for (int u = u_first; u <= u_last && !timed_out; ++u) {
        const UnitWork w = unit_work(p, u, slot0, slot1);
        if (w.nblk == 0) continue;
        // the exchange warps have copied the request's queries out of their two entries: hand the slots back
        if (!mbar_wait(q_full, (uint32_t)(units & 1))) { timed_out = true; break; }
        for (int e = 0; e < kQEntries; ++e) umma_commit(&empty[(rbase + e) % kStages]);
        for (int j = 0; j < w.nblk; ++j) {
          const int g = base + j, r = rbase + kQEntries + j, s = r % kStages;
          if (!mbar_wait(&full[s], (uint32_t)((r / kStages) & 1))) { timed_out = true; break; }
          PAIR_E(0, g, 0);
          if (g >= 1 && !mbar_wait(s_free, (uint32_t)((g - 1) & 1))) { timed_out = true; break; }
          PAIR_E(0, g, 1);
          fence_proxy_async();                          // rows written by cp.async, read by the tensor core
          tc_fence_after();
          const uint32_t kb_lo = k_lo + s * (kSlot >> 4);
#pragma unroll
          for (int kk = 0; kk < kKSteps; ++kk) {
            const int kq = rank * 2 + kk;               // 32-byte step inside the five blocks this CTA holds
            umma_f16_ts(tS, tQ + kk * 8, kb_lo + (kq >> 2) * (kBlkBytes >> 4) + (kq & 3) * 2, hi_k, idesc_qk,
                        kk > 0 ? 1u : 0u);
          }
          umma_commit(s_full);
          PAIR_E(0, g, 2);
        }
        base += w.nblk;
        rbase += kQEntries + w.nblk;
        ++units;
      }
    }
  } else if (warp == kWarpPV) {
    // ------------------------------------------------------------------------------ P.V issuer
    if (lane == 0) {
      const uint32_t idesc_pv = umma_idesc_16(128, 256, 1, p.bf16);
      const uint32_t hi_v = (uint32_t)(umma_desc_sw128_mn(0, kBlkBytes, 1024) >> 32);
      const uint32_t v_lo = (uint32_t)umma_desc_sw128_mn(0, kBlkBytes, 1024) + ((smem_u32(sK) >> 4) & 0x3FFF);
      const uint32_t tO = tmem_base + kColT, tP = tmem_base + kColP;
      int base = 0, rbase = 0, units = 0;
      for (int u = u_first; u <= u_last && !timed_out; ++u) {
        const UnitWork w = unit_work(p, u, slot0, slot1);
        if (w.nblk == 0) continue;
        // the request's first P.V starts O afresh: the request before must have been written out
        if (units >= 1 && !mbar_wait(o_free, (uint32_t)((units - 1) & 1))) { timed_out = true; break; }
        for (int j = 0; j < w.nblk; ++j) {
          const int g = base + j, s = (rbase + kQEntries + j) % kStages;
          if (!mbar_wait(p_full, (uint32_t)(g & 1))) { timed_out = true; break; }
          PAIR_E(0, g, 3);
          fence_proxy_async();
          tc_fence_after();
          // the value columns are the first four blocks of the slot: [64 keys][256 columns], MN-major
          const uint32_t vb = v_lo + s * (kSlot >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_f16_ts(tO, tP + k * 8, vb + k * (2048 >> 4), hi_v, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(pv_done);
          umma_commit(&empty[s]);
          PAIR_E(0, g, 5);
        }
        base += w.nblk;
        rbase += kQEntries + w.nblk;
        ++units;
      }
    }
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: the cluster meets (the peer copies into this CTA's shared memory until its last block), then the
  // allocating warp frees the tensor memory
  tc_fence_before();
  cluster_sync_all();
  if (warp == kWarpPV) {
    tc_fence_after();
    tmem_free(tmem_base, kCols);
  }
}

#ifdef VMK_MLA_TIMING
extern "C" VMK_API int vmk_debug_pair_trace(long long* out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_pair_trace, sizeof(long long) * 640);
}
#endif

// Merge of the requests a range boundary cuts.  Grid (ncl, 4, 8), 256 threads: CTA (c, hq, z) looks at the
// boundary where range c starts; if it lies inside a request and is the first such boundary of that request, it
// merges the request's partials (the last record of range c - 1, then the first record of ranges c, c + 1, ...
// while they start inside the request) for heads [32 hq, 32 hq + 32): lane = head, CTA z and warp w = the two
// column groups of four [16 z + 2 w, 16 z + 2 w + 2).
__global__ void __launch_bounds__(256) mla_pair_combine_kernel(const float* __restrict__ part_o,
                                                               const float* __restrict__ part_ml, int B, int ncl,
                                                               __half* __restrict__ out, int bf16) {
  const int c = blockIdx.x;
  const int total = B * kUnitSlots;
  const int s = range_start(c, total, ncl);
  pdl_wait();                                           // launched as a programmatic dependent of mla_pair_kernel
  if (c == 0 || s % kUnitSlots == 0) return;
  const int u = s / kUnitSlots;
  const int prev = range_start(c - 1, total, ncl);
  if (prev > u * kUnitSlots) return;                    // an earlier boundary inside the request does the merge
  const int head = blockIdx.y * 32 + (threadIdx.x & 31), cg0 = blockIdx.z * 16 + (threadIdx.x >> 5) * 2;
  const int unit_end = (u + 1) * kUnitSlots;
  // range c - 1 holds this request as its last one (record 1) unless it is also its first
  const size_t part_prev = (size_t)(c - 1) * 2 + (prev / kUnitSlots == u ? 0 : 1);
  int c_end = c;
  while (c_end < ncl && range_start(c_end, total, ncl) < unit_end) ++c_end;
  // Parts: t = 0 the record range c - 1 left, t >= 1 the first record of range c + t - 1.  Merged four at a time
  // with a running maximum, so that the loads of a group are all in flight together.
  const int nparts = 1 + (c_end - c);
  float M = -INFINITY, lsum = 0.f;
  float4 acc[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) acc[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int t0 = 0; t0 < nparts; t0 += 4) {
    float m[4], l[4];
    float4 o[4][2];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const int t = t0 + k;
      const bool on = t < nparts;
      const size_t part = t == 0 ? part_prev : (size_t)(c + t - 1) * 2;
      m[k] = -INFINITY;
      l[k] = 0.f;
      o[k][0] = o[k][1] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (on) {
        const float2 ml = *reinterpret_cast<const float2*>(part_ml + (part * kMH + head) * 2);
        m[k] = ml.x;
        l[k] = ml.y;
        const float4* src = reinterpret_cast<const float4*>(part_o) + (part * 128 + cg0) * kMH + head;
        o[k][0] = src[0];
        o[k][1] = src[kMH];
      }
    }
    const float Mn = fmaxf(fmaxf(fmaxf(m[0], m[1]), fmaxf(m[2], m[3])), M);
    const float mu = (Mn == -INFINITY) ? 0.f : Mn;
    const float a = exp2f(M - mu);                        // 0 while nothing has been accumulated (M = -inf)
    acc[0].x *= a; acc[0].y *= a; acc[0].z *= a; acc[0].w *= a;
    acc[1].x *= a; acc[1].y *= a; acc[1].z *= a; acc[1].w *= a;
    lsum *= a;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float w = (m[k] == -INFINITY) ? 0.f : exp2f(m[k] - mu);
      acc[0].x += w * o[k][0].x; acc[0].y += w * o[k][0].y; acc[0].z += w * o[k][0].z; acc[0].w += w * o[k][0].w;
      acc[1].x += w * o[k][1].x; acc[1].y += w * o[k][1].y; acc[1].z += w * o[k][1].z; acc[1].w += w * o[k][1].w;
      lsum += w * l[k];
    }
    M = Mn;
  }
  const float inv = 1.f / lsum;
  __half* dst = out + ((size_t)u * kMH + head) * kDV + cg0 * 4;
  uint4 v;
  v.x = pack2(acc[0].x * inv, acc[0].y * inv, bf16);
  v.y = pack2(acc[0].z * inv, acc[0].w * inv, bf16);
  v.z = pack2(acc[1].x * inv, acc[1].y * inv, bf16);
  v.w = pack2(acc[1].z * inv, acc[1].w * inv, bf16);
  *reinterpret_cast<uint4*>(dst) = v;
}

namespace {

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

cudaError_t configure_once() {
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev == dev) return cudaSuccess;
  cudaError_t e = cudaFuncSetAttribute(mla_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmem);
  if (e == cudaSuccess) configured_dev = dev;
  return e;
}

// Clusters of two that can be resident together (a GPC with an odd number of SMs leaves one unpaired).
int max_pairs() {
  static int cached_dev = -1, cached = 0;
  int dev = 0;
  cudaGetDevice(&dev);
  if (cached_dev == dev) return cached;
  int n = sm_count() / 2;
  if (configure_once() == cudaSuccess) {
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3(2 * n);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = kSmem;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int q = 0;
    if (cudaOccupancyMaxActiveClusters(&q, mla_pair_kernel, &cfg) == cudaSuccess && q > 0 && q < n) n = q;
    cudaGetLastError();
  }
  if (n < 1) n = 1;
  cached = n;
  cached_dev = dev;
  return n;
}

}  // namespace

// Number of ranges (= clusters).  With at least one request per resident cluster: one cluster per pair of SMs,
// ranges cut wherever they fall.  With fewer requests the ranges may be aligned to the requests instead (every
// request cut into the same power-of-two number of parts): parts per request minimise
// waves x (blocks per part + a fixed cost of about four blocks for loading Q and draining), and the aligned cut
// is taken when that beats the free-running one.
int mla_pair_clusters(int B) {
  const int pairs = max_pairs();
  if (g_batch_invariant) return B * 4;                  // every request cut into the same four parts, whatever B is
  if (B >= pairs) return pairs;
  long long best_cost = -1;
  int best = 1;
  for (int ns = 1; ns <= kUnitSlots / kMinSlotsPerCluster; ns *= 2) {
    const long long cost = (long long)cdiv(B * ns, pairs) * (kUnitSlots / ns + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ns; }
  }
  // free-running ranges pay about three more blocks for the partial records of nearly every request
  const long long free_cost = cdiv(B * kUnitSlots, pairs) + 4 + 3;
  return free_cost < best_cost ? pairs : B * best;
}

// Bytes of the partial (m, l, o[512]) records: two per cluster.
size_t mla_pair_workspace(int B) {
  const size_t n = (size_t)mla_pair_clusters(B) * 2 * kMH;
  return align_up(n * kDV * 4, 256) + align_up(n * 2 * 4, 256);
}

int mla_pair_launch(const MlaTcParams& p0, float* workspace, cudaStream_t stream) {
  cudaError_t e = configure_once();
  if (e != cudaSuccess) return check_launch(e);
  MlaTcParams p = p0;
  p.ncta = mla_pair_clusters(p.B);                      // ranges = clusters
  const size_t n = (size_t)p.ncta * 2 * kMH;
  p.part_o = workspace;
  p.part_ml = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + align_up(n * kDV * 4, 256));
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2 * p.ncta);
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = kSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int rc = check_launch(cudaLaunchKernelEx(&cfg, mla_pair_kernel, p));
  if (rc || p.ncta == 1) return rc;
  cfg.gridDim = dim3(p.ncta, 4, 8);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  cfg.numAttrs = 1;
  return check_launch(cudaLaunchKernelEx(&cfg, mla_pair_combine_kernel, (const float*)p.part_o, (const float*)p.part_ml, p.B,
                                         p.ncta, p.out, p.bf16));
}

}  // namespace vmk
