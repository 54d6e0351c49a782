// `dsa` stage 3 on the 5th-generation tensor cores: absorbed-MLA attention over the selected rows.
//
// The shapes fight the machine: 128 heads x 512 fp32 of output is all of tensor memory, and a 128 x 576
// fp16 query tile is 147 KB of shared memory.  This kernel therefore
//   * keeps Q in TENSOR MEMORY (288 columns of packed fp16 pairs) and feeds it to the MMA as the A operand
//     straight from there, so shared memory only holds the gathered rows;
//   * works in UNITS of (request, value half): all 128 heads but 256 of the 512 value columns, whose
//     output is accumulated in REGISTERS: every 64-key block the product P.V is written to a 128-column
//     scratch area of tensor memory, read back and added, first for value columns [0,128) of the half by
//     softmax group A, then for [128,256) by group B;
//   * is PERSISTENT: the 2 B units of 32 block slots each form one list, cut into equal contiguous ranges,
//     one per CTA (at most one CTA per SM), so that no wave of CTAs is left part-filled.  A unit that lies
//     inside one range is written out directly; a unit cut by a range boundary leaves (m, l, o) partials,
//     at most two per CTA (its first and its last unit), merged by mla_tc_combine_kernel.
// Shared memory is one ring of three 72 KiB slots.  A unit passes through it as the ENTRIES
//     Q rows 0-63, Q rows 64-127, key block 0, key block 1, ...
// each entry nine [64 rows][128 B] blocks with the 128-byte swizzle: for a key block the K-major operand of
// Q.K^T and, for four of its first eight blocks, the MN-major operand of P.V; for a Q entry the staging area
// from which the softmax threads copy their head's query row into tensor memory.  Q entries arrive by plain
// TMA tile loads, key blocks by the row gather.  The ring runs on across unit boundaries: the next unit's
// queries and first rows are fetched while this one drains.
// One CTA = 512 threads in four warp groups, with registers moved from the last two to the first two
// (setmaxnreg: 208 for the softmax threads, which hold 128 accumulators each; 48 for everybody else):
//   warps 0-3   softmax group A, warps 4-7 group B: one thread per head and group.  A takes keys [0,32) of
//               each block, B keys [32,64); the pair of a head exchanges block maxima through shared memory,
//               both store their share of P (packed fp16) to tensor memory, the A operand of P.V
//   warps 8-11  gather: warp w fetches rows [16 w, 16 w + 16) of every key block, by cp.async (8 lanes per row,
//               arrival on the slot's barrier when the copies land) or, in the second variant, by TMA
//               (tile::gather4: four rows x 128 B per instruction).  Four warps because what bounds the gather is
//               the instruction stream: 144 instructions of 512 bytes per block either way, about 50 cycles each
//               for a warp issuing cp.async, and about 35 cycles each for the SM's TMA unit however many warps
//               issue them, which is why the TMA variant is the slower one (5.4 k against 4.7 k cycles per block)
//   warp 12     issues S = Q.K^T: 36 x (M128 N64 K16, A from tensor memory) per block
//   warp 13     owns tensor memory and issues P.V: 4 + 4 x (M128 N128 K16, A = P from tensor memory)
// Ring slots and their barrier phases are indexed by the ring entry, the score / P / scratch barriers by the
// number of key blocks the CTA has processed so far.  Every mbarrier wait is bounded; a wait that runs out sets
// the status word and the CTA winds down through the common exit, where tensor memory is freed.
#include "dsa_mla_tc.cuh"
#include "tcgen05.cuh"

namespace vmk {

constexpr int kMlaTopK = VMK_DSA_TOPK;
constexpr int kMH = 128, kDK = 576, kDV = 512;
constexpr int kBK = 64;                               // keys per block
constexpr int kBlkBytes = kBK * 128;                  // one [64 keys][128 B] swizzled block
constexpr int kKTile = 9 * kBlkBytes;                 // 72 KiB: 64 gathered rows of 576 fp16
constexpr int kMlaStages = 3;
constexpr int kMlaThreads = 512;
constexpr int kGatherWarps = 4;                       // warps 8..11: 16 rows of every key block each
constexpr int kWarpQK = 12, kWarpPV = 13;
constexpr int kQEntries = 2;                          // ring entries that stage a unit's queries
constexpr int kColQ = 0;                              // 288 columns: Q as packed fp16 pairs
constexpr int kColS = 288;                            // 64 columns: scores
constexpr int kColT = 352;                            // 128 columns: P.V scratch
constexpr int kColP = 480;                            // 32 columns: P as packed fp16 pairs
constexpr int kMlaCols = 512;
constexpr int kMlaBars = 3 * kMlaStages + 12;
constexpr int kMlaTcSmem = kMlaStages * kKTile + kMlaBars * 8 + 16 + 8 * 128 * 4 + 1024;

constexpr int kUnitSlots = kMlaTopK / kBK;           // 32 block slots per unit
constexpr int kMinSlotsPerCta = 2;

// First block slot of CTA c when `total` slots are cut into `ncta` ranges.
__host__ __device__ __forceinline__ int range_start(int c, int total, int ncta) {
  return (int)(((long long)c * total) / ncta);
}

// One unit's share of a CTA's range.
struct UnitWork {
  int b, half, k0, k1, nblk;
  bool whole;
};
__device__ __forceinline__ UnitWork unit_work(const MlaTcParams& p, int u, int slot0, int slot1) {
  UnitWork w;
  w.b = u % p.B;
  w.half = u / p.B;
  const int ja = max(slot0 - u * kUnitSlots, 0), jb = min(slot1 - u * kUnitSlots, kUnitSlots);
  const int nb = max(0, min(p.cnt[w.b], kMlaTopK));
  w.k0 = ja * kBK;
  w.k1 = min(nb, jb * kBK);
  w.nblk = w.k1 > w.k0 ? (w.k1 - w.k0 + kBK - 1) / kBK : 0;
  w.whole = ja == 0 && jb == kUnitSlots;
  return w;
}

#ifdef VMK_MLA_TIMING
// Debug build only.  Time stamps of blocks 8..15 of CTA (0,0,0): [role][block - 8][event]
__device__ long long g_mla_trace[4 * 8 * 16];
#define MLA_E(role, j, ev) do { if (blockIdx.x == 0 && (j) >= 8 && (j) < 16 && lane == 0) \
    g_mla_trace[((role) * 8 + (j) - 8) * 16 + (ev)] = clock64(); } while (0)
// CTA-level marks of CTA 0: [mark]
__device__ long long g_mla_marks[16];
__device__ __forceinline__ long long mla_globaltimer() {
  long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
// marks 0..7: SM cycles; 8..15: the same points in nanoseconds of the global timer (for the clock the SM ran at)
#define MLA_M(k) do { if (blockIdx.x == 0 && lane == 0) { g_mla_marks[k] = clock64(); g_mla_marks[8 + (k)] = mla_globaltimer(); } } while (0)
// start and end of every CTA's softmax warp 0 on the global timer: [cta][0 = start, 1 = end]
__device__ long long g_mla_cta_ns[256 * 2];
#define MLA_CTA(k) do { if (lane == 0 && blockIdx.x < 256) g_mla_cta_ns[blockIdx.x * 2 + (k)] = mla_globaltimer(); } while (0)
#else
#define MLA_E(role, j, ev) do {} while (0)
#define MLA_M(k) do {} while (0)
#define MLA_CTA(k) do {} while (0)
#endif

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kMlaThreads, 1) mla_tc_kernel(const __grid_constant__ MlaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                   // [stages][9 blocks][64 rows][128 B]
  uint64_t* full = reinterpret_cast<uint64_t*>(sK + kMlaStages * kKTile);   // entry landed (128 gather lanes + bytes)
  uint64_t* empty = full + kMlaStages;                  // entry consumed by everybody          (MMA commit)
  uint64_t* empty_k = empty + kMlaStages;               // entry consumed by Q.K^T               (MMA commit)
  uint64_t* q_full = empty_k + kMlaStages;              // Q stored to tensor memory            (8 warps)
  uint64_t* s_full = q_full + 1;                        // scores ready                         (MMA commit)
  uint64_t* s_free = s_full + 1;                        // scores consumed                      (8 warps)
  uint64_t* p_full = s_free + 1;                        // P stored to tensor memory            (8 warps)
  uint64_t* pva_done = p_full + 1;                      // first half of P.V in the scratch     (MMA commit)
  uint64_t* pvb_done = pva_done + 1;                    // second half                          (MMA commit)
  uint64_t* ta_free = pvb_done + 1;                     // group A has read the scratch         (4 warps)
  uint64_t* tb_free = ta_free + 1;                      // group B has read the scratch         (4 warps)
  uint64_t* xch = tb_free + 1;                          // [4] pair of warps that share 32 heads exchanged values
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(xch + 4);
  float* smax = reinterpret_cast<float*>(tmem_slot + 4);    // [2 parities][2 groups][128 heads] block maxima
  float* ssum = smax + 4 * 128;                             // [2 parities][2 groups][128 heads] row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int total_slots = 2 * p.B * kUnitSlots;
  const int slot0 = range_start(blockIdx.x, total_slots, p.ncta), slot1 = range_start(blockIdx.x + 1, total_slots, p.ncta);
  const int u_first = slot0 / kUnitSlots, u_last = (slot1 - 1) / kUnitSlots;

  if (tid == 0) {
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(&full[s], kGatherWarps * 32);
      mbar_init(&empty[s], 1);
      mbar_init(&empty_k[s], 1);
    }
    mbar_init(q_full, 8);
    mbar_init(s_full, 1);
    mbar_init(s_free, 8);
    mbar_init(p_full, 8);
    mbar_init(pva_done, 1);
    mbar_init(pvb_done, 1);
    mbar_init(ta_free, 4);
    mbar_init(tb_free, 4);
    for (int q = 0; q < 4; ++q) mbar_init(&xch[q], 2);
    fence_mbar_init();
  }
  if (warp == kWarpPV) tmem_alloc(tmem_slot, kMlaCols);
  if (warp == 8 && lane == 0) {
    tma_prefetch_desc(&p.tmQ);
    if (p.gather_tma) tma_prefetch_desc(&p.tmKV);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // Launched as a programmatic dependent: everything above overlaps the tail of the kernel before (the top-k
  // selection, in the fused call); the candidate lists and counts are read only below this line.
  asm volatile("griddepcontrol.wait;" ::: "memory");

  bool timed_out = false;
  // Registers go where the accumulators are: the two softmax warp groups take 208 each, the gather and issuing
  // warp groups keep 48 (2 x 128 x 208 + 2 x 128 x 48 = 64 K, the register file).  Each side changes its share
  // as the first thing in its own branch; the branches meet again only at the common exit.
  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
  if (warp < 8 + kGatherWarps) {
    // ------------------------------------------------------------------------------ gather producers
    const int pw = warp - 8;                            // rows [16 pw, 16 pw + 16) of every key block
    const int rsub = lane >> 3, c8 = lane & 7;          // cp.async: 4 rows per instruction, 8 lanes (128 B) per row
    int rbase = 0;                                      // ring entries of the units before this one
    int base_blocks = 0;                                // key blocks of the units before this one (trace only)
    int last_r = -1;                                    // last ring entry this warp took part in
    bool last_tma = false;                              // ... and whether its bytes come by TMA
    for (int u = u_first; u <= u_last && !timed_out; ++u) {
      const UnitWork w = unit_work(p, u, slot0, slot1);
      if (w.nblk == 0) continue;
      const int32_t* idxb = p.idx + (size_t)w.b * kMlaTopK;
      const int own = w.half * 4, other = 4 - own;
      // ---- the unit's queries: two entries of 64 rows, nine TMA boxes of 64 x 64 each
      for (int e = 0; e < kQEntries && !timed_out; ++e) {
        const int r = rbase + e, s = r % kMlaStages;
        if (r >= kMlaStages) {
          const bool ok = mbar_wait(&empty[s], (uint32_t)(((r / kMlaStages) - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        }
        if (pw == 0 && lane == 0) {
          uint8_t* st = sK + s * kKTile;
          mbar_expect_tx(&full[s], kKTile);             // this lane's arrival, and the bytes to come
#pragma unroll
          for (int c = 0; c < 9; ++c) tma_load_3d(st + c * kBlkBytes, &p.tmQ, c * 64, e * 64, w.b, &full[s]);
        } else {
          mbar_arrive(&full[s]);
        }
        last_r = r;
        last_tma = true;
      }
      // ---- its key blocks
      for (int j = 0; j < w.nblk && !timed_out; ++j) {
        const int r = rbase + kQEntries + j, s = r % kMlaStages;
        uint8_t* st = sK + s * kKTile;
        // lanes 0-15 (and their mirrors 16-31) each look up one row of this warp's sixteen: its position in the
        // cache, then its row in the tensor the loads address (request base or page base); -1 = a row of zeros
        const int krow = w.k0 + j * kBK + pw * 16 + (lane & 15);
        int ridx = krow < w.k1 ? idxb[krow] : -1;
        if (ridx >= p.L) {
          report(p.status, kStatusBadIndex);
          ridx = 0;
        }
        int coord = -1;
        if (ridx >= 0) {
          if (p.page_table == nullptr) {
            coord = w.b * p.L + ridx;
          } else {
            const int pi = ridx / p.page_size;
            const int pg = p.page_table[(size_t)w.b * p.table_stride + pi];
            coord = (pg >= 0 && pg < p.pages) ? pg * p.page_size + (ridx - pi * p.page_size) : -1;   // outside the pool: zeros
          }
        }
        // Two passes over the rows.  Pass 0 fetches the five column blocks only Q.K^T reads (the other value
        // half and the rope block): their part of the slot is free as soon as Q.K^T of the entry three back is
        // done, one block earlier than the four value blocks of pass 1, which its P.V still reads.  That only
        // holds while that entry is a key block of this unit: another unit may have the other value half.
        if (p.gather_tma) {
          int r4[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int c = __shfl_sync(0xffffffffu, coord, (4 * lane + k) & 15);
            r4[k] = c < 0 ? p.rows_total : c;           // beyond the tensor: TMA fills the row with zeros
          }
          uint8_t* dst = st + (pw * 16 + 4 * (lane & 3)) * 128;   // lane l < 4: rows [4 l, 4 l + 4) of this warp's 16
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            if (r >= kMlaStages) {
              const uint32_t par = (uint32_t)(((r / kMlaStages) - 1) & 1);
              const bool ok = mbar_wait(pass == 0 && j >= kMlaStages ? &empty_k[s] : &empty[s], par);
              if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
            }
            MLA_E(1, base_blocks + j, pass * 2);
            if (pass == 0) {
              // every lane's arrival stands before the first byte can land; lane 0 also announces the 16 rows
              if (lane == 0) mbar_expect_tx(&full[s], 16 * kDK * 2); else mbar_arrive(&full[s]);
              __syncwarp();
            }
            if (lane < 4) {
              const int first = pass == 0 ? other : own;
#pragma unroll
              for (int blk = 0; blk < 4; ++blk)
                tma_gather4(dst + (first + blk) * kBlkBytes, &p.tmKV, (first + blk) * 64, r4[0], r4[1], r4[2], r4[3], &full[s]);
              if (pass == 0) tma_gather4(dst + 8 * kBlkBytes, &p.tmKV, 8 * 64, r4[0], r4[1], r4[2], r4[3], &full[s]);
            }
            MLA_E(1, base_blocks + j, pass * 2 + 1);
          }
          if (timed_out) break;
          last_r = r;
          last_tma = true;
        } else {
#pragma unroll 1
          for (int pass = 0; pass < 2; ++pass) {
            if (r >= kMlaStages) {
              const uint32_t par = (uint32_t)(((r / kMlaStages) - 1) & 1);
              const bool ok = mbar_wait(pass == 0 && j >= kMlaStages ? &empty_k[s] : &empty[s], par);
              if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
            }
            MLA_E(1, base_blocks + j, pass * 2);
            const int first = pass == 0 ? other : own;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int lr = 4 * i + rsub;              // row of this warp's sixteen
              const int c = __shfl_sync(0xffffffffu, coord, lr);
              const bool valid = c >= 0;
              const uint8_t* src = reinterpret_cast<const uint8_t*>(p.kv + (size_t)(valid ? c : 0) * kDK) + c8 * 16;
              const int row = pw * 16 + lr;
              uint8_t* dst = st + row * 128 + ((c8 ^ (row & 7)) << 4);
#pragma unroll
              for (int blk = 0; blk < 4; ++blk)
                cp_async16(dst + (first + blk) * kBlkBytes, src + (first + blk) * 128, valid ? 16 : 0);
              if (pass == 0) cp_async16(dst + 8 * kBlkBytes, src + 8 * 128, valid ? 16 : 0);
            }
            MLA_E(1, base_blocks + j, pass * 2 + 1);
          }
          if (timed_out) break;
          // this lane's arrival happens when its copies have landed; the warp moves on to the next entry at once.
          // The copies are generic-proxy writes: the issuing threads fence before they read the slot through the
          // tensor core's proxy
          cp_async_arrive_noinc(&full[s]);
          last_r = r;
          last_tma = false;
        }
      }
      rbase += kQEntries + w.nblk;
      base_blocks += w.nblk;
    }
    // No copy outlives the CTA, on the give-up path either: the cp.async copies are waited for here; the bytes of
    // a last entry filled by TMA have landed once its barrier phase is over (without a timeout the consumers have
    // waited for it already and this returns at once; the entry is the newest of its slot, so the parity is current)
    cp_async_commit();
    cp_async_wait<0>();
    if (last_r >= 0 && last_tma && !timed_out)
      mbar_wait(&full[last_r % kMlaStages], (uint32_t)((last_r / kMlaStages) & 1));
  } else if (warp == kWarpQK) {
    // ------------------------------------------------------------------------------ Q.K^T issuer
    // The tensor pipe buffers only an instruction or two, so every wait of an issuing thread drains it.  Two
    // issuers (this warp for S = Q . K^T, the next for P . V) keep it fed: while one waits for a hand-over,
    // the other's instructions run.
    if (lane == 0) {
      const uint32_t idesc_qk = umma_idesc_16(128, kBK, 0, p.bf16);
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      const uint32_t k_lo = (uint32_t)umma_desc_sw128(0) + (smem_u32(sK) >> 4);
      const uint32_t tQ = tmem_base + kColQ, tS = tmem_base + kColS;
      int base = 0, rbase = 0, units = 0;               // blocks / ring entries / non-empty units before this one
      for (int u = u_first; u <= u_last && !timed_out; ++u) {
        const UnitWork w = unit_work(p, u, slot0, slot1);
        if (w.nblk == 0) continue;
        // the softmax threads have copied the unit's queries out of their two entries: hand the slots back
        if (!mbar_wait(q_full, (uint32_t)(units & 1))) { timed_out = true; break; }
        for (int e = 0; e < kQEntries; ++e) {
          umma_commit(&empty[(rbase + e) % kMlaStages]);
          umma_commit(&empty_k[(rbase + e) % kMlaStages]);
        }
        for (int j = 0; j < w.nblk; ++j) {
          const int g = base + j, r = rbase + kQEntries + j, s = r % kMlaStages;
          if (!mbar_wait(&full[s], (uint32_t)((r / kMlaStages) & 1))) { timed_out = true; break; }
          MLA_E(0, g, 0);
          if (g >= 1 && !mbar_wait(s_free, (uint32_t)((g - 1) & 1))) { timed_out = true; break; }
          MLA_E(0, g, 1);
          if (!p.gather_tma) fence_proxy_async();       // rows written by cp.async, read by the tensor core
          tc_fence_after();
          const uint32_t kb_lo = k_lo + s * (kKTile >> 4);
#pragma unroll 12
          for (int kk = 0; kk < 36; ++kk)
            umma_f16_ts(tS, tQ + kk * 8, kb_lo + (kk >> 2) * (kBlkBytes >> 4) + (kk & 3) * 2, hi_k, idesc_qk,
                        kk > 0 ? 1u : 0u);
          umma_commit(s_full);
          umma_commit(&empty_k[s]);
          MLA_E(0, g, 2);
        }
        base += w.nblk;
        rbase += kQEntries + w.nblk;
        ++units;
      }
    }
  } else if (warp == kWarpPV) {
    // ------------------------------------------------------------------------------ P.V issuer
    if (lane == 0) {
      const uint32_t idesc_pv = umma_idesc_16(128, 128, 1, p.bf16);
      const uint32_t hi_v = (uint32_t)(umma_desc_sw128_mn(0, kBlkBytes, 1024) >> 32);
      const uint32_t v_lo = (uint32_t)umma_desc_sw128_mn(0, kBlkBytes, 1024) + (smem_u32(sK) >> 4);
      const uint32_t tT = tmem_base + kColT, tP = tmem_base + kColP;
      int base = 0, rbase = 0;
      for (int u = u_first; u <= u_last && !timed_out; ++u) {
        const UnitWork w = unit_work(p, u, slot0, slot1);
        if (w.nblk == 0) continue;
        // One 128-column part of P_g . V_g into the scratch.
        auto issue_pv_part = [&](int s, int part) {
          const uint32_t vb = v_lo + s * (kKTile >> 4) + (w.half * 4 + part * 2) * (kBlkBytes >> 4);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16_ts(tT, tP + k * 8, vb + k * (2048 >> 4), hi_v, idesc_pv, k > 0 ? 1u : 0u);
        };
        for (int j = 0; j < w.nblk; ++j) {
          const int g = base + j, s = (rbase + kQEntries + j) % kMlaStages;
          if (!mbar_wait(p_full, (uint32_t)(g & 1))) { timed_out = true; break; }
          MLA_E(0, g, 3);
          if (g >= 1 && !mbar_wait(tb_free, (uint32_t)((g - 1) & 1))) { timed_out = true; break; }
          MLA_E(0, g, 4);
          if (!p.gather_tma) fence_proxy_async();
          tc_fence_after();
          issue_pv_part(s, 0);
          umma_commit(pva_done);
          MLA_E(0, g, 5);
          if (!mbar_wait(ta_free, (uint32_t)(g & 1))) { timed_out = true; break; }
          MLA_E(0, g, 7);
          tc_fence_after();
          issue_pv_part(s, 1);
          umma_commit(pvb_done);
          umma_commit(&empty[s]);
          MLA_E(0, g, 8);
        }
        base += w.nblk;
        rbase += kQEntries + w.nblk;
      }
    }
  }
  } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    if (warp == 0) MLA_M(0);
    if (warp == 0) MLA_CTA(0);
    // ------------------------------------------------------------------------------ softmax groups
    // Group A owns keys [0,32) of every block and value columns [0,128) of the unit's half; group B keys
    // [32,64) and value columns [128,256).  The two threads of a head exchange their block maxima through
    // shared memory, so both follow the same running maximum.
    const int grp = warp >> 2;
    const int quarter = warp & 3;
    const int head = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tS = lane_base + kColS + grp * 32, tT = lane_base + kColT, tPw = lane_base + kColP + grp * 16;
    uint64_t* my_done = grp == 0 ? pva_done : pvb_done;
    uint64_t* my_free = grp == 0 ? ta_free : tb_free;
    int base = 0, rbase = 0;                            // blocks / ring entries of the units before this one
    uint32_t nx = 0;                                    // exchanges through xch so far

    float o[128];
    // o = (o + scratch) * scale: adds this group's 128 value columns of P_g . V_g, then hands the scratch back
    auto accumulate = [&](int g, float scale) -> bool {
      const bool ok = mbar_wait(my_done, (uint32_t)(g & 1));
      if (!__all_sync(0xffffffffu, ok)) return false;
      if (quarter == 0) MLA_E(2 + grp, g, 5);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 8; ++c) {                       // 16 columns at a time keeps the live registers low
        uint32_t t[16];
        tmem_ld16(tT + c * 16, t);
        tmem_ld_wait();
#pragma unroll
        for (int e = 0; e < 16; ++e) o[c * 16 + e] = (o[c * 16 + e] + __uint_as_float(t[e])) * scale;
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(my_free);
      if (quarter == 0) MLA_E(2 + grp, g, 6);
      return true;
    };

    for (int u = u_first; u <= u_last && !timed_out; ++u) {
      const UnitWork w = unit_work(p, u, slot0, slot1);
      if (w.nblk > 0) {
        // This head's query row: from the ring entry that holds it (rows 0-63 in the unit's first entry, 64-127 in
        // its second) to tensor memory, two fp16 per 32-bit column: group A elements [0,288), group B [288,576).
        // Every Q.K^T of the previous unit has completed: this thread has seen its last scores.
        const int rq = rbase + (head >> 6), sq = rq % kMlaStages;
        const bool okq = mbar_wait(&full[sq], (uint32_t)((rq / kMlaStages) & 1));
        if (!__all_sync(0xffffffffu, okq)) { timed_out = true; break; }
        const uint8_t* qs = sK + sq * kKTile;
        const int qrow = head & 63;
#pragma unroll 1
        for (int c0 = 0; c0 < 9; c0 += 3) {
          uint4 v[12];
#pragma unroll
          for (int i = 0; i < 12; ++i) {
            const int ch = grp * 36 + c0 * 4 + i;       // 16-byte chunk of the 1152-byte row
            v[i] = *reinterpret_cast<const uint4*>(qs + (ch >> 3) * kBlkBytes + swz128(qrow, ch & 7));
          }
#pragma unroll
          for (int c = 0; c < 3; ++c) {
            uint32_t rr[16];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              rr[4 * i] = v[c * 4 + i].x; rr[4 * i + 1] = v[c * 4 + i].y;
              rr[4 * i + 2] = v[c * 4 + i].z; rr[4 * i + 3] = v[c * 4 + i].w;
            }
            tmem_st16(lane_base + kColQ + (grp * 9 + c0 + c) * 16, rr);
          }
        }
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(q_full);
        if (warp == 0 && u == u_first) MLA_M(1);
        if (warp == 0 && u != u_first) MLA_M(5);
      }

      float m = -INFINITY, l = 0.f;
#pragma unroll
      for (int i = 0; i < 128; ++i) o[i] = 0.f;

      for (int j = 0; j < w.nblk; ++j) {
        const int g = base + j;
        bool ok = mbar_wait(s_full, (uint32_t)(g & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (quarter == 0) MLA_E(2 + grp, g, 0);
        if (warp == 0 && g == 0) MLA_M(2);
        tc_fence_after();
        uint32_t s[32];
        tmem_ld32(tS, s);
        tmem_ld_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(s_free);                  // the scores live in registers from here on
        if (quarter == 0) MLA_E(2 + grp, g, 1);
        const int kb = w.k0 + j * kBK + grp * 32;
        const bool tail = kb + 32 > w.k1;
        float bm = -INFINITY;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          float t = __uint_as_float(s[e]) * p.sc;
          if (tail && kb + e >= w.k1) t = -INFINITY;
          s[e] = __float_as_uint(t);
          bm = fmaxf(bm, t);
        }
        smax[((g & 1) * 2 + grp) * 128 + head] = bm;
        __syncwarp();
        if (lane == 0) mbar_arrive(&xch[quarter]);
        ok = mbar_wait(&xch[quarter], nx & 1);
        ++nx;
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        if (quarter == 0) MLA_E(2 + grp, g, 2);
        bm = fmaxf(bm, smax[((g & 1) * 2 + (grp ^ 1)) * 128 + head]);
        const float m_new = fmaxf(m, bm);
        const float mu = (m_new == -INFINITY) ? 0.f : m_new;
        const float alpha = ex2(m - mu);
        m = m_new;
        float ps = 0.f;
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const float pv = ex2(__uint_as_float(s[e]) - mu);
          ps += pv;
          s[e] = __float_as_uint(pv);
        }
        l = l * alpha + ps;
        if (g >= 1) {                                        // P is free once both parts of the previous P.V are done
          ok = mbar_wait(pvb_done, (uint32_t)((g - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        }
        if (quarter == 0) MLA_E(2 + grp, g, 3);
        {
          uint32_t pk[16];
#pragma unroll
          for (int e = 0; e < 16; ++e) pk[e] = pack_half2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
          if (p.bf16) {                                  // one uniform branch per block, not a choice per element
#pragma unroll
            for (int e = 0; e < 16; ++e) pk[e] = pack_bf16x2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
          }
          tmem_st16(tPw, pk);
          tmem_st_wait();
          tc_fence_before();
          __syncwarp();
          if (lane == 0) mbar_arrive(p_full);
          if (quarter == 0) MLA_E(2 + grp, g, 4);
        }
        if (grp == 0) {
          // A: rescale now, then add part A of this block's P.V as soon as it is there (the issuer needs the
          // scratch back for part B)
#pragma unroll
          for (int i = 0; i < 128; ++i) o[i] *= alpha;
          if (!accumulate(g, 1.f)) { timed_out = true; break; }
        } else if (j >= 1) {
          // B: part B of the PREVIOUS block is added here, after this block's P is on its way, and rescaled with it
          if (!accumulate(g - 1, alpha)) { timed_out = true; break; }
        }
      }
      if (!timed_out && w.nblk > 0 && grp == 1 && !accumulate(base + w.nblk - 1, 1.f)) timed_out = true;
      if (timed_out) break;
      base += w.nblk;
      if (w.nblk > 0) rbase += kQEntries + w.nblk;
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

      // ---- emit -----------------------------------------------------------------------------------------
      if (warp == 0 && u == u_first) MLA_M(3);
      const int dv0 = grp * 128;
      if (w.whole) {
        const float inv = 1.f / l;
        __half* dst = p.out + ((size_t)w.b * kMH + head) * kDV + w.half * 256 + dv0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          uint4 v;
          v.x = pack2(o[8 * i] * inv, o[8 * i + 1] * inv, p.bf16);
          v.y = pack2(o[8 * i + 2] * inv, o[8 * i + 3] * inv, p.bf16);
          v.z = pack2(o[8 * i + 4] * inv, o[8 * i + 5] * inv, p.bf16);
          v.w = pack2(o[8 * i + 6] * inv, o[8 * i + 7] * inv, p.bf16);
          reinterpret_cast<uint4*>(dst)[i] = v;
        }
      } else {
        // partial record, stored [column group of 4][head][4] so that a warp writes 512 contiguous bytes
        const size_t part = (size_t)blockIdx.x * 2 + (u == u_first ? 0 : 1);
        float4* dst = reinterpret_cast<float4*>(p.part_o) + (part * 64 + grp * 32) * kMH + head;
#pragma unroll
        for (int i = 0; i < 32; ++i) dst[(size_t)i * kMH] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        if (grp == 0) {
          p.part_ml[(part * kMH + head) * 2] = m;
          p.part_ml[(part * kMH + head) * 2 + 1] = l;
        }
      }
      if (warp == 0 && u == u_first) MLA_M(4);
    }
    if (warp == 0) MLA_M(6);
    if (warp == 0) MLA_CTA(1);
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: every warp arrives, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == kWarpPV) {
    tc_fence_after();
    tmem_free(tmem_base, kMlaCols);
  }
}

#ifdef VMK_MLA_TIMING
extern "C" VMK_API int vmk_debug_mla_trace(long long* out) {
  cudaDeviceSynchronize();
  cudaMemcpyFromSymbol(out + 512, g_mla_marks, sizeof(long long) * 16);
  cudaMemcpyFromSymbol(out + 528, g_mla_cta_ns, sizeof(long long) * 512);
  return (int)cudaMemcpyFromSymbol(out, g_mla_trace, sizeof(long long) * 512);
}
#endif

// Merge of the units a range boundary cuts.  grid (ncta, 4): CTA (c, hq) looks at the boundary where range c
// starts; if it lies inside a unit and is the first such boundary of that unit, it merges the unit's partials
// (the last unit of range c - 1, then the first unit of ranges c, c + 1, ... while they start inside the unit)
// for heads [32 hq, 32 hq + 32).  grid (ncta, 4, 4), 256 threads: lane = head, CTA z and warp w = the two column
// groups of four [16 z + 2 w, 16 z + 2 w + 2): short serial work per thread, since with few requests only a handful
// of CTAs have anything to merge.
__global__ void __launch_bounds__(256) mla_tc_combine_kernel(const float* __restrict__ part_o,
                                                             const float* __restrict__ part_ml, int B, int ncta,
                                                             __half* __restrict__ out, int bf16) {
  const int c = blockIdx.x;
  const int total = 2 * B * kUnitSlots;
  const int s = range_start(c, total, ncta);
  asm volatile("griddepcontrol.wait;" ::: "memory");    // launched as a programmatic dependent of mla_tc_kernel
  if (c == 0 || s % kUnitSlots == 0) return;
  const int u = s / kUnitSlots;
  const int prev = range_start(c - 1, total, ncta);
  if (prev > u * kUnitSlots) return;                    // an earlier boundary inside the unit does the merge
  const int head = blockIdx.y * 32 + (threadIdx.x & 31), cg0 = blockIdx.z * 16 + (threadIdx.x >> 5) * 2;
  const int unit_end = (u + 1) * kUnitSlots;
  // range c - 1 holds this unit as its last unit (record 1) unless the unit is also its first
  const size_t part_prev = (size_t)(c - 1) * 2 + (prev / kUnitSlots == u ? 0 : 1);
  int c_end = c;
  while (c_end < ncta && range_start(c_end, total, ncta) < unit_end) ++c_end;
  // Parts of the unit: t = 0 the record range c - 1 left, t >= 1 the first-unit record of range c + t - 1.  They
  // are merged four at a time with a running maximum, so that the (m, l, o) loads of a group are all in flight
  // together: done part by part, each part costs a round trip to L2, and a unit cut in 16 has 17 of them.
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
        const float4* src = reinterpret_cast<const float4*>(part_o) + (part * 64 + cg0) * kMH + head;
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
  __half* dst = out + ((size_t)(u % B) * kMH + head) * kDV + (u / B) * 256 + cg0 * 4;
  uint4 v;
  v.x = pack2(acc[0].x * inv, acc[0].y * inv, bf16);
  v.y = pack2(acc[0].z * inv, acc[0].w * inv, bf16);
  v.z = pack2(acc[1].x * inv, acc[1].y * inv, bf16);
  v.w = pack2(acc[1].z * inv, acc[1].w * inv, bf16);
  *reinterpret_cast<uint4*>(dst) = v;
}

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Number of ranges (= CTAs).  With at least one unit per SM: one CTA per SM, ranges cut wherever they fall.
// With fewer units the ranges may be aligned to the units instead (every unit cut into the same power-of-two
// number of parts), which keeps most partial records away: parts per unit minimise
// waves x (blocks per part + a fixed cost of about four blocks for loading Q and draining), and the aligned
// cut is taken when that beats the free-running one.
int mla_tc_ctas(int B) {
  const int sms = sm_count();
  if (g_batch_invariant) return 2 * B * 4;              // every unit cut into the same four parts, whatever B is
  if (2 * B >= sms) return sms;
  long long best_cost = -1;
  int best = 1;
  for (int ns = 1; ns <= kUnitSlots / kMinSlotsPerCta; ns *= 2) {
    const long long cost = (long long)cdiv(2 * B * ns, sms) * (kUnitSlots / ns + 4);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = ns; }
  }
  // free-running ranges pay about three more blocks for the partial records of nearly every unit
  const long long free_cost = cdiv(2 * B * kUnitSlots, sms) + 4 + 3;
  return free_cost < best_cost ? sms : 2 * B * best;
}

// Bytes of the partial (m, l, o) records: two per CTA.
size_t mla_tc_workspace(int B) {
  const size_t n = (size_t)mla_tc_ctas(B) * 2 * kMH;
  return align_up(n * 256 * 4, 256) + align_up(n * 2 * 4, 256);
}

int mla_tc_launch(const MlaTcParams& p0, float* workspace, cudaStream_t stream) {
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaTcSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  MlaTcParams p = p0;
  p.ncta = mla_tc_ctas(p.B);
  const size_t n = (size_t)p.ncta * 2 * kMH;
  p.part_o = workspace;
  p.part_ml = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(workspace) + align_up(n * 256 * 4, 256));
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(p.ncta);
  cfg.blockDim = dim3(kMlaThreads);
  cfg.dynamicSmemBytes = kMlaTcSmem;
  cfg.stream = stream;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int rc = check_launch(cudaLaunchKernelEx(&cfg, mla_tc_kernel, p));
  if (rc || p.ncta == 1) return rc;
  cfg.gridDim = dim3(p.ncta, 4, 4);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = 0;
  return check_launch(cudaLaunchKernelEx(&cfg, mla_tc_combine_kernel, (const float*)p.part_o, (const float*)p.part_ml, p.B,
                                         p.ncta, p.out, p.bf16));
}

}  // namespace vmk
