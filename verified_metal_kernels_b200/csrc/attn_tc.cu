// Split-KV decode attention on the 5th-generation tensor cores, for large stacks of query rows (many
// requests sharing a prefix, or a wide speculative tree): the regime where the op is bound by the
// tensor pipe rather than by HBM.
//
// One tcgen05.mma costs about 96 cycles whatever its width up to N = 128 (107 with A in shared memory), so
// the kernel works on 128-key blocks: S = Q.K^T is 8 instructions of M128 N128 K16 per block and tile, and
// P.V is 8 of M128 N128 K16 with P read from TENSOR MEMORY.
//
// One CTA = one (key group, 256-row tile, key split) and handles its rows as TWO 128-row tiles A and B
// that share every K/V tile brought into shared memory and alternate on the tensor pipe: while the softmax
// warps of one tile work, the products of the other run.  Tensor memory (512 columns): S_A, S_B, O_A, O_B,
// 128 columns each.  P (fp16 pairs, 64 columns) is written IN PLACE over the scores it came from, so S_t
// is rewritten by the next Q.K^T only after P_t.V has completed.  352 threads, warp-specialised:
//   warp 0      TMA producer: K_0, V_0, K_1, V_1, ... (128 keys x 128, four 64x64 swizzled boxes each) into
//               one ring of five 32 KiB slots; the products release the slots in the same order
//   warp 1      owns tensor memory and issues  S_t = Q_t . K_j^T        (A, B from shared memory, K-major)
//   warp 10     issues                          O_t += P_t . V_j          (A = P_t in tensor memory, V MN-major)
//               two issuing warps, because the tensor pipe buffers only an instruction or two and an
//               issuing thread that waits lets it drain
//   warps 2-5   softmax of tile A, warps 6-9 softmax of tile B, one thread per row: two passes over the
//               128 scores in tensor memory (row max; then exp2 / row sum / fp16 P back to tensor memory),
//               LAZY rescaling of O (only when the row max grew by more than 2^8, so P stays below 256
//               and the result exact)
// Partials (m, l, o) per row are emitted exactly as by the warp-level kernel, so the combine pass and
// the multi-GPU merge are shared.  Every mbarrier wait is bounded; a wait that runs out sets the status
// word and the CTA winds down through the common exit, where tensor memory is freed.
#include <type_traits>

#include "attn_core.cuh"
#include "tcgen05.cuh"

namespace vmk {

constexpr int kTcBK = 128;                       // keys per block
constexpr int kTcRows = 256;                     // rows per CTA (two tiles of 128)
constexpr int kQHalf = 128 * 128;                // [128 rows][128 B] swizzled: one 64-wide half of the head dim
constexpr int kQTile = 2 * kQHalf;               // 32 KiB per 128-row query tile
constexpr int kKvHalf = kTcBK * 128;             // [128 keys][128 B] swizzled (two 64-key TMA boxes)
constexpr int kKvTile = 2 * kKvHalf;             // 32 KiB
constexpr int kTcSlots = 5;                      // ring slots: K_j -> slot 2j % 5, V_j -> slot (2j + 1) % 5
constexpr int kTcThreads = 352;
constexpr int kTcCols = 512;
constexpr int kColS = 0;                         // S_A, S_B: 2 x 128 columns (P_t over the first 64 of S_t)
constexpr int kColO = 256;                       // O_A, O_B: 2 x 128 columns
constexpr float kLazyRescale = 8.f;              // log2 units
constexpr int kTcBars = 2 * kTcSlots + 2 + 2 + 2 + 2;
constexpr int kAttnTcSmem = 2 * kQTile + kTcSlots * kKvTile + kTcBars * 8 + 16 + 1024;

#ifdef VMK_TC_TIMING
// Debug build only.  Time stamps of blocks 8..15 of CTA 0: [role][block - 8][event]
__device__ long long g_tc_trace[5 * 8 * 8];
#define TC_E(role, j, ev) do { if (blockIdx.x == 0 && (j) >= 8 && (j) < 16 && lane == 0) \
    g_tc_trace[((role) * 8 + (j) - 8) * 8 + (ev)] = clock64(); } while (0)
#else
#define TC_E(role, j, ev) do {} while (0)
#endif

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kTcThreads, 1) attn_tc_kernel(const __grid_constant__ AttnParams p) {
  const AttnRole& R = p.a;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;                                   // [2 tiles][32 KiB]
  uint8_t* sKV = sQ + 2 * kQTile;                       // [slots][32 KiB]
  uint64_t* full = reinterpret_cast<uint64_t*>(sKV + kTcSlots * kKvTile);   // tile landed (TMA bytes)
  uint64_t* empty = full + kTcSlots;                    // tile consumed by both row tiles' product (MMA commit)
  uint64_t* s_full = empty + kTcSlots;                  // [tile] scores ready               (MMA commit)
  uint64_t* p_full = s_full + 2;                        // [tile] P stored to tensor memory  (4 warps)
  uint64_t* pv_done = p_full + 2;                       // [tile] P.V done: S_t and O_t free (MMA commit)
  uint64_t* q_full = pv_done + 2;                       // [tile] Q tile in shared memory    (4 warps)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which piece of work (same decomposition as the warp-level kernel) ---------------------------
  const int cta = blockIdx.x;
  const int split = cta % R.nsplit;
  const int t2 = cta / R.nsplit;
  const int tile = t2 % R.row_tiles;
  const int z = t2 / R.row_tiles;
  const int zg = z / R.Hkv, h = z % R.Hkv;
  const int rows = R.rows_outer * R.G;
  const int row0 = tile * kTcRows;
  const bool has_b = row0 + 128 < rows;                 // tile B holds at least one real row
  const int kbeg = R.key_lo + split * R.split_len;

  if (tid == 0) {
    for (int s = 0; s < kTcSlots; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&s_full[t], 1);
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
      mbar_init(&q_full[t], 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTcCols);
  if (warp == 0 && lane == 0) {
    // hints that start the HBM reads of the first tiles early (no shared memory, no barrier); like the barrier
    // and tensor-memory set-up above they touch nothing a kernel before this one could have written
    tma_prefetch_desc(&R.tmK);
    tma_prefetch_desc(&R.tmV);
    if (R.page_table == nullptr) {
      const int ke0 = min(kbeg + R.split_len, R.key_hi);
      for (int j = 0; j < 2 && kbeg + j * kTcBK < ke0; ++j) {
        for (int y = 0; y < kTcBK; y += 64) {
          tma_prefetch_3d(&R.tmK, 0, kbeg + j * kTcBK + y, z);
          tma_prefetch_3d(&R.tmK, 64, kbeg + j * kTcBK + y, z);
          tma_prefetch_3d(&R.tmV, 0, kbeg + j * kTcBK + y, z);
          tma_prefetch_3d(&R.tmV, 64, kbeg + j * kTcBK + y, z);
        }
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // launched as a programmatic dependent: in a chain of calls everything above overlaps the tail of the call
  // before; the inputs are read only below this line
  pdl_wait();
  int kend = min(kbeg + R.split_len, R.key_hi);
  if (R.klens != nullptr) kend = min(kend, max(0, min(R.klens[zg], R.klen)));
  const int nblk = kend > kbeg ? (kend - kbeg + kTcBK - 1) / kTcBK : 0;

  bool timed_out = false;
  if (warp == 0) {
    // ------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int issued = 0;                                     // tiles requested so far
      for (int i = 0; i < 2 * nblk; ++i) {
        const int s = i % kTcSlots;
        if (i >= kTcSlots && !mbar_wait(&empty[s], (uint32_t)(((i / kTcSlots) - 1) & 1))) {
          timed_out = true;
          break;
        }
        issued = i + 1;
        const CUtensorMap* tm = (i & 1) ? &R.tmV : &R.tmK;
        const int kb = kbeg + (i >> 1) * kTcBK;
        uint8_t* dst = sKV + s * kKvTile;
        TC_E(4, i >> 1, (i & 1) * 2);
        mbar_expect_tx(&full[s], kKvTile);
        // the tensor maps have 64 x 64 boxes: two boxes stacked along the keys make one [128][128 B] half.
        // Paged cache: each 64-key box lies inside one page; a page id outside the pool reads zeros.
        int y0 = kb, y1 = kb + 64, z0 = z, z1 = z;
        if (R.page_table != nullptr) {
          const int p0 = y0 / R.page_size, p1 = y1 / R.page_size;
          const int g0 = p0 < R.table_stride ? R.page_table[(size_t)zg * R.table_stride + p0] : -1;
          const int g1 = p1 < R.table_stride ? R.page_table[(size_t)zg * R.table_stride + p1] : -1;
          z0 = (g0 >= 0 && g0 * R.Hkv + h < R.page_groups) ? g0 * R.Hkv + h : R.page_groups;
          z1 = (g1 >= 0 && g1 * R.Hkv + h < R.page_groups) ? g1 * R.Hkv + h : R.page_groups;
          y0 -= p0 * R.page_size;
          y1 -= p1 * R.page_size;
        }
        tma_load_3d(dst, tm, 0, y0, z0, &full[s]);
        tma_load_3d(dst + kKvHalf / 2, tm, 0, y1, z1, &full[s]);
        tma_load_3d(dst + kKvHalf, tm, 64, y0, z0, &full[s]);
        tma_load_3d(dst + kKvHalf + kKvHalf / 2, tm, 64, y1, z1, &full[s]);
      }
      // No load outlives the CTA: the newest tile of every slot has landed before this warp goes to the exit.  In a
      // run without a timeout the consumers have waited for all of them already and these return at once; when a
      // consumer gave up, this keeps the SM from handing the shared memory to another CTA under a late load.
      for (int i = max(0, issued - kTcSlots); i < issued; ++i)
        mbar_wait(&full[i % kTcSlots], (uint32_t)((i / kTcSlots) & 1));
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------ Q.K^T issuer
    if (lane == 0 && nblk > 0) {
      const uint32_t idesc_qk = umma_idesc_16(128, kTcBK, 0, p.bf16);
      const int ntile = has_b ? 2 : 1;
      // Descriptor words.  High words are constants of the layout; low words are (address >> 4) plus a
      // constant per K step: +2 per 32-byte step inside a 128-byte swizzled row, + half-tile / 16 for the
      // second 64-wide half.
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      const uint32_t lo_k0 = (uint32_t)umma_desc_sw128(0);
      const uint32_t q_lo = lo_k0 + (smem_u32(sQ) >> 4), kv_lo = lo_k0 + (smem_u32(sKV) >> 4);
      for (int t = 0; t < ntile; ++t)
        if (!mbar_wait(&q_full[t], 0)) timed_out = true;
      for (int j = 0; j < nblk && !timed_out; ++j) {
        const int i = 2 * j, s = i % kTcSlots;
        if (!mbar_wait(&full[s], (uint32_t)((i / kTcSlots) & 1))) { timed_out = true; break; }
        const uint32_t kb_lo = kv_lo + s * (kKvTile >> 4);
        TC_E(0, j, 0);
        for (int t = 0; t < ntile; ++t) {
          // S_t (and the P_t inside it) is free once P_t . V_{j-1} has completed
          if (j >= 1 && !mbar_wait(&pv_done[t], (uint32_t)((j - 1) & 1))) { timed_out = true; break; }
          TC_E(0, j, 1 + 2 * t);
          tc_fence_after();
          const uint32_t d = tmem_base + kColS + t * 128;
          const uint32_t qa_lo = q_lo + t * (kQTile >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            umma_f16_w(d, qa_lo + (k >> 2) * (kQHalf >> 4) + (k & 3) * 2, hi_k,
                       kb_lo + (k >> 2) * (kKvHalf >> 4) + (k & 3) * 2, hi_k, idesc_qk, k > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t]);
          TC_E(0, j, 2 + 2 * t);
        }
        if (timed_out) break;
        umma_commit(&empty[s]);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------------------ P.V issuer
    if (lane == 0 && nblk > 0) {
      const uint32_t idesc_pv = umma_idesc_16(128, 128, 1, p.bf16);
      const int ntile = has_b ? 2 : 1;
      // V rows 16k .. 16k+16 (keys) x 128 d, MN-major: 8-key groups 1024 B apart (+128 per 16-key step), the
      // two 64-wide d halves kKvHalf apart.  P_t[:, 16k .. 16k+16) = 8 columns of packed fp16 pairs.
      const uint32_t hi_v = (uint32_t)(umma_desc_sw128_mn(0, kKvHalf, 1024) >> 32);
      const uint32_t v_lo = (uint32_t)umma_desc_sw128_mn(0, kKvHalf, 1024) + (smem_u32(sKV) >> 4);
      for (int j = 0; j < nblk && !timed_out; ++j) {
        const int i = 2 * j + 1, s = i % kTcSlots;
        if (!mbar_wait(&full[s], (uint32_t)((i / kTcSlots) & 1))) { timed_out = true; break; }
        const uint32_t vb_lo = v_lo + s * (kKvTile >> 4);
        TC_E(1, j, 0);
        for (int t = 0; t < ntile; ++t) {
          if (!mbar_wait(&p_full[t], (uint32_t)(j & 1))) { timed_out = true; break; }
          TC_E(1, j, 1 + 2 * t);
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k)
            umma_f16_ts(tmem_base + kColO + t * 128, tmem_base + kColS + t * 128 + k * 8, vb_lo + k * (2048 >> 4), hi_v,
                          idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          umma_commit(&pv_done[t]);
          TC_E(1, j, 2 + 2 * t);
        }
        if (timed_out) break;
        umma_commit(&empty[s]);
      }
    }
  } else if (warp >= 2 && warp <= 9) {
    // ------------------------------------------------------------------------------ softmax warps
    const int t = (warp - 2) >> 2;                        // 0: tile A, 1: tile B
    const int quarter = warp & 3;                         // tensor-memory lanes [32 q, 32 q + 32)
    const int row = quarter * 32 + lane;
    const int grow = row0 + t * 128 + row;
    const bool valid_row = grow < rows;
    const bool tile_on = t == 0 || has_b;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tS = lane_base + kColS + t * 128;
    const uint32_t tO = lane_base + kColO + t * 128;
    const size_t outer = (size_t)zg * R.rows_outer + (valid_row ? grow / R.G : 0);
    const int head = h * R.G + (valid_row ? grow % R.G : 0);

    if (tile_on) {
      // this thread's query row -> swizzled K-major operand tile
      const uint4* src = reinterpret_cast<const uint4*>(R.q + (outer * R.Hq + head) * kHD);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 v = valid_row ? src[c] : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(sQ + t * kQTile + (c >> 3) * kQHalf + swz128(row, c & 7)) = v;
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&q_full[t]);
    }
    uint32_t mw[kMaxMaskWords];
#pragma unroll
    for (int w = 0; w < kMaxMaskWords; ++w) {
      mw[w] = 0xffffffffu;
      if (R.bits != nullptr && valid_row && w < R.bits_words) mw[w] = R.bits[outer * R.bits_words + w];
    }
    // scaled score of key (kb + c * 32 + i), or -inf if the key is past the end or hidden from this draft row
    auto visible = [&](int key, int kend_) -> bool {
      bool vis = key < kend_;
      if (vis && key >= R.mask_start) {
        const int jb = key - R.mask_start;
        uint32_t word = mw[0];
#pragma unroll
        for (int w = 1; w < kMaxMaskWords; ++w) word = ((jb >> 5) == w) ? mw[w] : word;
        vis = (word >> (jb & 31)) & 1u;
      }
      return vis;
    };

    float m = -INFINITY, l = 0.f;
    const int nloop = tile_on ? nblk : 0;
    for (int j = 0; j < nloop; ++j) {
      bool ok = mbar_wait(&s_full[t], (uint32_t)(j & 1));
      if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      if (quarter == 2) TC_E(2 + t, j, 0);
      tc_fence_after();
      const int kb = kbeg + j * kTcBK;
      const bool tail = kb + kTcBK > kend;
      const bool edge = tail || (kb + kTcBK > R.mask_start);
      // the 128 scores of this row -> registers (one wait for the four loads)
      uint32_t s0[32], s1[32], s2[32], s3[32];
      tmem_ld32(tS, s0);
      tmem_ld32(tS + 32, s1);
      tmem_ld32(tS + 64, s2);
      tmem_ld32(tS + 96, s3);
      tmem_ld_wait();
      if (quarter == 2) TC_E(2 + t, j, 1);
      float bm = -INFINITY;
      if (!edge) {
        // interior block: every key visible.  Kept free of per-element branches.
        float b0 = -INFINITY, b1 = -INFINITY, b2 = -INFINITY, b3 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          b0 = fmaxf(b0, __uint_as_float(s0[i]));
          b1 = fmaxf(b1, __uint_as_float(s1[i]));
          b2 = fmaxf(b2, __uint_as_float(s2[i]));
          b3 = fmaxf(b3, __uint_as_float(s3[i]));
        }
        bm = fmaxf(fmaxf(b0, b1), fmaxf(b2, b3));
      } else {
        // block touching the end of the key range or the draft positions: hidden keys become -inf
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          if (!visible(kb + i, kend)) s0[i] = 0xff800000u;
          if (!visible(kb + 32 + i, kend)) s1[i] = 0xff800000u;
          if (!visible(kb + 64 + i, kend)) s2[i] = 0xff800000u;
          if (!visible(kb + 96 + i, kend)) s3[i] = 0xff800000u;
          bm = fmaxf(bm, fmaxf(fmaxf(__uint_as_float(s0[i]), __uint_as_float(s1[i])),
                               fmaxf(__uint_as_float(s2[i]), __uint_as_float(s3[i]))));
        }
      }
      bm *= p.sc;                                      // the scale is positive: max commutes with it
      const float m_new = fmaxf(m, bm);
      float alpha = 1.f;
      bool rescale = false;
      if (m == -INFINITY) {
        m = m_new;                                   // nothing accumulated for this row yet
      } else if (m_new > m + kLazyRescale) {
        alpha = fast_exp2(m - m_new);
        m = m_new;
        rescale = true;
      }
      l *= alpha;
      const float mu = (m == -INFINITY) ? 0.f : m;
      if (quarter == 2) TC_E(2 + t, j, 2);
      // O_t is at rest here: Q.K^T of this block was only issued after P.V of the previous one had completed
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < 8; ++c) {
          uint32_t o[16];
          tmem_ld16(tO + c * 16, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 16; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st16(tO + c * 16, o);
        }
      }
      // P = exp2(score * scale - m) (exactly 0 for a hidden key: fma(-inf) = -inf), row sum, fp16 pairs written
      // over the first 64 columns of the scores
      if (quarter == 2) TC_E(2 + t, j, 3);
      float ps0 = 0.f, ps1 = 0.f;
      // (the 16-bit type is a compile-time tag here: a per-element choice would put both conversions on the
      // XU pipe, which is the one this loop is bound by)
      auto to_p = [&](auto bf_tag, uint32_t (&sc32)[32], int c) {
        constexpr bool BF = decltype(bf_tag)::value;
        uint32_t pk[16];
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float a = fast_exp2(fmaf(__uint_as_float(sc32[i]), p.sc, -mu));
          const float b = fast_exp2(fmaf(__uint_as_float(sc32[i + 1]), p.sc, -mu));
          ps0 += a;
          ps1 += b;
          pk[i >> 1] = BF ? pack_bf16x2(a, b) : pack_half2(a, b);
        }
        tmem_st16(tS + c * 16, pk);
      };
      if (p.bf16) {
        to_p(std::true_type{}, s0, 0);
        to_p(std::true_type{}, s1, 1);
        to_p(std::true_type{}, s2, 2);
        to_p(std::true_type{}, s3, 3);
      } else {
        to_p(std::false_type{}, s0, 0);
        to_p(std::false_type{}, s1, 1);
        to_p(std::false_type{}, s2, 2);
        to_p(std::false_type{}, s3, 3);
      }
      l += ps0 + ps1;
      if (quarter == 2) TC_E(2 + t, j, 4);
      if (tail && (kend < R.klen || R.page_table != nullptr) && t == 0) {
        // keys past kend exist in memory: their V rows must not reach the MMA (0 * Inf would poison the
        // row).  Tile A's warps clear them; tile B's P.V is issued after tile A's p_full.
        const int i = 2 * j + 1, s = i % kTcSlots;
        ok = mbar_wait(&full[s], (uint32_t)((i / kTcSlots) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        uint8_t* v = sKV + s * kKvTile;
        const int r0 = kend - kb;
        for (int e = row; e < (kTcBK - r0) * 16; e += 128) {
          const int r = r0 + (e >> 4), c = e & 15;
          *reinterpret_cast<uint4*>(v + (c >> 3) * kKvHalf + swz128(r, c & 7)) = make_uint4(0u, 0u, 0u, 0u);
        }
        fence_proxy_async();
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      if (quarter == 2) TC_E(2 + t, j, 5);
    }

    // ---- emit this row's partial (or final) result ------------------------------------------------
    bool have_o = false;
    if (!timed_out && nloop > 0) {
      const bool ok = mbar_wait(&pv_done[t], (uint32_t)((nloop - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) timed_out = true; else have_o = true;
      tc_fence_after();
    }
    if (!timed_out && tile_on) {
      const size_t slot = (size_t)z * R.nsplit + split;
      const float inv = 1.f / l;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (have_o) {
          tmem_ld32(tO + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (!valid_row) continue;
        if (R.direct) {
          __half* dst = R.out + (outer * R.Hq + head) * kHD + c * 32;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv, p.bf16);
            v.y = pack2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv, p.bf16);
            v.z = pack2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv, p.bf16);
            v.w = pack2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv, p.bf16);
            reinterpret_cast<uint4*>(dst)[i] = v;
          }
        } else {
          float* dst = R.part_o + (slot * R.MP + grow) * kHD + c * 32;
#pragma unroll
          for (int i = 0; i < 8; ++i)
            reinterpret_cast<uint4*>(dst)[i] = make_uint4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        }
      }
      if (valid_row && !R.direct) {
        R.part_ml[(slot * R.MP + grow) * 2] = m;
        R.part_ml[(slot * R.MP + grow) * 2 + 1] = l;
      }
    }
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: every warp arrives, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_free(tmem_base, kTcCols);
  }
}

#ifdef VMK_TC_TIMING
extern "C" VMK_API int vmk_debug_tc_trace(long long* out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_tc_trace, sizeof(g_tc_trace));
}
#endif

int launch_attn_tc(const AttnParams& p, int n_cta, cudaStream_t stream) {
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kAttnTcSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(n_cta);
  cfg.blockDim = dim3(kTcThreads);
  cfg.dynamicSmemBytes = kAttnTcSmem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_launch(cudaLaunchKernelEx(&cfg, attn_tc_kernel, p));
}

}  // namespace vmk
