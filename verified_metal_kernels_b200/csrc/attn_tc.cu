// Split-KV decode attention on the 5th-generation tensor cores, for large stacks of query rows (many
// requests sharing a prefix, or a wide speculative tree): the regime where the op is bound by the
// tensor pipe rather than by HBM.
//
// One CTA = one (key group, 256-row tile, key split) and handles its rows as TWO 128-row tiles A and B
// that share every K/V tile brought into shared memory (half the L2 traffic per flop, and two softmax
// warpgroups to keep the tensor pipe fed).  384 threads, warp-specialised:
//   warp 0      TMA producer of K tiles (64 keys x 128, two 64-wide swizzled boxes), 3-stage ring released
//               as soon as both Q.K^T products have consumed a tile, so K runs ahead of the softmax
//   warp 10     TMA producer of V tiles, ring of its own, released after both P.V products
//   warp 1      owns tensor memory (512 columns: S_A[2], S_B[2], O_A, O_B) and issues
//                 S_t[j & 1] (128 x 64 fp32)  = Q_t . K_j^T      8 x tcgen05.mma M128 N64 K16, K-major operands
//               S is double buffered so the Q.K^T of block j+1 runs under the softmax of block j
//   warp 11     issues
//                 O_t        (128 x 128 fp32) += P_t . V_j        4 x tcgen05.mma M128 N128 K16, V MN-major
//   warps 2-5   softmax of tile A, warps 6-9 softmax of tile B, one thread per row: two passes over the
//               64 scores in tensor memory (row max, then exp2 / row sum / fp16 P into a swizzled
//               shared-memory operand tile), LAZY rescaling of O (only when the row max grew by more than
//               2^8, so P stays below 256 and the result exact)
// Partials (m, l, o) per row are emitted exactly as by the warp-level kernel, so the combine pass and
// the multi-GPU merge are shared.  Every mbarrier wait is bounded; a wait that runs out sets the status
// word and the CTA winds down through the common exit, where tensor memory is freed.
#include "attn_core.cuh"
#include "tcgen05.cuh"

namespace vmk {

constexpr int kTcBK = 64;                        // keys per block
constexpr int kTcRows = 256;                     // rows per CTA (two tiles of 128)
constexpr int kQHalf = 128 * 128;                // [128 rows][128 B] swizzled box
constexpr int kQTile = 2 * kQHalf;               // 32 KiB per 128-row query tile
constexpr int kKvHalf = kTcBK * 128;             // [64 keys][128 B] swizzled box
constexpr int kKvTile = 2 * kKvHalf;             // 16 KiB
constexpr int kPTile = 128 * kTcBK * 2;          // 16 KiB: [128 rows][64 keys] fp16, one swizzled box
constexpr int kTcStages = 3;
constexpr int kTcThreads = 384;
constexpr int kTcCols = 512;
constexpr int kColS = 0;                         // S_A[0], S_A[1], S_B[0], S_B[1]: 4 x 64 columns
constexpr int kColO = 256;                       // O_A, O_B: 2 x 128 columns
constexpr float kLazyRescale = 8.f;              // log2 units
constexpr int kTcBars = 4 * kTcStages + 4 + 4 + 2 + 2 + 2;
constexpr int kAttnTcSmem = 2 * kQTile + 2 * kTcStages * kKvTile + 2 * kPTile + kTcBars * 8 + 16 + 1024;

#ifdef VMK_TC_TIMING
// Debug build only: cycles spent per phase by CTA 0 (softmax warp 2 lane 0: slots 0-7, MMA thread: 8-15).
__device__ long long g_tc_timing[16];
#define TC_T0() long long _t0 = clock64()
#define TC_ACC(slot) do { if (blockIdx.x == 0) { long long _t1 = clock64(); g_tc_timing[slot] += _t1 - _t0; _t0 = _t1; } } while (0)
#else
#define TC_T0() do {} while (0)
#define TC_ACC(slot) do {} while (0)
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
  uint8_t* sK = sQ + 2 * kQTile;                        // [stages][16 KiB]
  uint8_t* sV = sK + kTcStages * kKvTile;               // [stages][16 KiB]
  uint8_t* sP = sV + kTcStages * kKvTile;               // [2 tiles][16 KiB]
  uint64_t* k_full = reinterpret_cast<uint64_t*>(sP + 2 * kPTile);
  uint64_t* k_empty = k_full + kTcStages;
  uint64_t* v_full = k_empty + kTcStages;
  uint64_t* v_empty = v_full + kTcStages;
  uint64_t* s_full = v_empty + kTcStages;               // [tile][buffer]
  uint64_t* s_empty = s_full + 4;                       // [tile][buffer]
  uint64_t* p_full = s_empty + 4;                       // [tile]
  uint64_t* pv_done = p_full + 2;                       // [tile]
  uint64_t* q_full = pv_done + 2;                       // [tile]
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
  int kend = min(kbeg + R.split_len, R.key_hi);
  if (R.klens != nullptr) kend = min(kend, max(0, min(R.klens[zg], R.klen)));
  const int nblk = kend > kbeg ? (kend - kbeg + kTcBK - 1) / kTcBK : 0;

  if (tid == 0) {
    for (int s = 0; s < kTcStages; ++s) {
      mbar_init(&k_full[s], 1);
      mbar_init(&k_empty[s], 1);
      mbar_init(&v_full[s], 1);
      mbar_init(&v_empty[s], 1);
    }
    for (int s = 0; s < 4; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    for (int t = 0; t < 2; ++t) {
      mbar_init(&p_full[t], 4);
      mbar_init(&pv_done[t], 1);
      mbar_init(&q_full[t], 4);
    }
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTcCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool timed_out = false;
  if (warp == 0 || warp == 10) {
    // ------------------------------------------------------------------------------ TMA producers
    if (lane == 0) {
      const bool is_k = warp == 0;
      uint64_t* full = is_k ? k_full : v_full;
      uint64_t* empty = is_k ? k_empty : v_empty;
      uint8_t* ring = is_k ? sK : sV;
      const CUtensorMap* tm = is_k ? &R.tmK : &R.tmV;
      for (int j = 0; j < nblk; ++j) {
        const int s = j % kTcStages;
        if (j >= kTcStages && !mbar_wait(&empty[s], (uint32_t)(((j / kTcStages) - 1) & 1))) {
          timed_out = true;
          break;
        }
        const int kb = kbeg + j * kTcBK;
        uint8_t* dst = ring + s * kKvTile;
        mbar_expect_tx(&full[s], kKvTile);
        tma_load_3d(dst, tm, 0, kb, z, &full[s]);
        tma_load_3d(dst + kKvHalf, tm, 64, kb, z, &full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------ Q.K^T issuer
    // The tensor pipe buffers only an instruction or two, so an issuing thread that waits lets it drain: the
    // two products are issued by two warps, and one's instructions run while the other waits.
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, kTcBK, 0);
      const int ntile = has_b ? 2 : 1;
      // Descriptor words.  High words are constants of the layout; low words are (address >> 4) plus a
      // constant per K step: +2 per 32-byte step inside a 128-byte swizzled row, + half-tile / 16 for the
      // second 64-wide half.
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      const uint32_t lo_k0 = (uint32_t)umma_desc_sw128(0);
      const uint32_t q_lo = lo_k0 + (smem_u32(sQ) >> 4), k_lo = lo_k0 + (smem_u32(sK) >> 4);
      for (int t = 0; t < ntile; ++t)
        if (!mbar_wait(&q_full[t], 0)) timed_out = true;
      for (int j = 0; j < nblk && !timed_out; ++j) {
        if (!mbar_wait(&k_full[j % kTcStages], (uint32_t)((j / kTcStages) & 1))) { timed_out = true; break; }
        const uint32_t kb_lo = k_lo + (j % kTcStages) * (kKvTile >> 4);
        // S_t[j & 1] = Q_t . K_j^T for both tiles; releases the K stage
        for (int t = 0; t < ntile; ++t) {
          if (j >= 2 && !mbar_wait(&s_empty[t * 2 + (j & 1)], (uint32_t)(((j >> 1) - 1) & 1))) { timed_out = true; break; }
          tc_fence_after();
          const uint32_t d = tmem_base + kColS + (t * 2 + (j & 1)) * kTcBK;
          const uint32_t qa_lo = q_lo + t * (kQTile >> 4);
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            umma_f16_w(d, qa_lo + (k >> 2) * (kQHalf >> 4) + (k & 3) * 2, hi_k,
                       kb_lo + (k >> 2) * (kKvHalf >> 4) + (k & 3) * 2, hi_k, idesc_qk, k > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[t * 2 + (j & 1)]);
        }
        if (timed_out) break;
        umma_commit(&k_empty[j % kTcStages]);
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------------------ P.V issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, 128, 1);
      const int ntile = has_b ? 2 : 1;
      // +128 per 16-key step of an MN-major V tile
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      const uint32_t hi_v = (uint32_t)(umma_desc_sw128_mn(0, kKvHalf, 1024) >> 32);
      const uint32_t p_lo = (uint32_t)umma_desc_sw128(0) + (smem_u32(sP) >> 4);
      const uint32_t v_lo = (uint32_t)umma_desc_sw128_mn(0, kKvHalf, 1024) + (smem_u32(sV) >> 4);
      for (int j = 0; j < nblk && !timed_out; ++j) {
        if (!mbar_wait(&v_full[j % kTcStages], (uint32_t)((j / kTcStages) & 1))) { timed_out = true; break; }
        const uint32_t vb_lo = v_lo + (j % kTcStages) * (kKvTile >> 4);
        for (int t = 0; t < ntile; ++t) {
          if (!mbar_wait(&p_full[t], (uint32_t)(j & 1))) { timed_out = true; break; }
          tc_fence_after();
#pragma unroll
          for (int k = 0; k < kTcBK / 16; ++k) {
            // A: P_t[:, 16k .. 16k+16) K-major (one 128-byte swizzled row per query row);
            // B: V rows 16k .. 16k+16 (keys) x 128 d, MN-major: 8-key groups 1024 B apart, the two 64-wide
            //    d halves kKvHalf apart.
            umma_f16_w(tmem_base + kColO + t * 128, p_lo + t * (kPTile >> 4) + k * 2, hi_k, vb_lo + k * (2048 >> 4), hi_v,
                       idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
          }
          umma_commit(&pv_done[t]);
        }
        if (timed_out) break;
        umma_commit(&v_empty[j % kTcStages]);
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
    const uint32_t tS = lane_base + kColS + t * 2 * kTcBK;
    const uint32_t tO = lane_base + kColO + t * 128;
    const size_t outer = (size_t)zg * R.rows_outer + (valid_row ? grow / R.G : 0);
    const int head = h * R.G + (valid_row ? grow % R.G : 0);
    uint8_t* myP = sP + t * kPTile;

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

    float m = -INFINITY, l = 0.f;
    const int nloop = tile_on ? nblk : 0;
#ifdef VMK_TC_TIMING
    const bool tc_probe = warp == 2 && lane == 0;
    long long _t0 = clock64();
#define SM_ACC(slot) do { if (tc_probe && blockIdx.x == 0) { long long _t1 = clock64(); g_tc_timing[slot] += _t1 - _t0; _t0 = _t1; } } while (0)
#else
#define SM_ACC(slot) do {} while (0)
#endif
    for (int j = 0; j < nloop; ++j) {
      const int sb = j & 1;
      bool ok = mbar_wait(&s_full[t * 2 + sb], (uint32_t)((j >> 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      SM_ACC(0);
      tc_fence_after();
      const int kb = kbeg + j * kTcBK;
      const bool tail = kb + kTcBK > kend;
      const bool edge = tail || (kb + kTcBK > R.mask_start);
      // pass 1: row maximum of the 64 scores
      uint32_t s0[32], s1[32];
      tmem_ld32(tS + sb * kTcBK, s0);
      tmem_ld32(tS + sb * kTcBK + 32, s1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[t * 2 + sb]);    // the scores now live in registers
      SM_ACC(1);
      float bm = -INFINITY;
      if (!edge) {
        // interior block: every key visible.  Kept free of per-element branches so the hot loop is a
        // short straight-line sequence.
        float bm1 = -INFINITY;
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float a = __uint_as_float(s0[i]) * p.sc, b = __uint_as_float(s1[i]) * p.sc;
          s0[i] = __float_as_uint(a);
          s1[i] = __float_as_uint(b);
          bm = fmaxf(bm, a);
          bm1 = fmaxf(bm1, b);
        }
        bm = fmaxf(bm, bm1);
      } else {
        // block touching the end of the key range or the draft positions: per-key visibility
#pragma unroll 1
        for (int half = 0; half < 2; ++half) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kb + half * 32 + i;
            bool vis = key < kend;
            if (vis && key >= R.mask_start) {
              const int jb = key - R.mask_start;
              uint32_t word = mw[0];
#pragma unroll
              for (int w = 1; w < kMaxMaskWords; ++w) word = ((jb >> 5) == w) ? mw[w] : word;
              vis = (word >> (jb & 31)) & 1u;
            }
            if (half == 0) {
              const float a = vis ? __uint_as_float(s0[i]) * p.sc : -INFINITY;
              s0[i] = __float_as_uint(a);
              bm = fmaxf(bm, a);
            } else {
              const float a = vis ? __uint_as_float(s1[i]) * p.sc : -INFINITY;
              s1[i] = __float_as_uint(a);
              bm = fmaxf(bm, a);
            }
          }
        }
      }
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
      float ps0 = 0.f, ps1 = 0.f;
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const float a = fast_exp2(__uint_as_float(s0[i]) - mu), b = fast_exp2(__uint_as_float(s1[i]) - mu);
        ps0 += a;
        ps1 += b;
        s0[i] = __float_as_uint(a);
        s1[i] = __float_as_uint(b);
      }
      l += ps0 + ps1;
      SM_ACC(2);

      // O_t and the P tile are free once P_{j-1} . V_{j-1} has completed
      if (j >= 1) {
        ok = mbar_wait(&pv_done[t], (uint32_t)((j - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        tc_fence_after();
      }
      SM_ACC(3);
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(tO + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(tO + c * 32, o);
        }
        tmem_st_wait();
      }
      if (tail && kend < R.klen && t == 0) {
        // keys past kend exist in memory: their V rows must not reach the MMA (0 * Inf would poison the
        // row).  Tile A's warps clear them; tile B's P.V is issued after tile A's p_full.
        ok = mbar_wait(&v_full[j % kTcStages], (uint32_t)((j / kTcStages) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        uint8_t* v = sV + (j % kTcStages) * kKvTile;
        const int r0 = kend - kb;
        for (int i = row; i < (kTcBK - r0) * 16; i += 128) {
          const int r = r0 + (i >> 4), c = i & 15;
          *reinterpret_cast<uint4*>(v + (c >> 3) * kKvHalf + swz128(r, c & 7)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      SM_ACC(4);
      // P (fp16) -> swizzled K-major operand tile: 64 keys = 8 chunks of 16 bytes per row
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const uint32_t* s8 = (c < 4) ? &s0[c * 8] : &s1[(c - 4) * 8];
        uint4 v;
        v.x = pack_half2(__uint_as_float(s8[0]), __uint_as_float(s8[1]));
        v.y = pack_half2(__uint_as_float(s8[2]), __uint_as_float(s8[3]));
        v.z = pack_half2(__uint_as_float(s8[4]), __uint_as_float(s8[5]));
        v.w = pack_half2(__uint_as_float(s8[6]), __uint_as_float(s8[7]));
        *reinterpret_cast<uint4*>(myP + swz128(row, c)) = v;
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&p_full[t]);
      SM_ACC(5);
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
            v.x = pack_half2(__uint_as_float(o[8 * i]) * inv, __uint_as_float(o[8 * i + 1]) * inv);
            v.y = pack_half2(__uint_as_float(o[8 * i + 2]) * inv, __uint_as_float(o[8 * i + 3]) * inv);
            v.z = pack_half2(__uint_as_float(o[8 * i + 4]) * inv, __uint_as_float(o[8 * i + 5]) * inv);
            v.w = pack_half2(__uint_as_float(o[8 * i + 6]) * inv, __uint_as_float(o[8 * i + 7]) * inv);
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
extern "C" VMK_API int vmk_debug_tc_timing(long long* out, int reset) {
  long long zero[16] = {0};
  cudaDeviceSynchronize();
  if (out) cudaMemcpyFromSymbol(out, g_tc_timing, sizeof(zero));
  if (reset) cudaMemcpyToSymbol(g_tc_timing, zero, sizeof(zero));
  return 0;
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
  attn_tc_kernel<<<n_cta, kTcThreads, kAttnTcSmem, stream>>>(p);
  return check_launch(cudaGetLastError());
}

}  // namespace vmk
