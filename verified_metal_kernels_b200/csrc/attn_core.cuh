// Split-KV decode attention core shared by `prefix` and `spec`.
//
// One CTA = one (key group z, row tile, key split).  The rows of a tile are the stacked query rows that
// share the group's keys (requests x GQA heads for the shared prefix, draft rows x GQA heads for
// speculative verification, the GQA heads alone for a private suffix).  Keys stream through a ring of
// TMA-filled shared-memory stages (K and V tiles of 64 keys x 128, 128-byte swizzle, out-of-range keys
// read as zero); scores, softmax statistics and the output accumulate in fp32; P is rounded to fp16 for
// the P.V product, as fused fp16 SDPA implementations do.  Each CTA emits an un-normalised partial
// (m, l, o) per row, m in the base-2 scaled-score domain; a combine pass merges the splits.
//
// Warp layout inside a CTA: RT row tiles of 16 rows x KS key slices; warp (rt, ks) owns rows
// [16 rt, 16 rt + 16) and keys [ks*64/KS, (ks+1)*64/KS) of every 64-key block, with private softmax
// statistics that are merged through shared memory at the end.  Small row counts therefore still use
// every warp (decode shapes have 4..32 rows), large ones get up to 128 rows per CTA.
#pragma once

#include <limits.h>

#include "common.cuh"

namespace vmk {

constexpr int kBK = 64;                       // keys per stage
constexpr int kHD = 128;                      // head dimension
constexpr int kHalfTile = kBK * 128;          // one swizzled [64 keys][128 B] box
constexpr int kStageBytes = 4 * kHalfTile;    // K lo, K hi, V lo, V hi = 32 KiB
constexpr int kQStride = kHD * 2 + 16;        // padded query row in shared memory (bank-conflict free)
constexpr int kMergeStride = 132;             // floats per row in the end-of-CTA merge buffer
constexpr int kMaxMaskWords = VMK_SPEC_MAX_DRAFTS / 32;

struct AttnRole {
  CUtensorMap tmK, tmV;     // fp16 (groups, keys, 128), box (64, 64, 1)
  const __half* q;          // queries; row (outer, head) at ((outer * Hq) + head) * 128
  __half* out;              // same layout as q; written only when `direct`
  const uint32_t* bits;     // draft visibility words, row (outer) at outer * bits_words; null = no mask
  const int32_t* klens;     // valid key count per outer group (ragged suffixes); null = klen
  const int32_t* page_table;  // paged cache: page of keys [i * page_size, (i+1) * page_size) of outer group zg at
                              // page_table[zg * table_stride + i]; the tensor maps then describe
                              // (128, page_size, pages * Hkv).  null = one contiguous cache per group
  int page_size, table_stride, page_groups;   // page_groups = pages * Hkv: the first group index out of range
  float* part_o;            // ((z * nsplit + split) * MP + row) * 128
  float* part_ml;           // ((z * nsplit + split) * MP + row) * 2  -> (m, l)
  int n_groups, Hkv, G, Hq;
  int rows_outer;           // outer rows (requests / drafts) stacked per group; rows = rows_outer * G
  int row_tiles;            // ceil(rows / (16 RT))
  int nsplit, split_len;    // split_len is a multiple of 64
  int klen;                 // key extent of the tensor
  int key_lo, key_hi;       // keys processed: [key_lo, key_hi)
  int mask_start;           // keys at or beyond it are subject to `bits` (INT_MAX = never)
  int bits_words;
  int MP;                   // padded rows per (group, split) in the partial arrays
  int direct;               // single split and nothing to merge with: write the fp16 result
  int n_cta;
};

struct AttnParams {
  AttnRole a, b;            // b is used only by kernels instantiated with HAS_B
  float sc;                 // softmax scale * log2(e)
  int32_t* status;
  int bf16;                 // q, K, V and out are bf16 instead of fp16
};

#ifdef VMK_ATTN_TIMING
// Debug build only.  Global-timer stamps of every CTA of the last split-KV launch: [cta][mark], and of the
// combine pass: [16 * 1024 + mark].
__device__ long long g_attn_marks[16 * 1025];
#define ATTN_M(cta, k) do { if (threadIdx.x == 0 && (cta) <= 1024) { long long _t; \
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(_t)); g_attn_marks[(cta) * 16 + (k)] = _t; } } while (0)
#else
#define ATTN_M(cta, k) do {} while (0)
#endif

template <int RT, int STAGES>
constexpr int attn_smem_bytes() {
  return STAGES * kStageBytes + RT * 16 * kQStride + STAGES * 8 + 1024 /* alignment slack */;
}

template <int RT, int KS, int STAGES, bool BF>
__device__ __forceinline__ void attn_core(const AttnRole& R, float sc, int32_t* status, int cta, uint8_t* smem) {
  // the warp-level MMA of the call's 16-bit type
  auto mma = [](float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (BF) mma_16816_bf16(c, a, b0, b1); else mma_16816(c, a, b0, b1);
  };
  constexpr int NW = RT * KS;          // computing warps
  constexpr int KPW = kBK / KS;        // keys per warp per block
  constexpr int NT8 = KPW / 8;         // score n-tiles per warp
  constexpr int MT = RT * 16;
  static_assert(KPW >= 16 && NW <= 8, "warp layout");

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nthreads = blockDim.x;
  const bool active = warp < NW;
  const int rt = warp / KS, ks = warp % KS;
  ATTN_M(blockIdx.x, 0);

  // ---- which piece of work --------------------------------------------------------------------
  const int split = cta % R.nsplit;
  const int t2 = cta / R.nsplit;
  const int tile = t2 % R.row_tiles;
  const int z = t2 / R.row_tiles;
  const int zg = z / R.Hkv, h = z % R.Hkv;
  const int rows = R.rows_outer * R.G;
  const int row0 = tile * MT;
  // Set-up that reads nothing a kernel before this one could have written: the barriers, the tensor-map
  // descriptors, and L2 prefetches of the first key blocks of the range (hints: they need no shared memory, and
  // a block beyond the group's true length is merely fetched for nothing).  The kernel is launched as a
  // programmatic dependent, so in a chain of calls all this overlaps the tail of the call before; every read of
  // the call's inputs stands after pdl_wait.
  uint8_t* stage0 = smem;
  uint8_t* sQ = smem + STAGES * kStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sQ + MT * kQStride);
  if (tid == 0) {
    for (int s = 0; s < STAGES; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
    tma_prefetch_desc(&R.tmK);
    tma_prefetch_desc(&R.tmV);
    if (R.page_table == nullptr) {
      const int kb0 = R.key_lo + split * R.split_len;
      const int ke0 = min(kb0 + R.split_len, R.key_hi);
      for (int j = 0; j < STAGES && kb0 + j * kBK < ke0; ++j) {
        tma_prefetch_3d(&R.tmK, 0, kb0 + j * kBK, z);
        tma_prefetch_3d(&R.tmK, 64, kb0 + j * kBK, z);
        tma_prefetch_3d(&R.tmV, 0, kb0 + j * kBK, z);
        tma_prefetch_3d(&R.tmV, 64, kb0 + j * kBK, z);
      }
    }
  }
  pdl_wait();
  ATTN_M(blockIdx.x, 8);

  // Every global load of the set-up is requested before any of them is waited for (on a cold cache each is a
  // round trip to DRAM: taken one after the other they used to be most of a small call's time): this thread's
  // part of the query tile, its draft-visibility words and the group's key count.
  constexpr int kQPer = (MT * 16 + 255) / 256;          // 16-byte chunks of the query tile per thread (256 threads)
  uint4 qreg[kQPer];
#pragma unroll
  for (int u = 0; u < kQPer; ++u) {
    const int i = tid + u * nthreads;
    const int r = i >> 4, c = i & 15;
    const int row = row0 + r;
    qreg[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < MT * 16 && row < rows) {
      const size_t outer = (size_t)zg * R.rows_outer + row / R.G;
      const int head = h * R.G + row % R.G;
      qreg[u] = *reinterpret_cast<const uint4*>(R.q + (outer * R.Hq + head) * kHD + c * 8);
    }
  }
  // The two rows this thread owns in its warp's 16-row tile, and their draft-visibility words.
  const int r_lo = row0 + rt * 16 + (lane >> 2), r_hi = r_lo + 8;
  uint32_t mw_lo[kMaxMaskWords], mw_hi[kMaxMaskWords];
#pragma unroll
  for (int w = 0; w < kMaxMaskWords; ++w) mw_lo[w] = mw_hi[w] = 0xffffffffu;
  if (R.bits != nullptr && active) {
#pragma unroll
    for (int w = 0; w < kMaxMaskWords; ++w) {
      if (w < R.bits_words) {
        if (r_lo < rows) mw_lo[w] = R.bits[((size_t)zg * R.rows_outer + r_lo / R.G) * R.bits_words + w];
        if (r_hi < rows) mw_hi[w] = R.bits[((size_t)zg * R.rows_outer + r_hi / R.G) * R.bits_words + w];
      }
    }
  }

  const int kbeg = R.key_lo + split * R.split_len;
  int kend = min(kbeg + R.split_len, R.key_hi);
  if (R.klens != nullptr) {
    int kv = R.klens[zg];
    if (kv < 0 || kv > R.klen) {
      report(status, kStatusBadIndex);
      kv = max(0, min(kv, R.klen));
    }
    kend = min(kend, kv);
  }
  const int nblk = kend > kbeg ? (kend - kbeg + kBK - 1) / kBK : 0;
  ATTN_M(blockIdx.x, 9);
  __syncthreads();                                      // the barriers are initialised
  ATTN_M(blockIdx.x, 10);

  auto issue = [&](int j) {
    const int s = j % STAGES;
    uint8_t* st = stage0 + s * kStageBytes;
    int kb = kbeg + j * kBK, zz = z;
    if (R.page_table != nullptr) {
      // a 64-key tile lies inside one page (page_size is a multiple of 64); a page id outside the pool makes
      // the TMA coordinate out of range, which reads zeros
      const int pi = kb / R.page_size;
      const int pg = pi < R.table_stride ? R.page_table[(size_t)zg * R.table_stride + pi] : -1;
      zz = (pg >= 0 && pg * R.Hkv + h < R.page_groups) ? pg * R.Hkv + h : R.page_groups;
      kb -= pi * R.page_size;
    }
    mbar_expect_tx(&bars[s], kStageBytes);
    tma_load_3d(st, &R.tmK, 0, kb, zz, &bars[s]);
    tma_load_3d(st + kHalfTile, &R.tmK, 64, kb, zz, &bars[s]);
    tma_load_3d(st + 2 * kHalfTile, &R.tmV, 0, kb, zz, &bars[s]);
    tma_load_3d(st + 3 * kHalfTile, &R.tmV, 64, kb, zz, &bars[s]);
  };
  if (tid == 0) {
    for (int j = 0; j < STAGES && j < nblk; ++j) issue(j);
  }
  ATTN_M(blockIdx.x, 11);

  // ---- query tile -> shared memory -> A fragments ------------------------------------------------
#pragma unroll
  for (int u = 0; u < kQPer; ++u) {
    const int i = tid + u * nthreads;
    if (i < MT * 16) *reinterpret_cast<uint4*>(sQ + (i >> 4) * kQStride + (i & 15) * 16) = qreg[u];
  }
  __syncthreads();
  ATTN_M(blockIdx.x, 12);

  uint32_t qf[8][4];
  if (active) {
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      ldsm_x4(qf[kk], smem_u32(sQ + (rt * 16 + (lane & 15)) * kQStride + (kk * 2 + (lane >> 4)) * 16));
  }

  auto visible = [&](const uint32_t (&mw)[kMaxMaskWords], int j) -> bool {
    uint32_t word = mw[0];
#pragma unroll
    for (int w = 1; w < kMaxMaskWords; ++w) word = ((j >> 5) == w) ? mw[w] : word;
    return (word >> (j & 31)) & 1u;
  };

  ATTN_M(blockIdx.x, 1);
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;

  // ---- key blocks ---------------------------------------------------------------------------------
  for (int j = 0; j < nblk; ++j) {
    const int s = j % STAGES;
    const bool arrived = mbar_wait(&bars[s], (uint32_t)((j / STAGES) & 1));
    if (__syncthreads_or(!arrived)) {   // also: every warp is done with block j-1
      // Give up.  The loads already requested (blocks j .. j + STAGES - 2, or the first STAGES blocks) may still be
      // landing in this CTA's shared memory: wait for them, with the same bound, so that the SM cannot hand the
      // memory to another CTA under them.  The whole call's output is invalid once the status bit is set.
      if (tid == 0) {
        report(status, kStatusTimeout);
        const int issued = min(nblk, j == 0 ? STAGES : j + STAGES - 1);
        for (int b = j; b < issued; ++b) mbar_wait(&bars[b % STAGES], (uint32_t)((b / STAGES) & 1));
      }
      __syncthreads();
      return;
    }
    if (tid == 0 && j >= 1 && j - 1 + STAGES < nblk) issue(j - 1 + STAGES);
    if (j == 0) ATTN_M(blockIdx.x, 2);

    uint8_t* st = stage0 + s * kStageBytes;
    const int kb = kbeg + j * kBK;
    const bool tail = kb + kBK > kend;
    if (tail && (kend < R.klen || R.page_table != nullptr)) {
      // Keys past kend exist in memory (ragged length / split of another rank / rest of a page): their V rows
      // must not reach the MMA, where 0 * Inf would poison the row.  Uniform across the CTA.
      const int r0 = kend - kb;
      for (int i = tid; i < (kBK - r0) * 16; i += nthreads) {
        const int r = r0 + (i >> 4), c = i & 15;
        *reinterpret_cast<uint4*>(st + (2 + (c >> 3)) * kHalfTile + swz128(r, c & 7)) = make_uint4(0u, 0u, 0u, 0u);
      }
      __syncthreads();
    }
    if (!active) continue;

    // S = Q K^T for this warp's 16 rows x KPW keys
    float sacc[NT8][4];
#pragma unroll
    for (int n = 0; n < NT8; ++n) sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
    const int key0 = ks * KPW;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
      for (int np = 0; np < KPW / 16; ++np) {
        // matrices: (keys 0-7, d 0-7) (keys 0-7, d 8-15) (keys 8-15, d 0-7) (keys 8-15, d 8-15)
        const int mi = lane >> 3;
        const uint32_t key = key0 + np * 16 + (mi >> 1) * 8 + (lane & 7);
        const uint32_t ch = kk * 2 + (mi & 1);
        uint32_t b[4];
        ldsm_x4(b, smem_u32(st + (ch >> 3) * kHalfTile + swz128(key, ch & 7)));
        mma(sacc[2 * np], qf[kk], b[0], b[1]);
        mma(sacc[2 * np + 1], qf[kk], b[2], b[3]);
      }
    }

    // scale, mask, online softmax
    float bm_lo = -INFINITY, bm_hi = -INFINITY;
    const bool edge = tail || (kb + kBK > R.mask_start);
    if (!edge) {
      // interior block: every key visible; no per-element branches in the hot path
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
        sacc[n][0] *= sc; sacc[n][1] *= sc; sacc[n][2] *= sc; sacc[n][3] *= sc;
        bm_lo = fmaxf(bm_lo, fmaxf(sacc[n][0], sacc[n][1]));
        bm_hi = fmaxf(bm_hi, fmaxf(sacc[n][2], sacc[n][3]));
      }
    } else {
#pragma unroll
      for (int n = 0; n < NT8; ++n) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int key = kb + key0 + n * 8 + 2 * (lane & 3) + (e & 1);
          bool ok = key < kend;
          if (ok && key >= R.mask_start) ok = visible((e < 2) ? mw_lo : mw_hi, key - R.mask_start);
          const float t = ok ? sacc[n][e] * sc : -INFINITY;
          sacc[n][e] = t;
          if (e < 2) bm_lo = fmaxf(bm_lo, t); else bm_hi = fmaxf(bm_hi, t);
        }
      }
    }
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 1));
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 2));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 1));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 2));
    const float mn_lo = fmaxf(m_lo, bm_lo), mn_hi = fmaxf(m_hi, bm_hi);
    const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float al_lo = exp2f(m_lo - mu_lo), al_hi = exp2f(m_hi - mu_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int n = 0; n < NT8; ++n) {
      sacc[n][0] = exp2f(sacc[n][0] - mu_lo);
      sacc[n][1] = exp2f(sacc[n][1] - mu_lo);
      sacc[n][2] = exp2f(sacc[n][2] - mu_hi);
      sacc[n][3] = exp2f(sacc[n][3] - mu_hi);
      ps_lo += sacc[n][0] + sacc[n][1];
      ps_hi += sacc[n][2] + sacc[n][3];
    }
    l_lo = l_lo * al_lo + ps_lo;
    l_hi = l_hi * al_hi + ps_hi;
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      oacc[i][0] *= al_lo;
      oacc[i][1] *= al_lo;
      oacc[i][2] *= al_hi;
      oacc[i][3] *= al_hi;
    }

    // O += P V
#pragma unroll
    for (int k2 = 0; k2 < KPW / 16; ++k2) {
      uint32_t pa[4];
      pa[0] = pack2(sacc[2 * k2][0], sacc[2 * k2][1], BF);
      pa[1] = pack2(sacc[2 * k2][2], sacc[2 * k2][3], BF);
      pa[2] = pack2(sacc[2 * k2 + 1][0], sacc[2 * k2 + 1][1], BF);
      pa[3] = pack2(sacc[2 * k2 + 1][2], sacc[2 * k2 + 1][3], BF);
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        // transposed matrices: (keys 0-7, d 0-7) (keys 8-15, d 0-7) (keys 0-7, d 8-15) (keys 8-15, d 8-15)
        const int mi = lane >> 3;
        const uint32_t key = key0 + k2 * 16 + (mi & 1) * 8 + (lane & 7);
        const uint32_t ch = dp * 2 + (mi >> 1);
        uint32_t b[4];
        ldsm_x4_t(b, smem_u32(st + (2 + (ch >> 3)) * kHalfTile + swz128(key, ch & 7)));
        mma(oacc[2 * dp], pa, b[0], b[1]);
        mma(oacc[2 * dp + 1], pa, b[2], b[3]);
      }
    }
  }

  // ---- merge the KS key slices of each row tile, emit ------------------------------------------
  __syncthreads();   // every stage has been consumed; the ring is reused as the merge buffer
  ATTN_M(blockIdx.x, 3);
  float* mo = reinterpret_cast<float*>(stage0);                      // [NW][16][kMergeStride]
  float* ml = mo + NW * 16 * kMergeStride;                           // [NW][16][2]
  if (active) {
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
    l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
    l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
    float* wo = mo + warp * 16 * kMergeStride;
    const int rl = lane >> 2, c0 = 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      *reinterpret_cast<float2*>(wo + rl * kMergeStride + i * 8 + c0) = make_float2(oacc[i][0], oacc[i][1]);
      *reinterpret_cast<float2*>(wo + (rl + 8) * kMergeStride + i * 8 + c0) = make_float2(oacc[i][2], oacc[i][3]);
    }
    if ((lane & 3) == 0) {
      ml[(warp * 16 + rl) * 2] = m_lo;
      ml[(warp * 16 + rl) * 2 + 1] = l_lo;
      ml[(warp * 16 + rl + 8) * 2] = m_hi;
      ml[(warp * 16 + rl + 8) * 2 + 1] = l_hi;
    }
  }
  __syncthreads();
  ATTN_M(blockIdx.x, 5);
  // per row: the common maximum of its KS slices, their weights 2^(m_k - M) and the merged row sum, computed
  // once (one thread per row) instead of once per output element
  float* wts = ml + NW * 16 * 2;                                     // [MT][KS]
  float* rowM = wts + MT * KS;                                       // [MT]
  float* rowL = rowM + MT;                                           // [MT]
  for (int row = tid; row < MT; row += nthreads) {
    const int wr = (row >> 4) * KS, rr = row & 15;
    float M = -INFINITY;
#pragma unroll
    for (int k = 0; k < KS; ++k) M = fmaxf(M, ml[((wr + k) * 16 + rr) * 2]);
    float lsum = 0.f;
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      const float mk = ml[((wr + k) * 16 + rr) * 2];
      const float wgt = (mk == -INFINITY) ? 0.f : exp2f(mk - M);
      wts[row * KS + k] = wgt;
      lsum += wgt * ml[((wr + k) * 16 + rr) * 2 + 1];
    }
    rowM[row] = M;
    rowL[row] = lsum;
  }
  __syncthreads();
  const size_t slot = (size_t)z * R.nsplit + split;
  for (int i = tid; i < MT * (kHD / 4); i += nthreads) {             // four columns per thread and step
    const int row = i >> 5, d = (i & 31) * 4;
    const int grow = row0 + row;
    if (grow >= rows) continue;
    const int wr = (row >> 4) * KS, rr = row & 15;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < KS; ++k) {
      const float wgt = wts[row * KS + k];
      const float4 v = *reinterpret_cast<const float4*>(mo + ((wr + k) * 16 + rr) * kMergeStride + d);
      acc.x += wgt * v.x; acc.y += wgt * v.y; acc.z += wgt * v.z; acc.w += wgt * v.w;
    }
    if (R.direct) {
      const size_t outer = (size_t)zg * R.rows_outer + grow / R.G;
      const int head = h * R.G + grow % R.G;
      const float lsum = rowL[row];
      uint2 pk;
      pk.x = pack2(acc.x / lsum, acc.y / lsum, BF);
      pk.y = pack2(acc.z / lsum, acc.w / lsum, BF);
      *reinterpret_cast<uint2*>(&R.out[(outer * R.Hq + head) * kHD + d]) = pk;
    } else {
      *reinterpret_cast<float4*>(R.part_o + (slot * R.MP + grow) * kHD + d) = acc;
      if (d == 0) *reinterpret_cast<float2*>(R.part_ml + (slot * R.MP + grow) * 2) = make_float2(rowM[row], rowL[row]);
    }
  }
  ATTN_M(blockIdx.x, 6);
  __syncthreads();
  ATTN_M(blockIdx.x, 4);
}

}  // namespace vmk
