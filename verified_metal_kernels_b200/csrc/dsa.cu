// `dsa`: indexer (stage 1), sparse absorbed-MLA attention (stage 3) and the fused entry point.
// Stage 2 (top-2048 select) lives in dsa_select.cu, the tcgen05 indexer in dsa_indexer_tc.cu.
#include "common.cuh"
#include "dsa_mla_tc.cuh"

namespace vmk {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kHI = 64;        // indexer heads
constexpr int kDI = 128;       // indexer width
constexpr int kMH = 128;       // attention heads
constexpr int kDK = 576;       // latent row: 512 latent + 64 rope
constexpr int kDV = 512;       // value = first 512 columns of the row

int indexer_tc_launch(const CUtensorMap& tmIK, const CUtensorMap& tmIQ, const float* w, const int32_t* lens,
                      float* scores, uint32_t* hist, int B, int L, int32_t* status, cudaStream_t stream, int bf16,
                      const int32_t* page_table, int page_size, int table_stride, int pages, const float* iq_scale,
                      const float* ik_scale);

int select_launch(const float* scores, const uint32_t* hist, const int32_t* lens, int32_t* idx, int32_t* cnt, int B,
                  int L, cudaStream_t stream);

// ================================================================================================
// Stage 1, mma.sync variant: scores[b,l] = sum_h w[b,h] * relu(iq[b,h] . ik[b,l])
//
// grid (chunks, B).  A CTA owns a contiguous run of 128-position tiles of one request, streams them
// through a 6-deep TMA ring (32 KiB per tile) and keeps the request's 64x128 indexer queries as B
// fragments in registers.  Warp w computes positions [16w, 16w+16) of each tile against all 64 heads
// (fp32 accumulation), applies ReLU and the head weights in fp32 and writes one score per position.
// ================================================================================================
constexpr int kIdxTile = 128;
constexpr int kIdxStages = 6;
constexpr int kIdxTileBytes = kIdxTile * kDI * 2;     // 32 KiB, two swizzled [128][128 B] boxes
constexpr int kIdxSmem = kIdxStages * kIdxTileBytes + kHI * kDI * 2 + (kIdxStages + 1) * 8 + 1024;

struct IndexerParams {
  CUtensorMap tmIK;      // (B, L, 128) box (64, 128, 1)
  CUtensorMap tmIQ;      // (B, 64, 128) box (64, 64, 1)
  const float* w;
  const int32_t* lens;
  float* scores;
  int B, L;
  int32_t* status;
};

__device__ __forceinline__ float relu_keep_nan(float x) { return (x < 0.f) ? 0.f : x; }

__global__ void __launch_bounds__(256, 1) indexer_mma_kernel(const __grid_constant__ IndexerParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sIQ = smem + kIdxStages * kIdxTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(sIQ + kHI * kDI * 2);   // [stages] + [iq]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  int n = p.L;
  if (p.lens != nullptr) n = max(0, min(p.lens[b], p.L));
  if (n <= kTopK) return;                               // every position is selected; no scores needed
  const int tiles = (n + kIdxTile - 1) / kIdxTile;
  const int per = (tiles + gridDim.x - 1) / gridDim.x;
  const int t0 = blockIdx.x * per;
  const int t1 = min(tiles, t0 + per);
  if (t0 >= t1) return;
  const int nt = t1 - t0;

  if (tid == 0) {
    for (int s = 0; s <= kIdxStages; ++s) mbar_init(&bars[s], 1);
    fence_mbar_init();
  }
  __syncthreads();
  auto issue = [&](int j) {
    const int s = j % kIdxStages;
    uint8_t* st = smem + s * kIdxTileBytes;
    mbar_expect_tx(&bars[s], kIdxTileBytes);
    tma_load_3d(st, &p.tmIK, 0, (t0 + j) * kIdxTile, b, &bars[s]);
    tma_load_3d(st + kIdxTileBytes / 2, &p.tmIK, 64, (t0 + j) * kIdxTile, b, &bars[s]);
  };
  if (tid == 0) {
    mbar_expect_tx(&bars[kIdxStages], kHI * kDI * 2);
    tma_load_3d(sIQ, &p.tmIQ, 0, 0, b, &bars[kIdxStages]);
    tma_load_3d(sIQ + kHI * 128, &p.tmIQ, 64, 0, b, &bars[kIdxStages]);
    for (int j = 0; j < kIdxStages && j < nt; ++j) issue(j);
  }
  {
    const bool ok = mbar_wait(&bars[kIdxStages], 0);
    if (__syncthreads_or(!ok)) {
      if (tid == 0) report(p.status, kStatusTimeout);
      return;
    }
  }
  // B fragments of iq: bq[kk][n8] covers heads [8 n8, 8 n8 + 8) x d [16 kk, 16 kk + 16)
  uint32_t bq[8][8][2];
#pragma unroll
  for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
    for (int np = 0; np < 4; ++np) {
      const int mi = lane >> 3;
      const uint32_t head = np * 16 + (mi >> 1) * 8 + (lane & 7);
      const uint32_t ch = kk * 2 + (mi & 1);
      uint32_t t[4];
      ldsm_x4(t, smem_u32(sIQ + (ch >> 3) * (kHI * 128) + swz128(head, ch & 7)));
      bq[kk][2 * np][0] = t[0];
      bq[kk][2 * np][1] = t[1];
      bq[kk][2 * np + 1][0] = t[2];
      bq[kk][2 * np + 1][1] = t[3];
    }
  }
  float wv[8][2];
#pragma unroll
  for (int n8 = 0; n8 < 8; ++n8) {
    wv[n8][0] = p.w[b * kHI + n8 * 8 + 2 * (lane & 3)];
    wv[n8][1] = p.w[b * kHI + n8 * 8 + 2 * (lane & 3) + 1];
  }

  for (int j = 0; j < nt; ++j) {
    const int s = j % kIdxStages;
    const bool ok = mbar_wait(&bars[s], (uint32_t)((j / kIdxStages) & 1));
    if (__syncthreads_or(!ok)) {
      if (tid == 0) report(p.status, kStatusTimeout);
      return;
    }
    if (tid == 0 && j >= 1 && j - 1 + kIdxStages < nt) issue(j - 1 + kIdxStages);
    const uint8_t* st = smem + s * kIdxTileBytes;
    float acc[8][4];
#pragma unroll
    for (int n8 = 0; n8 < 8; ++n8) acc[n8][0] = acc[n8][1] = acc[n8][2] = acc[n8][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < 8; ++kk) {
      const uint32_t row = warp * 16 + (lane & 15);
      const uint32_t ch = kk * 2 + (lane >> 4);
      uint32_t a[4];
      ldsm_x4(a, smem_u32(st + (ch >> 3) * (kIdxTileBytes / 2) + swz128(row, ch & 7)));
#pragma unroll
      for (int n8 = 0; n8 < 8; ++n8) mma_16816(acc[n8], a, bq[kk][n8][0], bq[kk][n8][1]);
    }
    float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
    for (int n8 = 0; n8 < 8; ++n8) {
      s_lo += wv[n8][0] * relu_keep_nan(acc[n8][0]) + wv[n8][1] * relu_keep_nan(acc[n8][1]);
      s_hi += wv[n8][0] * relu_keep_nan(acc[n8][2]) + wv[n8][1] * relu_keep_nan(acc[n8][3]);
    }
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
    s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
    s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
    s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
    if ((lane & 3) == 0) {
      const int pos = (t0 + j) * kIdxTile + warp * 16 + (lane >> 2);
      float* dst = p.scores + (size_t)b * p.L;
      if (pos < n) dst[pos] = s_lo;
      if (pos + 8 < n) dst[pos + 8] = s_hi;
    }
  }
}

// ================================================================================================
// Stage 3: absorbed-MLA attention over the selected rows.
//
// grid (splits, 4 head groups, B), 256 threads.  A CTA handles 32 heads of one request over a range of
// the selected positions, 64 at a time: the 576-wide latent rows are gathered by index into a padded
// shared-memory tile (cp.async, double buffered); warp (rt, sl) computes the scores of heads
// [16 rt, 16 rt + 16) against keys [16 sl, 16 sl + 16), the four warps of a row tile exchange row maxima
// and P through shared memory, and each then accumulates its 128-column slice of P.V, where V is the
// first 512 columns of the very same tile.
// ================================================================================================
constexpr int kMlaHeads = 32;                 // heads per CTA
constexpr int kMlaBK = 64;                    // gathered rows per block
constexpr int kRowStride = kDK * 2 + 16;      // 1168 B: padded so that ldmatrix rows fall in distinct banks
constexpr int kPStride = kMlaBK * 2 + 16;     // 144 B
constexpr int kMlaQBytes = kMlaHeads * kRowStride;
constexpr int kMlaStageBytes = kMlaBK * kRowStride;
constexpr int kMlaSmem = kMlaQBytes + 2 * kMlaStageBytes + kMlaHeads * kPStride + 2 * 4 * 16 * 4 * 2 + 128;

struct MlaParams {
  const __half* q;
  const __half* kv;
  const int32_t* idx;
  const int32_t* cnt;
  __half* out;
  float* part_o;       // ((b * nsplit + split) * 128 + head) * 512
  float* part_ml;      // ((b * nsplit + split) * 128 + head) * 2
  int B, L, nsplit, split_len;
  float sc;
  int32_t* status;
};

__device__ __forceinline__ void named_bar(int id, int count) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(count) : "memory");
}

__global__ void __launch_bounds__(256, 1) mla_kernel(const MlaParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kMlaQBytes;
  uint8_t* sP = sK + 2 * kMlaStageBytes;
  float* smax = reinterpret_cast<float*>(sP + kMlaHeads * kPStride);   // [2 rt][4 sl][16]
  float* ssum = smax + 2 * 4 * 16;                                      // [2 rt][4 sl][16]

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rt = warp >> 2, sl = warp & 3;
  const int split = blockIdx.x, hg = blockIdx.y, b = blockIdx.z;
  const int nb = max(0, min(p.cnt[b], kTopK));
  const int k0 = split * p.split_len;
  const int k1 = min(nb, k0 + p.split_len);
  const int nblk = k1 > k0 ? (k1 - k0 + kMlaBK - 1) / kMlaBK : 0;
  const __half* kvb = p.kv + (size_t)b * p.L * kDK;
  const int32_t* idxb = p.idx + (size_t)b * kTopK;

  // gather of block j into stage j & 1: 8 lanes per row, 32 rows per pass
  auto gather = [&](int j) {
    uint8_t* st = sK + (j & 1) * kMlaStageBytes;
#pragma unroll
    for (int pass = 0; pass < 2; ++pass) {
      const int r = (tid >> 3) + pass * 32;
      const int kidx = k0 + j * kMlaBK + r;
      const bool valid = kidx < k1;
      int row = valid ? idxb[kidx] : 0;
      if (row < 0 || row >= p.L) {
        report(p.status, kStatusBadIndex);
        row = 0;
      }
      const __half* src = kvb + (size_t)row * kDK;
      uint8_t* dst = st + r * kRowStride;
#pragma unroll
      for (int u = 0; u < 9; ++u) {
        const int c = (tid & 7) + 8 * u;
        cp_async16(dst + c * 16, src + c * 8, valid ? 16 : 0);
      }
    }
  };
  if (nblk > 0) gather(0);
  cp_async_commit();
  if (nblk > 1) gather(1);
  cp_async_commit();

  // Q tile: 32 heads x 576
  for (int i = tid; i < kMlaHeads * 72; i += 256) {
    const int r = i / 72, c = i % 72;
    const uint4 v = *reinterpret_cast<const uint4*>(p.q + ((size_t)b * kMH + hg * kMlaHeads + r) * kDK + c * 8);
    *reinterpret_cast<uint4*>(sQ + r * kRowStride + c * 16) = v;
  }

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float oacc[16][4];
#pragma unroll
  for (int i = 0; i < 16; ++i) oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.f;
  const int rl = lane >> 2;

  for (int j = 0; j < nblk; ++j) {
    cp_async_wait<1>();
    __syncthreads();                       // block j (and Q) visible to every warp
    const uint8_t* st = sK + (j & 1) * kMlaStageBytes;

    // S = Q K^T : 16 heads x 16 keys, K = 576
    // Two accumulator sets (even / odd K steps) halve the dependent-MMA chain of the 36-step reduction.
    float sacc[2][4], sodd[2][4];
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      sacc[n][0] = sacc[n][1] = sacc[n][2] = sacc[n][3] = 0.f;
      sodd[n][0] = sodd[n][1] = sodd[n][2] = sodd[n][3] = 0.f;
    }
    {
      const int mi = lane >> 3;
      const uint32_t qa = smem_u32(sQ + (rt * 16 + (lane & 15)) * kRowStride + (lane >> 4) * 16);
      const uint32_t ka = smem_u32(st + (sl * 16 + (mi >> 1) * 8 + (lane & 7)) * kRowStride + (mi & 1) * 16);
#pragma unroll 6
      for (int kk = 0; kk < kDK / 16; kk += 2) {
        uint32_t a0[4], b0[4], a1[4], b1[4];
        ldsm_x4(a0, qa + kk * 32);
        ldsm_x4(b0, ka + kk * 32);
        ldsm_x4(a1, qa + kk * 32 + 32);
        ldsm_x4(b1, ka + kk * 32 + 32);
        mma_16816(sacc[0], a0, b0[0], b0[1]);
        mma_16816(sacc[1], a0, b0[2], b0[3]);
        mma_16816(sodd[0], a1, b1[0], b1[1]);
        mma_16816(sodd[1], a1, b1[2], b1[3]);
      }
    }
#pragma unroll
    for (int n = 0; n < 2; ++n)
#pragma unroll
      for (int e = 0; e < 4; ++e) sacc[n][e] += sodd[n][e];
    float bm_lo = -INFINITY, bm_hi = -INFINITY;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = k0 + j * kMlaBK + sl * 16 + n * 8 + 2 * (lane & 3) + (e & 1);
        const float t = key < k1 ? sacc[n][e] * p.sc : -INFINITY;
        sacc[n][e] = t;
        if (e < 2) bm_lo = fmaxf(bm_lo, t); else bm_hi = fmaxf(bm_hi, t);
      }
    }
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 1));
    bm_lo = fmaxf(bm_lo, __shfl_xor_sync(0xffffffffu, bm_lo, 2));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 1));
    bm_hi = fmaxf(bm_hi, __shfl_xor_sync(0xffffffffu, bm_hi, 2));
    if ((lane & 3) == 0) {
      smax[(rt * 4 + sl) * 16 + rl] = bm_lo;
      smax[(rt * 4 + sl) * 16 + rl + 8] = bm_hi;
    }
    named_bar(1 + rt, 128);
    float mn_lo = m_lo, mn_hi = m_hi;
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mn_lo = fmaxf(mn_lo, smax[(rt * 4 + k) * 16 + rl]);
      mn_hi = fmaxf(mn_hi, smax[(rt * 4 + k) * 16 + rl + 8]);
    }
    const float mu_lo = (mn_lo == -INFINITY) ? 0.f : mn_lo, mu_hi = (mn_hi == -INFINITY) ? 0.f : mn_hi;
    const float al_lo = exp2f(m_lo - mu_lo), al_hi = exp2f(m_hi - mu_hi);
    m_lo = mn_lo;
    m_hi = mn_hi;
    float ps_lo = 0.f, ps_hi = 0.f;
#pragma unroll
    for (int n = 0; n < 2; ++n) {
      const float p0 = exp2f(sacc[n][0] - mu_lo), p1 = exp2f(sacc[n][1] - mu_lo);
      const float p2 = exp2f(sacc[n][2] - mu_hi), p3 = exp2f(sacc[n][3] - mu_hi);
      ps_lo += p0 + p1;
      ps_hi += p2 + p3;
      const int col = (sl * 16 + n * 8 + 2 * (lane & 3)) * 2;
      *reinterpret_cast<uint32_t*>(sP + (rt * 16 + rl) * kPStride + col) = pack_half2(p0, p1);
      *reinterpret_cast<uint32_t*>(sP + (rt * 16 + rl + 8) * kPStride + col) = pack_half2(p2, p3);
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
    named_bar(1 + rt, 128);

    // O[:, 128 sl : 128 sl + 128] += P V
#pragma unroll
    for (int k2 = 0; k2 < kMlaBK / 16; ++k2) {
      uint32_t pa[4];
      ldsm_x4(pa, smem_u32(sP + (rt * 16 + (lane & 15)) * kPStride + (k2 * 2 + (lane >> 4)) * 16));
#pragma unroll
      for (int dp = 0; dp < 8; ++dp) {
        const int mi = lane >> 3;
        const int key = k2 * 16 + (mi & 1) * 8 + (lane & 7);
        const int ch = sl * 16 + dp * 2 + (mi >> 1);
        uint32_t bb[4];
        ldsm_x4_t(bb, smem_u32(st + key * kRowStride + ch * 16));
        mma_16816(oacc[2 * dp], pa, bb[0], bb[1]);
        mma_16816(oacc[2 * dp + 1], pa, bb[2], bb[3]);
      }
    }
    __syncthreads();                       // stage j & 1 and sP are free again
    if (j + 2 < nblk) gather(j + 2);
    cp_async_commit();
  }
  cp_async_wait<0>();

  // ---- row sums across the four key slices, emit -----------------------------------------------
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  if ((lane & 3) == 0) {
    ssum[(rt * 4 + sl) * 16 + rl] = l_lo;
    ssum[(rt * 4 + sl) * 16 + rl + 8] = l_hi;
  }
  __syncthreads();
  float L_lo = 0.f, L_hi = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    L_lo += ssum[(rt * 4 + k) * 16 + rl];
    L_hi += ssum[(rt * 4 + k) * 16 + rl + 8];
  }
  const int head_lo = hg * kMlaHeads + rt * 16 + rl, head_hi = head_lo + 8;
  if (p.nsplit == 1) {
    __half* o_lo = p.out + ((size_t)b * kMH + head_lo) * kDV + sl * 128 + 2 * (lane & 3);
    __half* o_hi = p.out + ((size_t)b * kMH + head_hi) * kDV + sl * 128 + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      *reinterpret_cast<__half2*>(o_lo + i * 8) = __floats2half2_rn(oacc[i][0] / L_lo, oacc[i][1] / L_lo);
      *reinterpret_cast<__half2*>(o_hi + i * 8) = __floats2half2_rn(oacc[i][2] / L_hi, oacc[i][3] / L_hi);
    }
  } else {
    const size_t base = ((size_t)b * p.nsplit + split) * kMH;
    float* o_lo = p.part_o + (base + head_lo) * kDV + sl * 128 + 2 * (lane & 3);
    float* o_hi = p.part_o + (base + head_hi) * kDV + sl * 128 + 2 * (lane & 3);
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      *reinterpret_cast<float2*>(o_lo + i * 8) = make_float2(oacc[i][0], oacc[i][1]);
      *reinterpret_cast<float2*>(o_hi + i * 8) = make_float2(oacc[i][2], oacc[i][3]);
    }
    if (sl == 0 && (lane & 3) == 0) {
      p.part_ml[(base + head_lo) * 2] = m_lo;
      p.part_ml[(base + head_lo) * 2 + 1] = L_lo;
      p.part_ml[(base + head_hi) * 2] = m_hi;
      p.part_ml[(base + head_hi) * 2 + 1] = L_hi;
    }
  }
}

// Merge of the key splits: one CTA per (request, head), thread t owns value columns 4t..4t+3.
__global__ void __launch_bounds__(128) mla_combine_kernel(const float* __restrict__ part_o,
                                                          const float* __restrict__ part_ml, int nsplit,
                                                          __half* __restrict__ out) {
  const int head = blockIdx.x, b = blockIdx.y, t = threadIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < nsplit; ++s) M = fmaxf(M, part_ml[(((size_t)b * nsplit + s) * kMH + head) * 2]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
  for (int s = 0; s < nsplit; ++s) {
    const size_t r = ((size_t)b * nsplit + s) * kMH + head;
    const float m = part_ml[r * 2];
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    const float4 o = *reinterpret_cast<const float4*>(part_o + r * kDV + t * 4);
    acc.x += w * o.x; acc.y += w * o.y; acc.z += w * o.z; acc.w += w * o.w;
    lsum += w * part_ml[r * 2 + 1];
  }
  __half2* dst = reinterpret_cast<__half2*>(out + ((size_t)b * kMH + head) * kDV + t * 4);
  dst[0] = __floats2half2_rn(acc.x / lsum, acc.y / lsum);
  dst[1] = __floats2half2_rn(acc.z / lsum, acc.w / lsum);
}

// Compaction of the selected rows: kv_sel[b][j] = kv[b][idx[b][j]] for j < cnt[b], idx_sel[b][j] = j.  One warp
// per row (1152 B = 72 x 16 B).  `kv` only has to be readable from the device, so it may be page-locked HOST
// memory: a caller whose latent cache lives on the host then moves 2048 rows per request over the link instead
// of the whole cache.  grid (64, B), 256 threads: 32 rows per CTA.
__global__ void __launch_bounds__(256) gather_rows_kernel(const __half* __restrict__ kv, const int32_t* __restrict__ idx,
                                                          const int32_t* __restrict__ cnt, __half* __restrict__ kv_sel,
                                                          int32_t* __restrict__ idx_sel, int L, int32_t* status) {
  const int b = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = max(0, min(cnt[b], kTopK));
  const uint4* src_b = reinterpret_cast<const uint4*>(kv + (size_t)b * L * kDK);
  uint4* dst_b = reinterpret_cast<uint4*>(kv_sel + (size_t)b * kTopK * kDK);
#pragma unroll
  for (int r = 0; r < 4; ++r) {
    const int j = blockIdx.x * 32 + warp * 4 + r;
    if (j >= n) break;
    int row = idx[(size_t)b * kTopK + j];
    if (row < 0 || row >= L) {
      report(status, kStatusBadIndex);
      row = 0;
    }
    const uint4* src = src_b + (size_t)row * (kDK / 8);
    uint4* dst = dst_b + (size_t)j * (kDK / 8);
    const uint4 v0 = src[lane], v1 = src[lane + 32];
    uint4 v2 = make_uint4(0u, 0u, 0u, 0u);
    if (lane < 8) v2 = src[lane + 64];
    dst[lane] = v0;
    dst[lane + 32] = v1;
    if (lane < 8) dst[lane + 64] = v2;
    if (lane == 0) idx_sel[(size_t)b * kTopK + j] = j;
  }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// 0 = warp-level mma.sync kernel, 1 = tcgen05 kernel, one CTA per (request, value half), 2 = the same with a TMA row
// gather, 3 = tcgen05 kernel, a cluster of two CTAs per request (default)
static int g_attend_variant = 3;

// Key splits of the warp-level kernel.
static int mla_splits(int B) {
  int s = sm_count() / (B * (kMH / kMlaHeads));
  if (s < 1) s = 1;
  if (s > kTopK / (2 * kMlaBK)) s = kTopK / (2 * kMlaBK);   // at least two blocks per split
  return s;
}

struct DsaPlan {
  size_t off_scores, off_idx, off_cnt, off_hist, off_attend, ws_bytes;
};

// Stage-3 scratch: the larger of what the two implementations need, so a size queried under one test hook
// setting is valid under the other.
static size_t attend_ws(int B) {
  const int ns = mla_splits(B);
  const size_t warp_level =
      ns == 1 ? 256 : align_up((size_t)B * ns * kMH * kDV * 4, 256) + align_up((size_t)B * ns * kMH * 2 * 4, 256);
  size_t tc = mla_tc_workspace(B);
  const size_t pair = mla_pair_workspace(B);
  if (pair > tc) tc = pair;
  return warp_level > tc ? warp_level : tc;
}

static DsaPlan plan_dsa(int B, int L) {
  DsaPlan pl;
  pl.off_scores = 0;
  pl.off_idx = align_up((size_t)B * L * 4, 256);
  pl.off_cnt = pl.off_idx + align_up((size_t)B * kTopK * 4, 256);
  pl.off_hist = pl.off_cnt + align_up((size_t)B * 4, 256);
  pl.off_attend = pl.off_hist + align_up((size_t)B * kSelBins * 4, 256);
  pl.ws_bytes = pl.off_attend + attend_ws(B);
  return pl;
}

// Runs of tiles per request: CTAs are equal-sized and one is resident per SM, so the grid is chosen to
// fill whole waves (chunks * B close to a multiple of the SM count) with runs of at least 8 tiles.
int indexer_chunks(int B, int tiles) {
  const int sms = sm_count();
  int cmax = tiles / 8;
  if (cmax < 1) cmax = 1;
  if (cmax > 1024) cmax = 1024;
  int best = 1;
  double best_eff = -1.0;
  for (int c = 1; c <= cmax; ++c) {
    const double ctas = (double)c * B;
    const double waves = ctas / sms;
    const double eff = waves / (double)((long long)((ctas + sms - 1) / sms));
    // prefer more CTAs per wave-efficiency tie only while runs stay long; stop growing past 8 waves
    if (eff > best_eff + 1e-9 && (waves <= 8.0 || best_eff < 0)) {
      best_eff = eff;
      best = c;
    }
  }
  return best;
}

// Paged caches: the index keys (pages, page_size, 128) and the latent rows (pages, page_size, 576) share one page
// table (B, table_stride); pages == 0 means contiguous (B, L, .) tensors.
struct DsaPages {
  const int32_t* table;
  int pages, page_size, table_stride;
};

// bf16 = 1: the 16-bit tensors of the call are bf16 (only the tcgen05 implementations take them, and only they
// take a paged cache).
// Argument checks of stage 1, separate from the launch so that the entry points can run every check of a call
// before they enqueue anything (a refused call leaves the stream and the outputs untouched).
static int indexer_check(const void* iq, const void* ik, const float* w, const float* scores, int B, int L, int variant,
                         int bf16, const DsaPages& pg) {
  if (!iq || !ik || !w || !scores || B <= 0 || L <= 0) return VMK_E_BADARG;
  if ((bf16 || pg.pages > 0) && variant != 1) return VMK_E_UNSUPPORTED;
  if (pg.pages > 0 && (!pg.table || pg.page_size < kIdxTile || pg.page_size % kIdxTile != 0 || pg.table_stride <= 0 ||
                       (long long)pg.table_stride * pg.page_size < L))
    return VMK_E_BADARG;
  if (!aligned16(iq) || !aligned16(ik) || B > 65535) return VMK_E_BADARG;
  return VMK_OK;
}

static int indexer_impl(const void* iq, const void* ik, const float* w, const int32_t* lens, float* scores,
                        uint32_t* hist, int B, int L, int32_t* status, cudaStream_t stream, int variant, int bf16 = 0,
                        DsaPages pg = DsaPages{nullptr, 0, 0, 0}) {
  const int bad = indexer_check(iq, ik, w, scores, B, L, variant, bf16, pg);
  if (bad) return bad;
  if (L <= kTopK) return VMK_OK;                        // nothing to rank
  IndexerParams p;
  memset(&p, 0, sizeof(p));
  int rc = pg.pages > 0 ? make_tmap_3d(&p.tmIK, ik, kDI, pg.page_size, pg.pages, 64, kIdxTile)
                        : make_tmap_3d(&p.tmIK, ik, kDI, L, B, 64, kIdxTile);
  if (rc) return rc;
  rc = make_tmap_3d(&p.tmIQ, iq, kDI, kHI, B, 64, kHI);
  if (rc) return rc;
  if (variant == 1)
    return indexer_tc_launch(p.tmIK, p.tmIQ, w, lens, scores, hist, B, L, status, stream, bf16, pg.table, pg.page_size,
                             pg.table_stride, pg.pages, nullptr, nullptr);
  p.w = w; p.lens = lens; p.scores = scores; p.B = B; p.L = L; p.status = status;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(indexer_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kIdxSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  const int chunks = indexer_chunks(B, cdiv(L, kIdxTile));
  indexer_mma_kernel<<<dim3(chunks, B), 256, kIdxSmem, stream>>>(p);
  return check_launch(cudaGetLastError());
}

static int attend_check(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, const void* out, int B,
                        int L, const void* ws, size_t ws_bytes, int bf16, const DsaPages& pg) {
  if (!q || !kv || !idx || !cnt || !out || B <= 0 || L <= 0) return VMK_E_BADARG;
  if ((bf16 || pg.pages > 0) && g_attend_variant == 0) return VMK_E_UNSUPPORTED;
  if (!aligned16(q) || !aligned16(kv) || !aligned16(out) || B > 65535) return VMK_E_BADARG;
  if (!ws || ws_bytes < attend_ws(B) || (reinterpret_cast<uintptr_t>(ws) & 255)) return VMK_E_WORKSPACE;
  return VMK_OK;
}

static int attend_impl(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, void* out, int B,
                       int L, void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream, int bf16 = 0,
                       DsaPages pg = DsaPages{nullptr, 0, 0, 0}) {
  const int bad = attend_check(q, kv, idx, cnt, out, B, L, ws, ws_bytes, bf16, pg);
  if (bad) return bad;
  const int ns = mla_splits(B);
  MlaParams p;
  memset(&p, 0, sizeof(p));
  p.q = static_cast<const __half*>(q);
  p.kv = static_cast<const __half*>(kv);
  p.idx = idx; p.cnt = cnt;
  p.out = static_cast<__half*>(out);
  p.B = B; p.L = L; p.nsplit = ns;
  p.split_len = cdiv(cdiv(kTopK, ns), kMlaBK) * kMlaBK;
  p.sc = kLog2e / sqrtf(192.f);
  p.status = status;
  if (ns > 1) {
    p.part_o = static_cast<float*>(ws);
    p.part_ml = reinterpret_cast<float*>(static_cast<uint8_t*>(ws) + align_up((size_t)B * ns * kMH * kDV * 4, 256));
  }
  if (g_attend_variant >= 1) {
    MlaTcParams t;
    memset(&t, 0, sizeof(t));
    t.gather_tma = g_attend_variant == 2 ? 1 : 0;
    t.rows_total = pg.pages > 0 ? pg.pages * pg.page_size : B * L;
    if ((long long)t.rows_total != (pg.pages > 0 ? (long long)pg.pages * pg.page_size : (long long)B * L))
      return VMK_E_UNSUPPORTED;                        // row coordinates are 32-bit
    if (t.gather_tma) {
      const int rc = make_tmap_rows(&t.tmKV, kv, kDK, (uint64_t)t.rows_total);
      if (rc) return rc;
    }
    {
      const int rc = make_tmap_3d(&t.tmQ, q, kDK, kMH, (uint64_t)B, 64, 64);
      if (rc) return rc;
    }
    t.q = p.q; t.kv = p.kv; t.idx = p.idx; t.cnt = p.cnt; t.out = p.out; t.part_o = nullptr; t.part_ml = nullptr;
    t.B = B; t.L = L; t.ncta = 0; t.sc = p.sc; t.status = status; t.bf16 = bf16;
    t.page_table = pg.pages > 0 ? pg.table : nullptr;
    t.page_size = pg.page_size; t.table_stride = pg.table_stride; t.pages = pg.pages;
    if (g_attend_variant == 3) return mla_pair_launch(t, static_cast<float*>(ws), stream);
    return mla_tc_launch(t, static_cast<float*>(ws), stream);
  }
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(mla_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  mla_kernel<<<dim3(ns, kMH / kMlaHeads, B), 256, kMlaSmem, stream>>>(p);
  int rc = check_launch(cudaGetLastError());
  if (rc || ns == 1) return rc;
  mla_combine_kernel<<<dim3(kMH, B), 128, 0, stream>>>(p.part_o, p.part_ml, ns, p.out);
  return check_launch(cudaGetLastError());
}

static int g_indexer_variant = 1;   // 0 = mma.sync (warp-level), 1 = tcgen05 + tensor memory (default)

}  // namespace vmk

using namespace vmk;

// Test hook: chooses the stage-3 implementation (0 = warp-level mma.sync, 1 = tcgen05, one CTA per (request, value
// half), rows gathered by cp.async from four warps, 2 = the same with the rows gathered by TMA tile::gather4,
// 3 = tcgen05, a cluster of two CTAs per request that share the score product (default)).
extern "C" VMK_API int vmk_dsa_set_attend_variant(int v) {
  if (v < 0 || v > 3) return VMK_E_BADARG;
  g_attend_variant = v;
  return VMK_OK;
}

// Test hook: chooses the stage-1 implementation (0 = mma.sync, 1 = tcgen05).
extern "C" VMK_API int vmk_dsa_set_indexer_variant(int v) {
  if (v != 0 && v != 1) return VMK_E_BADARG;
  g_indexer_variant = v;
  return VMK_OK;
}

extern "C" int vmk_dsa_indexer(const void* iq, const void* ik, const float* w, const int32_t* lens, float* scores,
                               int B, int L, int32_t* status, void* stream) {
  return indexer_impl(iq, ik, w, lens, scores, nullptr, B, L, status, static_cast<cudaStream_t>(stream),
                      g_indexer_variant);
}

extern "C" int vmk_dsa_indexer_hist(const void* iq, const void* ik, const float* w, const int32_t* lens, float* scores,
                                    uint32_t* hist, int B, int L, int32_t* status, void* stream) {
  if (!hist) return VMK_E_BADARG;
  const int bad = indexer_check(iq, ik, w, scores, B, L, 1, 0, DsaPages{nullptr, 0, 0, 0});
  if (bad) return bad;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(hist, 0, (size_t)B * kSelBins * 4, st) != cudaSuccess) return VMK_E_LAUNCH;
  return indexer_impl(iq, ik, w, lens, scores, hist, B, L, status, st, 1);
}

extern "C" int vmk_dsa_select_hist(const float* scores, const uint32_t* hist, const int32_t* lens, int32_t* idx,
                                   int32_t* cnt, int B, int L, void* stream) {
  if (!hist) return VMK_E_BADARG;
  return select_launch(scores, hist, lens, idx, cnt, B, L, static_cast<cudaStream_t>(stream));
}

extern "C" size_t vmk_dsa_attend_workspace_bytes(int B) { return B > 0 ? attend_ws(B) : 0; }

extern "C" int vmk_dsa_attend(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, void* out, int B,
                              int L, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  return attend_impl(q, kv, idx, cnt, out, B, L, ws, ws_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" int vmk_dsa_gather(const void* kv, const int32_t* idx, const int32_t* cnt, void* kv_sel, int32_t* idx_sel,
                              int B, int L, int32_t* status, void* stream) {
  if (!kv || !idx || !cnt || !kv_sel || !idx_sel || B <= 0 || L <= 0 || B > 65535) return VMK_E_BADARG;
  if (!aligned16(kv) || !aligned16(kv_sel)) return VMK_E_BADARG;
  gather_rows_kernel<<<dim3(kTopK / 32, B), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(kv), idx, cnt, static_cast<__half*>(kv_sel), idx_sel, L, status);
  return check_launch(cudaGetLastError());
}

extern "C" size_t vmk_dsa_workspace_bytes(int B, int L) { return (B > 0 && L > 0) ? plan_dsa(B, L).ws_bytes : 0; }

static int decode_impl(const void* q, const void* kv, const void* iq, const void* ik, const float* w,
                       const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out, int B, int L, void* ws,
                       size_t ws_bytes, int32_t* status, void* stream, int bf16,
                       DsaPages pg = DsaPages{nullptr, 0, 0, 0}) {
  if (B <= 0 || L <= 0 || !ws || (reinterpret_cast<uintptr_t>(ws) & 255)) return VMK_E_BADARG;
  const DsaPlan pl = plan_dsa(B, L);
  if (ws_bytes < pl.ws_bytes) return VMK_E_WORKSPACE;
  uint8_t* base = static_cast<uint8_t*>(ws);
  float* scores = reinterpret_cast<float*>(base + pl.off_scores);
  int32_t* idx = idx_out ? idx_out : reinterpret_cast<int32_t*>(base + pl.off_idx);
  int32_t* cnt = cnt_out ? cnt_out : reinterpret_cast<int32_t*>(base + pl.off_cnt);
  // every argument check of the three stages before the first thing is enqueued
  int bad = indexer_check(iq, ik, w, scores, B, L, g_indexer_variant, bf16, pg);
  if (!bad) bad = attend_check(q, kv, idx, cnt, out, B, L, base + pl.off_attend, attend_ws(B), bf16, pg);
  if (bad) return bad;
  // The tcgen05 indexer also accumulates the first radix level of the select (a 2048-bin histogram per
  // request); the mma.sync variant does not, and the select then builds it in a pass of its own.
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  uint32_t* hist = nullptr;
  if (g_indexer_variant == 1 && L > kTopK) {
    hist = reinterpret_cast<uint32_t*>(base + pl.off_hist);
    if (cudaMemsetAsync(hist, 0, (size_t)B * kSelBins * 4, st) != cudaSuccess) return VMK_E_LAUNCH;
  }
  int rc = indexer_impl(iq, ik, w, lens, scores, hist, B, L, status, st, g_indexer_variant, bf16, pg);
  if (rc) return rc;
  if (!idx || !cnt) return VMK_E_BADARG;
  rc = select_launch(scores, hist, lens, idx, cnt, B, L, st);
  if (rc) return rc;
  return attend_impl(q, kv, idx, cnt, out, B, L, base + pl.off_attend, attend_ws(B), status, st, bf16, pg);
}

extern "C" int vmk_dsa_decode(const void* q, const void* kv, const void* iq, const void* ik, const float* w,
                              const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out, int B, int L,
                              void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  return decode_impl(q, kv, iq, ik, w, lens, out, idx_out, cnt_out, B, L, ws, ws_bytes, status, stream, 0);
}

// ---- the same op on bf16 tensors (q, kv, iq, ik and out; w stays fp32) ---------------------------------------
extern "C" int vmk_dsa_decode_bf16(const void* q, const void* kv, const void* iq, const void* ik, const float* w,
                                   const int32_t* lens, void* out, int32_t* idx_out, int32_t* cnt_out, int B, int L,
                                   void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  return decode_impl(q, kv, iq, ik, w, lens, out, idx_out, cnt_out, B, L, ws, ws_bytes, status, stream, 1);
}

extern "C" int vmk_dsa_indexer_hist_bf16(const void* iq, const void* ik, const float* w, const int32_t* lens,
                                         float* scores, uint32_t* hist, int B, int L, int32_t* status, void* stream) {
  if (!hist) return VMK_E_BADARG;
  const int bad = indexer_check(iq, ik, w, scores, B, L, 1, 1, DsaPages{nullptr, 0, 0, 0});
  if (bad) return bad;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(hist, 0, (size_t)B * kSelBins * 4, st) != cudaSuccess) return VMK_E_LAUNCH;
  return indexer_impl(iq, ik, w, lens, scores, hist, B, L, status, st, 1, 1);
}

extern "C" int vmk_dsa_attend_bf16(const void* q, const void* kv, const int32_t* idx, const int32_t* cnt, void* out,
                                   int B, int L, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  return attend_impl(q, kv, idx, cnt, out, B, L, ws, ws_bytes, status, static_cast<cudaStream_t>(stream), 1);
}

// ---- the op over a paged cache (index keys and latent rows paged alike) ----------------------------------------
extern "C" int vmk_dsa_decode_paged(const void* q, const void* kv_pages, const void* iq, const void* ik_pages,
                                    const float* w, const int32_t* page_table, int pages, int page_size,
                                    int table_stride, const int32_t* lens, void* out, int32_t* idx_out,
                                    int32_t* cnt_out, int B, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status,
                                    void* stream) {
  if (pages <= 0 || !page_table || !lens || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  if (L <= kTopK) return VMK_E_UNSUPPORTED;          // a cache this short is not worth paging: use vmk_dsa_decode
  return decode_impl(q, kv_pages, iq, ik_pages, w, lens, out, idx_out, cnt_out, B, L, ws, ws_bytes, status, stream, bf16,
                     DsaPages{page_table, pages, page_size, table_stride});
}

// ---- stage 1 with the index queries and keys in fp8 (e4m3) ------------------------------------------------------
extern "C" int vmk_dsa_indexer_hist_fp8(const void* iq8, const float* iq_scale, const void* ik8, const float* ik_scale,
                                        const float* w, const int32_t* lens, float* scores, uint32_t* hist, int B, int L,
                                        int32_t* status, void* stream) {
  if (!iq8 || !iq_scale || !ik8 || !ik_scale || !w || !scores || !hist || B <= 0 || L <= 0 || B > 65535)
    return VMK_E_BADARG;
  if (!aligned16(iq8) || !aligned16(ik8)) return VMK_E_BADARG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (cudaMemsetAsync(hist, 0, (size_t)B * kSelBins * 4, st) != cudaSuccess) return VMK_E_LAUNCH;
  if (L <= kTopK) return VMK_OK;                        // nothing to rank
  CUtensorMap tmIK, tmIQ;
  int rc = make_tmap_3d_u8(&tmIK, ik8, L, B, kIdxTile);
  if (rc) return rc;
  rc = make_tmap_3d_u8(&tmIQ, iq8, kHI, B, kHI);
  if (rc) return rc;
  return indexer_tc_launch(tmIK, tmIQ, w, lens, scores, hist, B, L, status, st, 0, nullptr, 0, 0, 0, iq_scale, ik_scale);
}
