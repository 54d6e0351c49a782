// `dsa` stage 3 on the 5th-generation tensor cores: absorbed-MLA attention over the selected rows.
//
// The shapes fight the machine: 128 heads x 512 fp32 of output is all of tensor memory, and a 128 x 576
// fp16 query tile is 147 KB of shared memory.  This kernel therefore
//   * keeps Q in TENSOR MEMORY (288 columns of packed fp16 pairs) and feeds it to the MMA as the A operand
//     straight from there, so shared memory only holds the gathered rows;
//   * gives each CTA all 128 heads but only HALF of the value columns (grid.y = 2), and accumulates that
//     half of the output in REGISTERS: every 64-key block the product P.V is written to a 128-column
//     scratch area of tensor memory, read back and added, first for value columns [0,128) of the half by
//     softmax group A, then for [128,256) by group B.
// One CTA = (key split, value half, request), 384 threads:
//   warps 0-3   softmax group A, warps 4-7 group B: one thread per head and group.  Both groups read the
//               64 scores of their head from tensor memory (two passes: row max, then exp2 and row sum);
//               group A also stores P (packed fp16) to tensor memory, the A operand of P.V
//   warps 8-10  gather the selected 576-wide rows by index (cp.async, 8 lanes per row, three of the nine
//               128-byte column blocks per warp) into a three-stage
//               ring laid out as nine [64 keys][128 B] blocks with the 128-byte swizzle, i.e. the K-major
//               operand of Q.K^T and, for its first eight blocks, the MN-major operand of P.V
//   warp 11     owns tensor memory and issues the MMAs: 36 x (M128 N64 K16, A from tensor memory) for
//               S = Q.K^T, then 4 + 4 x (M128 N128 K16, A = P from tensor memory) for the two parts of P.V
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA winds down
// through the common exit, where tensor memory is freed.
#include "tcgen05.cuh"

namespace vmk {

constexpr int kMlaTopK = VMK_DSA_TOPK;
constexpr int kMH = 128, kDK = 576, kDV = 512;
constexpr int kBK = 64;                               // keys per block
constexpr int kBlkBytes = kBK * 128;                  // one [64 keys][128 B] swizzled block
constexpr int kKTile = 9 * kBlkBytes;                 // 72 KiB: 64 gathered rows of 576 fp16
constexpr int kMlaStages = 3;
constexpr int kMlaThreads = 384;
constexpr int kMlaProducers = 2;                      // gather warps: they take alternate blocks
constexpr int kColQ = 0;                              // 288 columns: Q as packed fp16 pairs
constexpr int kColS = 288;                            // 64 columns: scores
constexpr int kColT = 352;                            // 128 columns: P.V scratch
constexpr int kColP = 480;                            // 32 columns: P as packed fp16 pairs
constexpr int kMlaCols = 512;
constexpr int kMlaBars = 3 * kMlaStages + 12;
constexpr int kMlaTcSmem = kMlaStages * kKTile + kMlaBars * 8 + 16 + 6 * 128 * 4 + 1024;

struct MlaTcParams {
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

#ifdef VMK_MLA_TIMING
// Debug build only.  Time stamps of blocks 8..15 of CTA (0,0,0): [role][block - 8][event]
__device__ long long g_mla_trace[4 * 8 * 16];
#define MLA_E(role, j, ev) do { if (blockIdx.x + blockIdx.y + blockIdx.z == 0 && (j) >= 8 && (j) < 16 && lane == 0) \
    g_mla_trace[((role) * 8 + (j) - 8) * 16 + (ev)] = clock64(); } while (0)
#else
#define MLA_E(role, j, ev) do {} while (0)
#endif

// D[tmem] (+)= A[tmem] * B[smem descriptor]
__device__ __forceinline__ void umma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint32_t b_lo, uint32_t b_hi, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      ".reg .b64 db;\n"
      "setp.ne.b32 p, %5, 0;\n"
      "mov.b64 db, {%2, %3};\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, p;\n"
      "}\n" ::"r"(tmem_d), "r"(tmem_a), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
      : "memory");
}

__device__ __forceinline__ float ex2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

__global__ void __launch_bounds__(kMlaThreads, 1) mla_tc_kernel(const MlaTcParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;                                   // [stages][9 blocks][64 keys][128 B]
  uint64_t* full = reinterpret_cast<uint64_t*>(sK + kMlaStages * kKTile);   // gathered tile landed (32 producer lanes)
  uint64_t* empty = full + kMlaStages;                  // tile consumed by Q.K^T and P.V       (MMA commit)
  uint64_t* empty_k = empty + kMlaStages;               // tile consumed by Q.K^T               (MMA commit)
  uint64_t* q_full = empty_k + kMlaStages;                // Q stored to tensor memory            (4 warps)
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
  float* ssum = smax + 4 * 128;                             // [2 groups][128 heads] row sums

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int split = blockIdx.x, half = blockIdx.y, b = blockIdx.z;
  const int nb = max(0, min(p.cnt[b], kMlaTopK));
  const int k0 = split * p.split_len;
  const int k1 = min(nb, k0 + p.split_len);
  const int nblk = k1 > k0 ? (k1 - k0 + kBK - 1) / kBK : 0;

  if (tid == 0) {
    for (int s = 0; s < kMlaStages; ++s) {
      mbar_init(&full[s], 32);
      mbar_init(&empty[s], 1);
      mbar_init(&empty_k[s], 1);
    }
    mbar_init(q_full, 4);
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
  if (warp == 11) tmem_alloc(tmem_slot, kMlaCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool timed_out = false;
  if (warp >= 8 && warp < 8 + kMlaProducers) {
    // ------------------------------------------------------------------------------ gather producers
    // The two warps take alternate blocks (64 rows x 1152 B each) and publish each as soon as it has landed, so
    // two blocks are in flight and neither warp's wait holds up the other's copies.
    const __half* kvb = p.kv + (size_t)b * p.L * kDK;
    const int32_t* idxb = p.idx + (size_t)b * kMlaTopK;
    const int rsub = lane >> 3, c8 = lane & 7;          // 4 rows per instruction, 8 lanes (128 B) per row
    for (int j = warp - 8; j < nblk; j += kMlaProducers) {
      const int s = j % kMlaStages;
      uint8_t* st = sK + s * kKTile;
      // this lane's two candidate row indices of the block (rows lane and lane + 32), requested early so that
      // their latency hides behind the wait below
      const int ka = k0 + j * kBK + lane, kb2 = ka + 32;
      int ia = ka < k1 ? idxb[ka] : -1, ib = kb2 < k1 ? idxb[kb2] : -1;
      if (ia >= p.L || ib >= p.L) {
        report(p.status, kStatusBadIndex);
        ia = ia >= p.L ? 0 : ia;
        ib = ib >= p.L ? 0 : ib;
      }
      // Two passes over the rows.  Pass 0 copies the five column blocks only Q.K^T reads (the other CTA's value
      // half and the rope block): their part of the slot is free as soon as Q.K^T of block j - 3 is done, one
      // block earlier than the four value blocks of pass 1, which P.V of block j - 3 still reads.
#pragma unroll 1
      for (int pass = 0; pass < 2; ++pass) {
        if (j >= kMlaStages) {
          const bool ok = mbar_wait(pass == 0 ? &empty_k[s] : &empty[s], (uint32_t)(((j / kMlaStages) - 1) & 1));
          if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        }
        MLA_E(1, j, pass * 2);
        const int own = half * 4, other = 4 - own;
#pragma unroll 4
        for (int g = 0; g < 16; ++g) {
          const int row = g * 4 + rsub;
          const int ridx = (g < 8) ? __shfl_sync(0xffffffffu, ia, row & 31) : __shfl_sync(0xffffffffu, ib, row & 31);
          const bool valid = ridx >= 0;
          const uint8_t* src = reinterpret_cast<const uint8_t*>(kvb + (size_t)(valid ? ridx : 0) * kDK) + c8 * 16;
          uint8_t* dst = st + row * 128 + ((c8 ^ (row & 7)) << 4);
          const int first = pass == 0 ? other : own;
#pragma unroll
          for (int blk = 0; blk < 4; ++blk)
            cp_async16(dst + (first + blk) * kBlkBytes, src + (first + blk) * 128, valid ? 16 : 0);
          if (pass == 0) cp_async16(dst + 8 * kBlkBytes, src + 8 * 128, valid ? 16 : 0);
        }
        MLA_E(1, j, pass * 2 + 1);
      }
      if (timed_out) break;
      cp_async_commit();
      cp_async_wait<0>();
      MLA_E(1, j, 4);
      fence_proxy_async();
      mbar_arrive(&full[s]);
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------------------------ Q.K^T issuer
    // The tensor pipe buffers only an instruction or two, so every wait of an issuing thread drains it.  Two
    // issuers (this warp for S_j = Q . K_j^T, the next for P_j . V_j) keep it fed: while one waits for a
    // hand-over, the other's instructions run.
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, kBK, 0);
      const uint32_t hi_k = (uint32_t)(umma_desc_sw128(0) >> 32);
      const uint32_t k_lo = (uint32_t)umma_desc_sw128(0) + (smem_u32(sK) >> 4);
      const uint32_t tQ = tmem_base + kColQ, tS = tmem_base + kColS;
      if (!mbar_wait(q_full, 0)) timed_out = true;
      for (int j = 0; j < nblk && !timed_out; ++j) {
        if (!mbar_wait(&full[j % kMlaStages], (uint32_t)((j / kMlaStages) & 1))) { timed_out = true; break; }
        MLA_E(0, j, 0);
        if (j >= 1 && !mbar_wait(s_free, (uint32_t)((j - 1) & 1))) { timed_out = true; break; }
        MLA_E(0, j, 1);
        tc_fence_after();
        const uint32_t kb_lo = k_lo + (j % kMlaStages) * (kKTile >> 4);
#pragma unroll 12
        for (int kk = 0; kk < 36; ++kk)
          umma_f16_ts(tS, tQ + kk * 8, kb_lo + (kk >> 2) * (kBlkBytes >> 4) + (kk & 3) * 2, hi_k, idesc_qk,
                      kk > 0 ? 1u : 0u);
        umma_commit(s_full);
        umma_commit(&empty_k[j % kMlaStages]);
        MLA_E(0, j, 2);
      }
    }
  } else if (warp == 11) {
    // ------------------------------------------------------------------------------ P.V issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, 128, 1);
      const uint32_t hi_v = (uint32_t)(umma_desc_sw128_mn(0, kBlkBytes, 1024) >> 32);
      const uint32_t v_lo = (uint32_t)umma_desc_sw128_mn(0, kBlkBytes, 1024) + (smem_u32(sK) >> 4);
      const uint32_t tT = tmem_base + kColT, tP = tmem_base + kColP;
      // One 128-column part of P_i . V_i into the scratch.
      auto issue_pv_part = [&](int i, int part) {
        const uint32_t vb = v_lo + (i % kMlaStages) * (kKTile >> 4) + (half * 4 + part * 2) * (kBlkBytes >> 4);
#pragma unroll
        for (int k = 0; k < 4; ++k) umma_f16_ts(tT, tP + k * 8, vb + k * (2048 >> 4), hi_v, idesc_pv, k > 0 ? 1u : 0u);
      };
      for (int j = 0; j < nblk; ++j) {
        if (!mbar_wait(p_full, (uint32_t)(j & 1))) { timed_out = true; break; }
        MLA_E(0, j, 3);
        if (j >= 1 && !mbar_wait(tb_free, (uint32_t)((j - 1) & 1))) { timed_out = true; break; }
        MLA_E(0, j, 4);
        tc_fence_after();
        issue_pv_part(j, 0);
        umma_commit(pva_done);
        MLA_E(0, j, 5);
        if (!mbar_wait(ta_free, (uint32_t)(j & 1))) { timed_out = true; break; }
        MLA_E(0, j, 7);
        tc_fence_after();
        issue_pv_part(j, 1);
        umma_commit(pvb_done);
        umma_commit(&empty[j % kMlaStages]);
        MLA_E(0, j, 8);
      }
    }
  } else if (warp < 8) {
    // ------------------------------------------------------------------------------ softmax groups
    // Group A owns keys [0,32) of every block and value columns [0,128) of this CTA's half; group B keys
    // [32,64) and value columns [128,256).  The two threads of a head exchange their block maxima through
    // shared memory, so both follow the same running maximum.
    const int grp = warp >> 2;
    const int quarter = warp & 3;
    const int head = quarter * 32 + lane;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const uint32_t tS = lane_base + kColS + grp * 32, tT = lane_base + kColT, tPw = lane_base + kColP + grp * 16;
    uint64_t* my_done = grp == 0 ? pva_done : pvb_done;
    uint64_t* my_free = grp == 0 ? ta_free : tb_free;

    if (grp == 0) {
      // this head's query row -> tensor memory, two fp16 per 32-bit column
      const uint4* src = reinterpret_cast<const uint4*>(p.q + ((size_t)b * kMH + head) * kDK);
#pragma unroll 1
      for (int c = 0; c < 18; ++c) {
        uint32_t r[16];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint4 v = src[c * 4 + i];
          r[4 * i] = v.x; r[4 * i + 1] = v.y; r[4 * i + 2] = v.z; r[4 * i + 3] = v.w;
        }
        tmem_st16(lane_base + kColQ + c * 16, r);
      }
      tmem_st_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }

    float m = -INFINITY, l = 0.f;
    float o[128];
#pragma unroll
    for (int i = 0; i < 128; ++i) o[i] = 0.f;

    // o = (o + scratch) * scale: adds this group's 128 value columns of P_i . V_i, then hands the scratch back
    auto accumulate = [&](int i, float scale) -> bool {
      const bool ok = mbar_wait(my_done, (uint32_t)(i & 1));
      if (!__all_sync(0xffffffffu, ok)) return false;
      if (quarter == 0) MLA_E(2 + grp, i, 5);
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
      if (quarter == 0) MLA_E(2 + grp, i, 6);
      return true;
    };

    for (int j = 0; j < nblk; ++j) {
      bool ok = mbar_wait(s_full, (uint32_t)(j & 1));
      if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      if (quarter == 0) MLA_E(2 + grp, j, 0);
      tc_fence_after();
      uint32_t s[32];
      tmem_ld32(tS, s);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(s_free);                  // the scores live in registers from here on
      if (quarter == 0) MLA_E(2 + grp, j, 1);
      const int kb = k0 + j * kBK + grp * 32;
      const bool tail = kb + 32 > k1;
      float bm = -INFINITY;
#pragma unroll
      for (int e = 0; e < 32; ++e) {
        float t = __uint_as_float(s[e]) * p.sc;
        if (tail && kb + e >= k1) t = -INFINITY;
        s[e] = __float_as_uint(t);
        bm = fmaxf(bm, t);
      }
      smax[((j & 1) * 2 + grp) * 128 + head] = bm;
      __syncwarp();
      if (lane == 0) mbar_arrive(&xch[quarter]);
      ok = mbar_wait(&xch[quarter], (uint32_t)(j & 1));
      if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      if (quarter == 0) MLA_E(2 + grp, j, 2);
      bm = fmaxf(bm, smax[((j & 1) * 2 + (grp ^ 1)) * 128 + head]);
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
      if (j >= 1) {                                        // P is free once both parts of P_{j-1} . V_{j-1} are done
        ok = mbar_wait(pvb_done, (uint32_t)((j - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      }
      if (quarter == 0) MLA_E(2 + grp, j, 3);
      {
        uint32_t pk[16];
#pragma unroll
        for (int e = 0; e < 16; ++e) pk[e] = pack_half2(__uint_as_float(s[2 * e]), __uint_as_float(s[2 * e + 1]));
        tmem_st16(tPw, pk);
        tmem_st_wait();
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(p_full);
        if (quarter == 0) MLA_E(2 + grp, j, 4);
      }
      if (grp == 0) {
        // A: rescale now, then add part A of P_j . V_j as soon as it is there (the MMA warp needs the scratch back)
#pragma unroll
        for (int i = 0; i < 128; ++i) o[i] *= alpha;
        if (!accumulate(j, 1.f)) { timed_out = true; break; }
      } else {
        // B: part B of the PREVIOUS block is added here, after this block's P is on its way, and rescaled with it
        if (j >= 1) {
          if (!accumulate(j - 1, alpha)) { timed_out = true; break; }
        }
      }
    }
    if (!timed_out && nblk > 0 && grp == 1 && !accumulate(nblk - 1, 1.f)) timed_out = true;
    // row sums of the two key halves
    if (!timed_out) {
      ssum[grp * 128 + head] = l;
      __syncwarp();
      if (lane == 0) mbar_arrive(&xch[quarter]);
      const bool ok = mbar_wait(&xch[quarter], (uint32_t)(nblk & 1));
      if (!__all_sync(0xffffffffu, ok)) timed_out = true;
      l += ssum[(grp ^ 1) * 128 + head];
    }

    // ---- emit -------------------------------------------------------------------------------------------
    if (!timed_out) {
      const int dv0 = half * 256 + grp * 128;
      if (p.nsplit == 1) {
        const float inv = 1.f / l;
        __half* dst = p.out + ((size_t)b * kMH + head) * kDV + dv0;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          uint4 v;
          v.x = pack_half2(o[8 * i] * inv, o[8 * i + 1] * inv);
          v.y = pack_half2(o[8 * i + 2] * inv, o[8 * i + 3] * inv);
          v.z = pack_half2(o[8 * i + 4] * inv, o[8 * i + 5] * inv);
          v.w = pack_half2(o[8 * i + 6] * inv, o[8 * i + 7] * inv);
          reinterpret_cast<uint4*>(dst)[i] = v;
        }
      } else {
        const size_t row = ((size_t)b * p.nsplit + split) * kMH + head;
        float* dst = p.part_o + row * kDV + dv0;
#pragma unroll
        for (int i = 0; i < 32; ++i)
          reinterpret_cast<float4*>(dst)[i] = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
        if (half == 0 && grp == 0) {
          p.part_ml[row * 2] = m;
          p.part_ml[row * 2 + 1] = l;
        }
      }
    }
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: every warp arrives, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 11) {
    tc_fence_after();
    tmem_free(tmem_base, kMlaCols);
  }
}

#ifdef VMK_MLA_TIMING
extern "C" VMK_API int vmk_debug_mla_trace(long long* out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_mla_trace, sizeof(long long) * 512);
}
#endif

int mla_tc_launch(const MlaTcParams& p, cudaStream_t stream) {
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(mla_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMlaTcSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  mla_tc_kernel<<<dim3(p.nsplit, 2, p.B), kMlaThreads, kMlaTcSmem, stream>>>(p);
  return check_launch(cudaGetLastError());
}

}  // namespace vmk
