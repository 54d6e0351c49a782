// Split-KV decode attention on the 5th-generation tensor cores, for row tiles of 128 stacked rows
// (many requests sharing a prefix, or a wide speculative tree): the regime where the op is bound by
// the tensor pipe rather than by HBM.
//
// One CTA = one (key group, 128-row tile, key split), 192 threads, warp-specialised:
//   warp 0      TMA producer: K and V tiles of 128 keys x 128 (two 64-wide swizzled boxes each) into a
//               two-stage ring
//   warp 1      owns tensor memory (512 columns) and issues the MMAs:
//                 S[j & 1] (128 x 128 fp32) = Q . K_j^T            8 x tcgen05.mma M128 N128 K16, K-major
//                 O        (128 x 128 fp32) += P_j . V_j           8 x tcgen05.mma, V as an MN-major operand
//               S is double buffered so Q.K^T of block j+1 runs under the softmax of block j
//   warps 2-5   softmax, one thread per row: tcgen05.ld of the 128 scores, scale + visibility mask,
//               running max with LAZY rescaling (O in tensor memory is rescaled only when the max grew
//               by more than 2^8, so P stays below 256 and exact), P rounded to fp16 into a swizzled
//               shared-memory tile that the second MMA reads, row sums in fp32
// Partials (m, l, o) per row are emitted exactly as by the warp-level kernel, so the combine pass and
// the multi-GPU merge are shared.  Every mbarrier wait is bounded.
#include "attn_core.cuh"
#include "tcgen05.cuh"

namespace vmk {

constexpr int kTcBK = 128;                       // keys per block
constexpr int kTcHalf = 128 * 128;               // one swizzled [128 rows][128 B] box
constexpr int kTcTile = 2 * kTcHalf;             // 32 KiB: a 128 x 128 fp16 operand tile
constexpr int kTcKvStages = 2;
constexpr int kTcThreads = 192;
constexpr int kTcCols = 512;                     // S0 | S1 | O | (unused)
constexpr float kLazyRescale = 8.f;              // log2 units
constexpr int kTcBars = 2 * kTcKvStages + 2 + 2 + 3;
constexpr int kAttnTcSmem = kTcTile * (1 + 2 * kTcKvStages + 1) + kTcBars * 8 + 16 + 1024;

__global__ void __launch_bounds__(kTcThreads, 1) attn_tc_kernel(const __grid_constant__ AttnParams p) {
  const AttnRole& R = p.a;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + kTcTile;
  uint8_t* sV = sK + kTcKvStages * kTcTile;
  uint8_t* sP = sV + kTcKvStages * kTcTile;
  uint64_t* kv_full = reinterpret_cast<uint64_t*>(sP + kTcTile);
  uint64_t* kv_empty = kv_full + kTcKvStages;
  uint64_t* s_full = kv_empty + kTcKvStages;
  uint64_t* s_empty = s_full + 2;
  uint64_t* p_full = s_empty + 2;
  uint64_t* pv_done = p_full + 1;
  uint64_t* q_full = pv_done + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_full + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  // ---- which piece of work (same decomposition as the warp-level kernel, 128-key blocks) -------------
  const int cta = blockIdx.x;
  const int split = cta % R.nsplit;
  const int t2 = cta / R.nsplit;
  const int tile = t2 % R.row_tiles;
  const int z = t2 / R.row_tiles;
  const int zg = z / R.Hkv, h = z % R.Hkv;
  const int rows = R.rows_outer * R.G;
  const int row0 = tile * 128;
  const int kbeg = R.key_lo + split * R.split_len;
  int kend = min(kbeg + R.split_len, R.key_hi);
  if (R.klens != nullptr) kend = min(kend, max(0, min(R.klens[zg], R.klen)));
  const int nblk = kend > kbeg ? (kend - kbeg + kTcBK - 1) / kTcBK : 0;

  if (tid == 0) {
    for (int s = 0; s < kTcKvStages; ++s) {
      mbar_init(&kv_full[s], 1);
      mbar_init(&kv_empty[s], 1);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(&s_full[s], 1);
      mbar_init(&s_empty[s], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    mbar_init(q_full, 4);
    fence_mbar_init();
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTcCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + 256;

  bool timed_out = false;
  if (warp == 0) {
    // ------------------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int j = 0; j < nblk; ++j) {
        const int s = j % kTcKvStages;
        if (j >= kTcKvStages && !mbar_wait(&kv_empty[s], (uint32_t)(((j / kTcKvStages) - 1) & 1))) {
          timed_out = true;
          break;
        }
        const int kb = kbeg + j * kTcBK;
        uint8_t* k = sK + s * kTcTile;
        uint8_t* v = sV + s * kTcTile;
        mbar_expect_tx(&kv_full[s], 2 * kTcTile);
        tma_load_3d(k, &R.tmK, 0, kb, z, &kv_full[s]);
        tma_load_3d(k + kTcHalf, &R.tmK, 64, kb, z, &kv_full[s]);
        tma_load_3d(v, &R.tmV, 0, kb, z, &kv_full[s]);
        tma_load_3d(v + kTcHalf, &R.tmV, 64, kb, z, &kv_full[s]);
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------ MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16(128, 128, 0);
      constexpr uint32_t idesc_pv = umma_idesc_f16(128, 128, 1);
      const uint32_t q_addr = smem_u32(sQ), p_addr = smem_u32(sP);
      auto issue_qk = [&](int j) {
        const int s = j & 1;
        const uint32_t k_addr = smem_u32(sK + (j % kTcKvStages) * kTcTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          const uint32_t off = (k >> 2) * kTcHalf + (k & 3) * 32;
          umma_f16(tmem_base + s * 128, umma_desc_sw128(q_addr + off), umma_desc_sw128(k_addr + off), idesc_qk,
                   k > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[s]);
      };
      if (!mbar_wait(q_full, 0) || !mbar_wait(&kv_full[0], 0)) timed_out = true;
      if (!timed_out) {
        tc_fence_after();
        issue_qk(0);
      }
      for (int j = 0; j < nblk && !timed_out; ++j) {
        if (j + 1 < nblk) {
          const int j1 = j + 1, s1 = j1 & 1;
          if (!mbar_wait(&kv_full[j1 % kTcKvStages], (uint32_t)((j1 / kTcKvStages) & 1))) { timed_out = true; break; }
          if (j1 >= 2 && !mbar_wait(&s_empty[s1], (uint32_t)(((j1 >> 1) - 1) & 1))) { timed_out = true; break; }
          tc_fence_after();
          issue_qk(j1);
        }
        if (!mbar_wait(p_full, (uint32_t)(j & 1))) { timed_out = true; break; }
        tc_fence_after();
        const uint32_t v_addr = smem_u32(sV + (j % kTcKvStages) * kTcTile);
#pragma unroll
        for (int k = 0; k < 8; ++k) {
          // A: P[:, 16k .. 16k+16) K-major; B: V rows 16k .. 16k+16 (keys) x 128 d, MN-major:
          // 8-key groups 1024 B apart, the two 64-wide d halves kTcHalf apart.
          const uint64_t da = umma_desc_sw128(p_addr + (k >> 2) * kTcHalf + (k & 3) * 32);
          const uint64_t db = umma_desc_sw128_mn(v_addr + k * 2048, kTcHalf, 1024);
          umma_f16(tO, da, db, idesc_pv, (j > 0 || k > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[j % kTcKvStages]);
        umma_commit(pv_done);
      }
    }
  } else {
    // ------------------------------------------------------------------------------ softmax warps
    const int quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int grow = row0 + row;
    const bool valid_row = grow < rows;
    const uint32_t lane_base = tmem_base + ((uint32_t)(quarter * 32) << 16);
    const size_t outer = (size_t)zg * R.rows_outer + (valid_row ? grow / R.G : 0);
    const int head = h * R.G + (valid_row ? grow % R.G : 0);

    // this thread's query row -> swizzled K-major operand tile
    {
      const uint4* src = reinterpret_cast<const uint4*>(R.q + (outer * R.Hq + head) * kHD);
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const uint4 v = valid_row ? src[c] : make_uint4(0u, 0u, 0u, 0u);
        *reinterpret_cast<uint4*>(sQ + (c >> 3) * kTcHalf + swz128(row, c & 7)) = v;
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(q_full);
    }
    uint32_t mw[kMaxMaskWords];
#pragma unroll
    for (int w = 0; w < kMaxMaskWords; ++w) {
      mw[w] = 0xffffffffu;
      if (R.bits != nullptr && valid_row && w < R.bits_words) mw[w] = R.bits[outer * R.bits_words + w];
    }

    float m = -INFINITY, l = 0.f;
    for (int j = 0; j < nblk; ++j) {
      const int sb = j & 1;
      bool ok = mbar_wait(&s_full[sb], (uint32_t)((j >> 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
      tc_fence_after();
      uint32_t sr[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(lane_base + sb * 128 + c * 32, sr[c]);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);

      const int kb = kbeg + j * kTcBK;
      const bool tail = kb + kTcBK > kend;
      const bool edge = tail || (kb + kTcBK > R.mask_start);
      float bm = -INFINITY;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float t = __uint_as_float(sr[c][i]) * p.sc;
          if (edge) {
            const int key = kb + c * 32 + i;
            bool vis = key < kend;
            if (vis && key >= R.mask_start) {
              const int jb = key - R.mask_start;
              uint32_t word = mw[0];
#pragma unroll
              for (int w = 1; w < kMaxMaskWords; ++w) word = ((jb >> 5) == w) ? mw[w] : word;
              vis = (word >> (jb & 31)) & 1u;
            }
            t = vis ? t : -INFINITY;
          }
          sr[c][i] = __float_as_uint(t);
          bm = fmaxf(bm, t);
        }
      }
      const float m_new = fmaxf(m, bm);
      float alpha = 1.f;
      bool rescale = false;
      if (m == -INFINITY) {
        m = m_new;                                   // nothing accumulated for this row yet
      } else if (m_new > m + kLazyRescale) {
        alpha = exp2f(m - m_new);
        m = m_new;
        rescale = true;
      }
      l *= alpha;
      const float mu = (m == -INFINITY) ? 0.f : m;
      float ps = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          const float pv = exp2f(__uint_as_float(sr[c][i]) - mu);
          ps += pv;
          sr[c][i] = __float_as_uint(pv);
        }
      }
      l += ps;

      // O and the P tile are free once P_{j-1} . V_{j-1} has completed
      if (j >= 1) {
        ok = mbar_wait(pv_done, (uint32_t)((j - 1) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        tc_fence_after();
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t o[32];
          tmem_ld32(lane_base + 256 + c * 32, o);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
          tmem_st32(lane_base + 256 + c * 32, o);
        }
        tmem_st_wait();
      }
      if (tail && kend < R.klen) {
        // keys past kend exist in memory: their V rows must not reach the MMA (0 * Inf would poison the row)
        ok = mbar_wait(&kv_full[j % kTcKvStages], (uint32_t)((j / kTcKvStages) & 1));
        if (!__all_sync(0xffffffffu, ok)) { timed_out = true; break; }
        uint8_t* v = sV + (j % kTcKvStages) * kTcTile;
        const int r0 = kend - kb;
        for (int i = row; i < (kTcBK - r0) * 16; i += 128) {
          const int r = r0 + (i >> 4), c = i & 15;
          *reinterpret_cast<uint4*>(v + (c >> 3) * kTcHalf + swz128(r, c & 7)) = make_uint4(0u, 0u, 0u, 0u);
        }
      }
      // P (fp16) -> swizzled K-major operand tile
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        uint4 v;
        const uint32_t* s8 = &sr[c >> 2][(c & 3) * 8];
        v.x = pack_half2(__uint_as_float(s8[0]), __uint_as_float(s8[1]));
        v.y = pack_half2(__uint_as_float(s8[2]), __uint_as_float(s8[3]));
        v.z = pack_half2(__uint_as_float(s8[4]), __uint_as_float(s8[5]));
        v.w = pack_half2(__uint_as_float(s8[6]), __uint_as_float(s8[7]));
        *reinterpret_cast<uint4*>(sP + (c >> 3) * kTcHalf + swz128(row, c & 7)) = v;
      }
      fence_proxy_async();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }

    // ---- emit this row's partial (or final) result ------------------------------------------------
    bool have_o = false;
    if (!timed_out && nblk > 0) {
      const bool ok = mbar_wait(pv_done, (uint32_t)((nblk - 1) & 1));
      if (!__all_sync(0xffffffffu, ok)) timed_out = true; else have_o = true;
      tc_fence_after();
    }
    if (!timed_out) {
      const size_t slot = (size_t)z * R.nsplit + split;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t o[32];
        if (have_o) {
          tmem_ld32(lane_base + 256 + c * 32, o);
          tmem_ld_wait();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) o[i] = 0u;
        }
        if (!valid_row) continue;
        if (R.direct) {
          __half* dst = R.out + (outer * R.Hq + head) * kHD + c * 32;
          const float inv = 1.f / l;
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
