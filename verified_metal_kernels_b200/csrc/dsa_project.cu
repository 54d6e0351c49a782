// The step before `dsa` stage 1: the projection that produces the indexer's queries and head weights from the
// token's activation, which the reference leaves outside its op (ops/dsa.py:8-9: "the projections that produce
// q / iq / w are not part of the op").
//
//     iq[b, h, d] = round16( sum_k x[b, k] * Wq[h * 128 + d, k] )          (B, 64, 128), fp16 or bf16
//     w[b, h]     = w_scale * sum_k x[b, k] * Ww[h, k]                      (B, 64), fp32
//
// One GEMM, C[m = request][n = output feature] = X[m][:] . W[n][:], with both operands K-major exactly as they are
// stored (activations (B, Dx), weights (out, in) as a linear layer keeps them), so TMA brings them in unchanged.
// The 8192 + 64 output features are cut into 129 tiles of 64; a CTA owns one feature tile and one tile of 128
// requests (rows beyond B are filled with zeros by TMA) and runs over Dx in blocks of 64 through a 4-slot ring:
//   warp 0     TMA producer: X block (128 x 64, 16 KiB) and W block (64 x 64, 8 KiB) per slot
//   warp 1     owns 64 columns of tensor memory and issues 4 x tcgen05.mma (M128 N64 K16) per block
//   warps 2-5  epilogue: one thread per request reads its 64 fp32 sums and stores them (16-bit iq, or fp32 w)
// The weights (25 MB at Dx = 1536) are read once per tile of 128 requests, each CTA streaming its own 64 rows:
// the kernel is bound by that stream.  It is a launch of its own rather than a prologue of the indexer because
// every indexer CTA would have to stream the whole weight matrix to rebuild its request's 64 x 128 queries.
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA winds down through the
// common exit, where tensor memory is freed.
#include "tcgen05.cuh"

namespace vmk {

constexpr int kPjHeads = 64, kPjWidth = 128;
constexpr int kPjFeatures = kPjHeads * kPjWidth;       // 8192 query features, then 64 weight features
constexpr int kPjTileN = 64;
constexpr int kPjTileM = 128;
constexpr int kPjBK = 64;
constexpr int kPjStages = 4;
constexpr int kPjABytes = kPjTileM * kPjBK * 2;        // 16 KiB
constexpr int kPjBBytes = kPjTileN * kPjBK * 2;        // 8 KiB
constexpr int kPjSlot = kPjABytes + kPjBBytes;
constexpr int kPjThreads = 192;
constexpr int kPjSmem = kPjStages * kPjSlot + (2 * kPjStages + 1) * 8 + 16 + 1024;

struct ProjectParams {
  CUtensorMap tmX;       // (1, B, Dx) box (64, 128, 1)
  CUtensorMap tmWq;      // (1, 8192, Dx) box (64, 64, 1)
  CUtensorMap tmWw;      // (1, 64, Dx) box (64, 64, 1)
  __half* iq;            // (B, 64, 128)
  float* w;              // (B, 64)
  float w_scale;
  int B, Dx, bf16;
  int32_t* status;
};

__global__ void __launch_bounds__(kPjThreads, 1) index_project_kernel(const __grid_constant__ ProjectParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + kPjStages * kPjSlot);
  uint64_t* empty = full + kPjStages;
  uint64_t* acc_full = empty + kPjStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_full + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int nt = blockIdx.x;                                // feature tile: 0..127 queries, 128 the head weights
  const int m0 = blockIdx.y * kPjTileM;                     // first request of the tile
  const bool weights = nt == kPjFeatures / kPjTileN;
  const int nk = (p.Dx + kPjBK - 1) / kPjBK;

  if (tid == 0) {
    for (int s = 0; s < kPjStages; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    mbar_init(acc_full, 1);
    fence_mbar_init();
    tma_prefetch_desc(&p.tmX);
    tma_prefetch_desc(weights ? &p.tmWw : &p.tmWq);
  }
  if (warp == 1) tmem_alloc(tmem_slot, kPjTileN);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  pdl_wait();                                               // the activation may come from the kernel before this one

  bool timed_out = false;
  if (warp == 0) {
    if (lane == 0) {
      const CUtensorMap* tmW = weights ? &p.tmWw : &p.tmWq;
      const int wrow = weights ? 0 : nt * kPjTileN;
      int issued = 0;
      for (int j = 0; j < nk; ++j) {
        const int s = j % kPjStages;
        if (j >= kPjStages && !mbar_wait(&empty[s], (uint32_t)(((j / kPjStages) - 1) & 1))) {
          timed_out = true;
          break;
        }
        uint8_t* st = smem + s * kPjSlot;
        mbar_expect_tx(&full[s], kPjSlot);
        tma_load_3d(st, &p.tmX, j * kPjBK, m0, 0, &full[s]);
        tma_load_3d(st + kPjABytes, tmW, j * kPjBK, wrow, 0, &full[s]);
        issued = j + 1;
      }
      // no load outlives the CTA (returns at once unless a consumer gave up before it had waited for them)
      for (int j = max(0, issued - kPjStages); j < issued; ++j)
        mbar_wait(&full[j % kPjStages], (uint32_t)((j / kPjStages) & 1));
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_16(kPjTileM, kPjTileN, 0, p.bf16);
      for (int j = 0; j < nk; ++j) {
        const int s = j % kPjStages;
        if (!mbar_wait(&full[s], (uint32_t)((j / kPjStages) & 1))) {
          timed_out = true;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * kPjSlot), b_addr = a_addr + kPjABytes;
#pragma unroll
        for (int k = 0; k < kPjBK / 16; ++k)                  // K step k: 32 bytes further inside the 128-byte swizzled row
          umma_f16(tmem_base, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(b_addr + k * 32), idesc,
                   (j > 0 || k > 0) ? 1u : 0u);
        umma_commit(&empty[s]);
      }
      if (!timed_out) umma_commit(acc_full);
    }
  } else {
    // ---------------------------------------------------------------------------- epilogue (warps 2..5)
    const int quarter = warp & 3;                           // tensor-memory lanes [32 q, 32 q + 32)
    const int m = m0 + quarter * 32 + lane;
    const bool ok = mbar_wait(acc_full, 0);
    if (!__all_sync(0xffffffffu, ok)) {
      timed_out = true;
    } else {
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16);
      uint32_t r0[32], r1[32];
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32, r1);
      tmem_ld_wait();
      if (m < p.B) {
        if (weights) {
          float4* dst = reinterpret_cast<float4*>(p.w + (size_t)m * kPjHeads);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[i] = make_float4(__uint_as_float(r0[4 * i]) * p.w_scale, __uint_as_float(r0[4 * i + 1]) * p.w_scale,
                                 __uint_as_float(r0[4 * i + 2]) * p.w_scale, __uint_as_float(r0[4 * i + 3]) * p.w_scale);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            dst[8 + i] = make_float4(__uint_as_float(r1[4 * i]) * p.w_scale, __uint_as_float(r1[4 * i + 1]) * p.w_scale,
                                     __uint_as_float(r1[4 * i + 2]) * p.w_scale, __uint_as_float(r1[4 * i + 3]) * p.w_scale);
        } else {
          uint4* dst = reinterpret_cast<uint4*>(p.iq + (size_t)m * kPjFeatures + nt * kPjTileN);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2(__uint_as_float(r0[8 * i]), __uint_as_float(r0[8 * i + 1]), p.bf16);
            v.y = pack2(__uint_as_float(r0[8 * i + 2]), __uint_as_float(r0[8 * i + 3]), p.bf16);
            v.z = pack2(__uint_as_float(r0[8 * i + 4]), __uint_as_float(r0[8 * i + 5]), p.bf16);
            v.w = pack2(__uint_as_float(r0[8 * i + 6]), __uint_as_float(r0[8 * i + 7]), p.bf16);
            dst[i] = v;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            uint4 v;
            v.x = pack2(__uint_as_float(r1[8 * i]), __uint_as_float(r1[8 * i + 1]), p.bf16);
            v.y = pack2(__uint_as_float(r1[8 * i + 2]), __uint_as_float(r1[8 * i + 3]), p.bf16);
            v.z = pack2(__uint_as_float(r1[8 * i + 4]), __uint_as_float(r1[8 * i + 5]), p.bf16);
            v.w = pack2(__uint_as_float(r1[8 * i + 6]), __uint_as_float(r1[8 * i + 7]), p.bf16);
            dst[4 + i] = v;
          }
        }
      }
    }
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: every warp arrives here, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_free(tmem_base, kPjTileN);
  }
}

static bool pj_aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace vmk

using namespace vmk;

extern "C" int vmk_dsa_index_project(const void* x, const void* wq, const void* ww, float w_scale, void* iq_out,
                                     float* w_out, int B, int Dx, int bf16, int32_t* status, void* stream) {
  if (!x || !wq || !ww || !iq_out || !w_out || B <= 0 || Dx <= 0 || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  if (!pj_aligned16(x) || !pj_aligned16(wq) || !pj_aligned16(ww) || !pj_aligned16(iq_out) || !pj_aligned16(w_out))
    return VMK_E_BADARG;
  if (Dx % 8 != 0 || B > 65535 * kPjTileM) return VMK_E_UNSUPPORTED;   // rows must start on 16-byte boundaries
  ProjectParams p;
  memset(&p, 0, sizeof(p));
  int rc = make_tmap_3d(&p.tmX, x, (uint64_t)Dx, (uint64_t)B, 1, kPjBK, kPjTileM);
  if (rc) return rc;
  rc = make_tmap_3d(&p.tmWq, wq, (uint64_t)Dx, kPjFeatures, 1, kPjBK, kPjTileN);
  if (rc) return rc;
  rc = make_tmap_3d(&p.tmWw, ww, (uint64_t)Dx, kPjHeads, 1, kPjBK, kPjTileN);
  if (rc) return rc;
  p.iq = static_cast<__half*>(iq_out);
  p.w = w_out;
  p.w_scale = w_scale;
  p.B = B; p.Dx = Dx; p.bf16 = bf16;
  p.status = status;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(index_project_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPjSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(kPjFeatures / kPjTileN + 1, (B + kPjTileM - 1) / kPjTileM);
  cfg.blockDim = dim3(kPjThreads);
  cfg.dynamicSmemBytes = kPjSmem;
  cfg.stream = static_cast<cudaStream_t>(stream);
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_launch(cudaLaunchKernelEx(&cfg, index_project_kernel, p));
}
