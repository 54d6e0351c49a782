// `dsa` stage 1 on the 5th-generation tensor cores: scores[b,l] = sum_h w[b,h] * relu(iq[b,h] . ik[b,l]).
//
// Per 128-position tile the product T = ik_tile (128 x 128, K-major) . iq^T (64 x 128, K-major) is one
// tcgen05 accumulator of 128 lanes x 64 fp32 columns in tensor memory.  A CTA owns a contiguous run of
// tiles of one request and is warp-specialised:
//   warp 0     TMA producer: 32 KiB ik tiles into a 6-deep shared-memory ring (128-byte swizzle)
//   warp 1     (and warp 10 for fp8 keys) allocates tensor memory, issues 8 tcgen05.mma (M128 N64 K16) per tile into one of four
//              accumulator buffers, commits the ring slot back to the producer and the accumulator
//              to the epilogue
//   warps 2-9  epilogue, two sets of four warps on alternate tiles: tcgen05.ld of their 32 lanes x 64 columns,
//              fp32 ReLU and head-weighted sum, one coalesced fp32 score per position
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA winds down
// through the common exit, where the allocating warp frees its tensor memory.
#include "tcgen05.cuh"

namespace vmk {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kHI = 64, kDI = 128;
constexpr int kTile = 128;
constexpr int kStages = 6;
constexpr int kAccs = 4;                               // accumulator buffers of 64 columns
constexpr int kTileBytes = kTile * kDI * 2;            // 32 KiB
constexpr int kIqBytes = kHI * kDI * 2;                // 16 KiB
constexpr int kTmemCols = kAccs * kHI;                 // 256
constexpr int kTcThreads = 352;
// ring | iq | w | histogram | barriers | tmem base
constexpr int kTcSmem =
    kStages * kTileBytes + kIqBytes + kHI * 4 + kSelBins * 4 + (2 * kStages + 2 * kAccs + 1) * 8 + 16 + 1024;

struct TcParams {
  CUtensorMap tmIK;      // (B, L, 128) box (64, 128, 1), 128-byte swizzle
  CUtensorMap tmIQ;      // (B, 64, 128) box (64, 64, 1)
  const float* w;
  const int32_t* lens;
  float* scores;
  uint32_t* hist;        // (B, 2048) counts of the top 11 key bits, accumulated with atomics; nullable
  int B, L;
  int bf16;              // the index queries and keys are bf16 instead of fp16
  const int32_t* page_table;   // paged keys: positions [i * page_size, (i+1) * page_size) of request b are page
                               // page_table[b * table_stride + i] of tmIK = (pages, page_size, 128); null = (B, L, 128)
  int page_size, table_stride, pages;
  const float* iq_scale;       // fp8 index keys only: per (request, head) scale of iq (B, 64), and
  const float* ik_scale;       // per position scale of ik (B, L); tmIK / tmIQ then describe bytes
  int32_t* status;
};

__device__ __forceinline__ float relu_nan(float x) { return (x < 0.f) ? 0.f : x; }

// FP8: ik and iq are e4m3 bytes with scales (a tile is 16 KiB, one 128-byte swizzled row per position; four
// kind::f8f6f4 MMAs of K = 32 per tile).  The shared-memory layout keeps the fp16 sizes.
template <bool FP8>
__global__ void __launch_bounds__(kTcThreads, 1) indexer_tc_kernel(const __grid_constant__ TcParams p) {
  constexpr int kTileLoad = FP8 ? kTileBytes / 2 : kTileBytes;   // bytes one tile brings in = size of a ring slot
  constexpr int kSt = kStages;                                   // ring slots (twelve fp8 slots were no faster)
  constexpr int kIqLoad = FP8 ? kIqBytes / 2 : kIqBytes;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sIQ = smem + kStages * kTileBytes;
  float* sW = reinterpret_cast<float*>(sIQ + kIqBytes);
  uint32_t* sHist = reinterpret_cast<uint32_t*>(sW + kHI);
  uint64_t* full = reinterpret_cast<uint64_t*>(sHist + kSelBins);
  uint64_t* empty = full + kSt;
  uint64_t* acc_full = empty + kSt;
  uint64_t* acc_empty = acc_full + kAccs;
  uint64_t* iq_full = acc_empty + kAccs;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(iq_full + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.y;
  // the top-k selection is launched as a programmatic dependent of this grid: it may set itself up from here on,
  // and waits for this grid to finish before it reads the scores
  pdl_release();
  int n = p.L;
  if (p.lens != nullptr) n = max(0, min(p.lens[b], p.L));
  if (n <= kTopK) return;                                   // uniform: nothing to rank for this request
  const int tiles = (n + kTile - 1) / kTile;
  const int per = (tiles + gridDim.x - 1) / gridDim.x;
  const int t0 = blockIdx.x * per;
  const int t1 = min(tiles, t0 + per);
  if (t0 >= t1) return;                                     // uniform
  const int nt = t1 - t0;

  if (tid == 0) {
    for (int s = 0; s < kSt; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < kAccs; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    mbar_init(iq_full, 1);
    fence_mbar_init();
  }
  if (tid < kHI) sW[tid] = p.w[b * kHI + tid] * (FP8 ? p.iq_scale[b * kHI + tid] : 1.f);
  if (p.hist != nullptr)
    for (int i = tid; i < kSelBins; i += kTcThreads) sHist[i] = 0u;
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  bool timed_out = false;
  if (warp == 0) {
    // ---------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      mbar_expect_tx(iq_full, kIqLoad);
      tma_load_3d(sIQ, &p.tmIQ, 0, 0, b, iq_full);
      if (!FP8) tma_load_3d(sIQ + kIqBytes / 2, &p.tmIQ, 64, 0, b, iq_full);
      // Paged keys: a 128-position tile lies inside one page (page_size is a multiple of 128).  The table entry of
      // the NEXT tile is requested one iteration ahead, so that its latency hides behind the wait for a free slot.
      auto page_of = [&](int pos) -> int {
        const int pi = pos / p.page_size;
        return pi < p.table_stride ? p.page_table[(size_t)b * p.table_stride + pi] : -1;
      };
      int pg_next = (p.page_table != nullptr && nt > 0) ? page_of(t0 * kTile) : 0;
      for (int j = 0; j < nt; ++j) {
        const int s = j % kSt;
        const int pg = pg_next;
        if (p.page_table != nullptr && j + 1 < nt) pg_next = page_of((t0 + j + 1) * kTile);
        if (j >= kSt && !mbar_wait(&empty[s], (uint32_t)(((j / kSt) - 1) & 1))) {
          timed_out = true;
          break;
        }
        uint8_t* st = smem + s * kTileLoad;
        mbar_expect_tx(&full[s], kTileLoad);
        int y = (t0 + j) * kTile, z = b;
        if (p.page_table != nullptr) {
          // a page id outside the pool makes the TMA coordinate out of range, which reads zeros
          z = (pg >= 0 && pg < p.pages) ? pg : p.pages;
          y %= p.page_size;
        }
        tma_load_3d(st, &p.tmIK, 0, y, z, &full[s]);
        if (!FP8) tma_load_3d(st + kTileBytes / 2, &p.tmIK, 64, y, z, &full[s]);
      }
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------------------------------------------------------------------- MMA issuers
    // With fp8 keys the two issuing threads take alternate tiles (their accumulators differ): a tile's four
    // instructions take ~390 cycles, and the two waits in front of them would otherwise cost as much again.
    constexpr int kIssuers = FP8 ? 2 : 1;
    const int mi = warp == 1 ? 0 : 1;
    if (lane == 0 && mi < kIssuers) {
      if (!mbar_wait(iq_full, 0)) timed_out = true;
      const uint32_t iq_addr = smem_u32(sIQ);
      // Instruction descriptor: fp16 or bf16 A and B (both K-major), fp32 accumulate, M = 128, N = 64.
      const uint32_t idesc = umma_idesc_16(kTile, kHI, 0, FP8 ? 0 : p.bf16);
      for (int j = mi; j < nt && !timed_out; j += kIssuers) {
        const int s = j % kSt, a = j % kAccs;
        if (j >= kAccs && !mbar_wait(&acc_empty[a], (uint32_t)(((j / kAccs) - 1) & 1))) {
          timed_out = true;
          break;
        }
        if (!mbar_wait(&full[s], (uint32_t)((j / kSt) & 1))) {
          timed_out = true;
          break;
        }
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * kTileLoad);
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * kHI);
        if (FP8) {
#pragma unroll
          for (int k = 0; k < kDI / 32; ++k)    // K step k: 32 bytes further inside the one 128-byte swizzled row
            umma_f8(d_tmem, umma_desc_sw128(a_addr + k * 32), umma_desc_sw128(iq_addr + k * 32), idesc, k > 0 ? 1u : 0u);
        } else {
#pragma unroll
          for (int k = 0; k < kDI / 16; ++k) {
            // K step k: 64-element half (k / 4), 32-byte offset (k % 4) inside the 128-byte swizzled row
            const uint64_t da = umma_desc_sw128(a_addr + (k >> 2) * (kTileBytes / 2) + (k & 3) * 32);
            const uint64_t db = umma_desc_sw128(iq_addr + (k >> 2) * (kIqBytes / 2) + (k & 3) * 32);
            umma_f16(d_tmem, da, db, idesc, k > 0 ? 1u : 0u);
          }
        }
        umma_commit(&empty[s]);        // the ring slot may be refilled once these MMAs have read it
        umma_commit(&acc_full[a]);     // the accumulator is complete
      }
    }
  } else if (warp >= 2 && warp <= 9) {
    // ---------------------------------------------------------------------------- epilogue (warps 2..9)
    // Two sets of four warps take alternate tiles (tile j uses accumulator j % 4, so a set always sees the same two
    // accumulators): with fp8 keys a tile arrives every ~700 cycles at the HBM rate, more than one set can keep up with.
    const int set = (warp - 2) >> 2;
    const int quarter = warp & 3;                         // tensor-memory lanes [32 q, 32 q + 32)
    const int row = quarter * 32 + lane;                  // position inside the tile
    float* dst = p.scores + (size_t)b * p.L;
    // (16-bit keys are HBM-bound with one set: the second set then stays idle)
    constexpr int kSets = FP8 ? 2 : 1;
    for (int j = set < kSets ? set : nt; j < nt; j += kSets) {
      const int a = j % kAccs;
      const int pos = (t0 + j) * kTile + row;
      // fp8: this position's key scale, requested before the wait so that its latency hides behind it
      float kscale = 1.f;
      if (FP8 && pos < n) kscale = p.ik_scale[(size_t)b * p.L + pos];
      const bool ok = mbar_wait(&acc_full[a], (uint32_t)((j / kAccs) & 1));
      if (!__all_sync(0xffffffffu, ok)) {
        timed_out = true;
        break;
      }
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(a * kHI);
      uint32_t r0[32], r1[32];
      tmem_ld32(taddr, r0);
      tmem_ld32(taddr + 32, r1);
      tmem_ld_wait();
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&acc_empty[a]);          // this warp's quarter has been read out
      float s = 0.f;
#pragma unroll
      for (int h = 0; h < 32; ++h) s += sW[h] * relu_nan(__uint_as_float(r0[h]));
#pragma unroll
      for (int h = 0; h < 32; ++h) s += sW[32 + h] * relu_nan(__uint_as_float(r1[h]));
      if (pos < n) {
        if (FP8) s *= kscale;
        dst[pos] = s;
        // first level of the top-k radix select, fused here so that the select pass starts one level down
        if (p.hist != nullptr) atomicAdd(&sHist[score_key(s) >> kSelShift], 1u);
      }
    }
  }
  if (timed_out) report(p.status, kStatusTimeout);

  // common exit: every warp arrives here, then the allocating warp frees the tensor memory
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_free(tmem_base, kTmemCols);
  }
  if (p.hist != nullptr) {
    for (int i = tid; i < kSelBins; i += kTcThreads) {
      const uint32_t c = sHist[i];
      if (c != 0u) atomicAdd(&p.hist[(size_t)b * kSelBins + i], c);
    }
  }
}

int indexer_chunks(int B, int tiles);

int indexer_tc_launch(const CUtensorMap& tmIK, const CUtensorMap& tmIQ, const float* w, const int32_t* lens,
                      float* scores, uint32_t* hist, int B, int L, int32_t* status, cudaStream_t stream, int bf16, const int32_t* page_table, int page_size,
                      int table_stride, int pages, const float* iq_scale, const float* ik_scale) {
  TcParams p;
  memset(&p, 0, sizeof(p));
  p.tmIK = tmIK;
  p.tmIQ = tmIQ;
  p.w = w; p.lens = lens; p.scores = scores; p.hist = hist; p.B = B; p.L = L; p.status = status;
  p.bf16 = bf16;
  p.page_table = page_table; p.page_size = page_size; p.table_stride = table_stride; p.pages = pages;
  p.iq_scale = iq_scale; p.ik_scale = ik_scale;
  const bool fp8 = iq_scale != nullptr;
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(indexer_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
    if (e != cudaSuccess) return check_launch(e);
    e = cudaFuncSetAttribute(indexer_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, kTcSmem);
    if (e != cudaSuccess) return check_launch(e);
    configured_dev = dev;
  }
  const int chunks = indexer_chunks(B, cdiv(L, kTile));
  if (fp8) indexer_tc_kernel<true><<<dim3(chunks, B), kTcThreads, kTcSmem, stream>>>(p);
  else indexer_tc_kernel<false><<<dim3(chunks, B), kTcThreads, kTcSmem, stream>>>(p);
  return check_launch(cudaGetLastError());
}

}  // namespace vmk
