// `dsa` stage 1 on the 5th-generation tensor cores: scores[b,l] = sum_h w[b,h] * relu(iq[b,h] . ik[b,l]).
//
// Per 128-position tile the product T = ik_tile (128 x 128, K-major) . iq^T (64 x 128, K-major) is one
// tcgen05 accumulator of 128 lanes x 64 fp32 columns in tensor memory.  The kernel is PERSISTENT: the tiles
// of all requests that have something to rank form one list, cut into equal contiguous ranges, one per CTA
// and one CTA per SM, so that no wave of CTAs is left part-filled and every SM pays the set-up once.  A range
// may cross from one request into the next: the index queries are double-buffered in shared memory, the head
// weights and the histogram are switched between requests by the epilogue warps.  Warp-specialised:
//   warp 0     TMA producer: a request's 16 KiB of index queries, then its 32 KiB ik tiles into a 5-deep
//              shared-memory ring (128-byte swizzle; ten 16 KiB slots with fp8 keys)
//   warp 1     (and warp 10 for fp8 keys) allocates tensor memory, issues 8 tcgen05.mma (M128 N64 K16) per tile
//              into one of four accumulator buffers, commits the ring slot back to the producer and the
//              accumulator to the epilogue
//   warps 2-9  epilogue, two sets of four warps on alternate tiles (the second set only with fp8 keys):
//              tcgen05.ld of their 32 lanes x 64 columns, fp32 ReLU and head-weighted sum, one coalesced fp32
//              score per position, and the count of the score's top 11 key bits in a shared-memory histogram
//              that is added to the request's global one when the range leaves the request
// Every mbarrier wait is bounded; a wait that runs out sets the status word and the CTA winds down
// through the common exit, where the allocating warp frees its tensor memory.
#include "tcgen05.cuh"

namespace vmk {

constexpr int kTopK = VMK_DSA_TOPK;
constexpr int kHI = 64, kDI = 128;
constexpr int kTile = 128;
constexpr int kStages = 5;
constexpr int kAccs = 4;                               // accumulator buffers of 64 columns
constexpr int kTileBytes = kTile * kDI * 2;            // 32 KiB
constexpr int kIqBytes = kHI * kDI * 2;                // 16 KiB
constexpr int kTmemCols = kAccs * kHI;                 // 256
constexpr int kTcThreads = 352;
// ring | iq x 2 | w | histogram | barriers | tmem base
constexpr int kTcSmem =
    kStages * kTileBytes + 2 * kIqBytes + kHI * 4 + kSelBins * 4 + (4 * kStages + 2 * kAccs + 4) * 8 + 16 + 1024;

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

// Length of request b, and the tiles it contributes: none when it has nothing to rank.
__device__ __forceinline__ int req_len(const TcParams& p, int b) {
  return p.lens != nullptr ? max(0, min(p.lens[b], p.L)) : p.L;
}
__device__ __forceinline__ int req_tiles(int n) { return n > kTopK ? (n + kTile - 1) / kTile : 0; }

// Walks the requests that a CTA's tile range [g0, g1) touches.  `base` counts the tiles of the requests before b.
struct RunWalk {
  int b, base;
  int n, ta, tb;      // the current run: request length, tiles [ta, tb) of that request
  int req;            // the request of the current run
};
__device__ __forceinline__ bool next_run(const TcParams& p, RunWalk& w, int g0, int g1) {
  while (w.b < p.B && w.base < g1) {
    w.n = req_len(p, w.b);
    const int rt = req_tiles(w.n);
    w.ta = max(g0 - w.base, 0);
    w.tb = min(g1 - w.base, rt);
    w.req = w.b;
    w.base += rt;
    ++w.b;
    if (w.ta < w.tb) return true;
  }
  return false;
}

// FP8: ik and iq are e4m3 bytes with scales (a tile is 16 KiB, one 128-byte swizzled row per position; four
// kind::f8f6f4 MMAs of K = 32 per tile).  The shared-memory layout keeps the fp16 sizes.
template <bool FP8>
__global__ void __launch_bounds__(kTcThreads, 1) indexer_tc_kernel(const __grid_constant__ TcParams p) {
  constexpr int kTileLoad = FP8 ? kTileBytes / 2 : kTileBytes;   // bytes one tile brings in = size of a ring slot
  // Ring slots.  With fp8 keys there are two issuing threads on alternate tiles, and the number of slots must be
  // EVEN so that a slot always comes back to the same thread: a thread that ran ahead and asked for a slot that still
  // holds the other thread's earlier tile would see the parity of the phase before and take the old tile for its own.
  constexpr int kSt = FP8 ? 2 * kStages : kStages;
  static_assert(!FP8 || (kSt % 2 == 0 && kAccs % 2 == 0), "two issuing threads: slots and accumulators must not change hands");
  constexpr int kIqLoad = FP8 ? kIqBytes / 2 : kIqBytes;
  constexpr int kIssuers = FP8 ? 2 : 1;
  constexpr int kSets = FP8 ? 2 : 1;
  constexpr int kWarps = kTcThreads / 32;
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_wsum[kWarps];
  __shared__ int s_first[2];                                     // first request of the range, tiles before it
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sIQ = smem + kStages * kTileBytes;                    // two buffers of 16 KiB
  float* sW = reinterpret_cast<float*>(sIQ + 2 * kIqBytes);
  uint32_t* sHist = reinterpret_cast<uint32_t*>(sW + kHI);
  uint64_t* full = reinterpret_cast<uint64_t*>(sHist + kSelBins);
  uint64_t* empty = full + kSt;
  uint64_t* acc_full = empty + kSt;
  uint64_t* acc_empty = acc_full + kAccs;
  uint64_t* iq_full = acc_empty + kAccs;                         // [2] a request's queries have landed
  uint64_t* iq_empty = iq_full + 2;                              // [2] every MMA that reads them is done
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(iq_empty + 2);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // the top-k selection is launched as a programmatic dependent of this grid: it may set itself up from here on,
  // and waits for this grid to finish before it reads the scores
  pdl_release();

  if (tid == 0) {
    for (int s = 0; s < kSt; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int a = 0; a < kAccs; ++a) {
      mbar_init(&acc_full[a], 1);
      mbar_init(&acc_empty[a], 4);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&iq_full[i], 1);
      mbar_init(&iq_empty[i], kIssuers);
    }
    fence_mbar_init();
  }
  if (p.hist != nullptr)
    for (int i = tid; i < kSelBins; i += kTcThreads) sHist[i] = 0u;
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);

  // This CTA's range of the tile list.  Each thread counts the tiles of a contiguous segment of requests; an
  // exclusive scan over the block gives the total and the segment that holds the range's first tile.
  const int seg = (p.B + kTcThreads - 1) / kTcThreads;
  const int sb0 = min(p.B, tid * seg), sb1 = min(p.B, sb0 + seg);
  int mine = 0;
  for (int b = sb0; b < sb1; ++b) mine += req_tiles(req_len(p, b));
  int incl = mine;
#pragma unroll
  for (int d = 1; d < 32; d <<= 1) {
    const int v = __shfl_up_sync(0xffffffffu, incl, d);
    if (lane >= d) incl += v;
  }
  if (lane == 31) s_wsum[warp] = incl;
  __syncthreads();
  int total = 0, wbase = 0;
#pragma unroll
  for (int i = 0; i < kWarps; ++i) {
    if (i < warp) wbase += s_wsum[i];
    total += s_wsum[i];
  }
  const int g0 = (int)((long long)total * blockIdx.x / gridDim.x);
  const int g1 = (int)((long long)total * (blockIdx.x + 1) / gridDim.x);
  {
    const int excl = wbase + incl - mine;
    if (g0 < g1 && g0 >= excl && g0 < excl + mine) {
      int acc = excl;
      for (int b = sb0; b < sb1; ++b) {
        const int rt = req_tiles(req_len(p, b));
        if (g0 < acc + rt) {
          s_first[0] = b;
          s_first[1] = acc;
          break;
        }
        acc += rt;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  RunWalk run;
  run.b = g0 < g1 ? s_first[0] : p.B;
  run.base = g0 < g1 ? s_first[1] : 0;

  bool timed_out = false;
  if (warp == 0) {
    // ---------------------------------------------------------------------------- TMA producer
    if (lane == 0) {
      // Paged keys: a 128-position tile lies inside one page (page_size is a multiple of 128).  The table entry of
      // the NEXT tile is requested one iteration ahead, so that its latency hides behind the wait for a free slot.
      int b = 0;
      auto page_of = [&](int pos) -> int {
        const int pi = pos / p.page_size;
        return pi < p.table_stride ? p.page_table[(size_t)b * p.table_stride + pi] : -1;
      };
      int j = 0, q = 0;                                            // tiles, requests so far
      while (!timed_out && next_run(p, run, g0, g1)) {
        b = run.req;
        const int iqs = q & 1;
        if (q >= 2 && !mbar_wait(&iq_empty[iqs], (uint32_t)(((q >> 1) - 1) & 1))) {
          timed_out = true;
          break;
        }
        mbar_expect_tx(&iq_full[iqs], kIqLoad);
        tma_load_3d(sIQ + iqs * kIqBytes, &p.tmIQ, 0, 0, b, &iq_full[iqs]);
        if (!FP8) tma_load_3d(sIQ + iqs * kIqBytes + kIqBytes / 2, &p.tmIQ, 64, 0, b, &iq_full[iqs]);
        int pg_next = p.page_table != nullptr ? page_of(run.ta * kTile) : 0;
        for (int t = run.ta; t < run.tb; ++t, ++j) {
          const int s = j % kSt;
          const int pg = pg_next;
          if (p.page_table != nullptr && t + 1 < run.tb) pg_next = page_of((t + 1) * kTile);
          if (j >= kSt && !mbar_wait(&empty[s], (uint32_t)(((j / kSt) - 1) & 1))) {
            timed_out = true;
            break;
          }
          uint8_t* st = smem + s * kTileLoad;
          mbar_expect_tx(&full[s], kTileLoad);
          int y = t * kTile, z = b;
          if (p.page_table != nullptr) {
            // a page id outside the pool makes the TMA coordinate out of range, which reads zeros
            z = (pg >= 0 && pg < p.pages) ? pg : p.pages;
            y %= p.page_size;
          }
          tma_load_3d(st, &p.tmIK, 0, y, z, &full[s]);
          if (!FP8) tma_load_3d(st + kTileBytes / 2, &p.tmIK, 64, y, z, &full[s]);
        }
        ++q;
      }
      // no load outlives the CTA: returns at once unless a consumer gave up before it had waited for them
      for (int i = max(0, j - kSt); i < j; ++i) mbar_wait(&full[i % kSt], (uint32_t)((i / kSt) & 1));
    }
  } else if (warp == 1 || warp == 10) {
    // ---------------------------------------------------------------------------- MMA issuers
    // With fp8 keys the two issuing threads take alternate tiles (their accumulators differ): a tile's four
    // instructions take ~390 cycles, and the two waits in front of them would otherwise cost as much again.
    const int mi = warp == 1 ? 0 : 1;
    if (lane == 0 && mi < kIssuers) {
      // Instruction descriptor: fp16 or bf16 A and B (both K-major), fp32 accumulate, M = 128, N = 64.
      const uint32_t idesc = umma_idesc_16(kTile, kHI, 0, FP8 ? 0 : p.bf16);
      int j = 0, q = 0;
      while (!timed_out && next_run(p, run, g0, g1)) {
        const int iqs = q & 1;
        if (!mbar_wait(&iq_full[iqs], (uint32_t)((q >> 1) & 1))) {
          timed_out = true;
          break;
        }
        const uint32_t iq_addr = smem_u32(sIQ + iqs * kIqBytes);
        for (int t = run.ta; t < run.tb; ++t, ++j) {
          if (j % kIssuers != mi) continue;
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
        if (timed_out) break;
        umma_commit(&iq_empty[iqs]);     // this thread's MMAs on the request's queries are done
        ++q;
      }
    }
  } else if (warp >= 2 && warp <= 9) {
    // ---------------------------------------------------------------------------- epilogue (warps 2..9)
    // Two sets of four warps take alternate tiles (tile j uses accumulator j % 4, so a set always sees the same two
    // accumulators): with fp8 keys a tile arrives every ~700 cycles at the HBM rate, more than one set can keep up
    // with.  16-bit keys are HBM-bound with one set: the second set then stays out altogether.
    const int set = (warp - 2) >> 2;
    const int quarter = warp & 3;                         // tensor-memory lanes [32 q, 32 q + 32)
    const int row = quarter * 32 + lane;                  // position inside the tile
    const int et = tid - 64;                              // thread index among the epilogue warps
    // the participating epilogue threads meet at both ends of every request (named barrier 1)
    auto ebar = [&]() { asm volatile("bar.sync 1, %0;" ::"n"(kSets * 128) : "memory"); };
    if (set < kSets) {
      int j = 0;
      uint64_t score_policy;
      asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(score_policy));
      while (next_run(p, run, g0, g1)) {
        const int b = run.req, n = run.n;
        // the request's head weights (times its query scales with fp8 keys): everybody is past the closing
        // barrier of the request before, so nobody reads the old ones any more
        if (et < kHI) sW[et] = p.w[b * kHI + et] * (FP8 ? p.iq_scale[b * kHI + et] : 1.f);
        ebar();
        float* dst = p.scores + (size_t)b * p.L;
        for (int t = run.ta; t < run.tb && !timed_out; ++t, ++j) {
          if (j % kSets != set) continue;
          const int a = j % kAccs;
          const int pos = t * kTile + row;
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
            // the scores are read again at once by the selection: last to leave L2 among what this kernel streams
            asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(dst + pos), "f"(s), "l"(score_policy) : "memory");
            // first level of the top-k radix select, fused here so that the select pass starts one level down
            if (p.hist != nullptr) atomicAdd(&sHist[score_key(s) >> kSelShift], 1u);
          }
        }
        // Leaving the request: its counts go to its global histogram and the shared one starts again from zero.
        // A warp that gave up skips the remaining tiles, not the barriers, so nobody is left waiting at one.
        ebar();
        if (p.hist != nullptr) {
          for (int i = et; i < kSelBins; i += kSets * 128) {
            const uint32_t c = sHist[i];
            if (c != 0u) {
              atomicAdd(&p.hist[(size_t)b * kSelBins + i], c);
              sHist[i] = 0u;
            }
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
    tmem_free(tmem_base, kTmemCols);
  }
}

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
  // one CTA per SM; fewer when the tiles would not give each of them two (a small call is all latency: spreading
  // it thin costs a CTA's set-up once, in parallel, and shortens every CTA's run)
  const long long tiles = (long long)B * cdiv(L, kTile);
  int ncta = sm_count();
  if (tiles < (long long)ncta * 2) ncta = (int)((tiles + 1) / 2);
  if (ncta < 1) ncta = 1;
  if (fp8) indexer_tc_kernel<true><<<ncta, kTcThreads, kTcSmem, stream>>>(p);
  else indexer_tc_kernel<false><<<ncta, kTcThreads, kTcSmem, stream>>>(p);
  return check_launch(cudaGetLastError());
}

}  // namespace vmk
