// `prefix` and `spec` entry points: launch planning, the split-KV kernel instantiations and the
// log-sum-exp combine pass.
#include "attn_core.cuh"

namespace vmk {

// ------------------------------------------------------------------------------------------------
// kernels
// ------------------------------------------------------------------------------------------------
template <int RT, int KS, int STAGES, bool HAS_B, int MIN_CTAS, bool BF>
__global__ void __launch_bounds__(256, MIN_CTAS) attn_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int cta = blockIdx.x;
  if (!HAS_B || cta < p.a.n_cta) {
    attn_core<RT, KS, STAGES, BF>(p.a, p.sc, p.status, cta, smem);
  } else {
    attn_core<1, 4, STAGES, BF>(p.b, p.sc, p.status, cta - p.a.n_cta, smem);
  }
}

struct CombineSide {
  const float* part_o;
  const float* part_ml;
  int nsplit, MP, rows_outer;
};

struct CombineParams {
  CombineSide a, b;
  int has_b;
  int Hkv, G, Hq;
  __half* out;       // (outers, Hq, 128) fp16 or bf16, or null
  int bf16;
  float* pm;         // when out is null: un-normalised merged partial per row, row r at pm[r * ml_stride],
  float* pl;         // pl[r * ml_stride] and po[r * o_stride + d]; (1, 128) for separate arrays, (130, 130) with
  float* po;         // pl = pm + 1, po = pm + 2 for one packed record (m, l, o[128]) per row
  int ml_stride, o_stride;
};

constexpr int kMaxParts = 640;     // upper bound of splits merged into one row (both sides together)

// One CTA of NG x 32 threads per output row (outer, head): NG groups of 32 lanes; group g merges the splits
// t = g, g + NG, g + 2 NG, ... and lane l owns columns [4 l, 4 l + 4).  Every thread requests its first four
// partial rows (4 NG splits per CTA) at once, before the (m, l) pairs that give them their weights have even
// arrived, so that a row of the usual 9-37 splits costs one round trip to L2 instead of one per eight splits;
// the group sums meet in shared memory.  NG = 8 for decode-sized calls (few rows, many splits: latency is all
// there is), NG = 4 when there are thousands of rows.  Launched with programmatic stream serialisation: the grid
// may be scheduled while the split kernel is still running and waits here for its results.
template <int NG>
__global__ void __launch_bounds__(NG * 32) combine_kernel(const CombineParams p) {
  __shared__ float s_m[kMaxParts], s_l[kMaxParts];
  __shared__ float4 s_red[NG][32];
  __shared__ float s_lred[NG];
  if (blockIdx.x == 0) ATTN_M(1024, 0);
  // the next call's split kernel (a programmatic dependent of this grid) may be scheduled from here on: it sets
  // itself up and waits for this grid to finish before it reads anything
  pdl_release();
  pdl_wait();
  if (blockIdx.x == 0) ATTN_M(1024, 1);
  const int row = blockIdx.x;
  const int tid = threadIdx.x, lane = tid & 31, grp = tid >> 5;
  const int outer = row / p.Hq, hq = row % p.Hq;
  const int h = hq / p.G, g = hq % p.G;
  const int nA = p.a.nsplit, nB = p.has_b ? p.b.nsplit : 0;
  const int total = min(nA + nB, kMaxParts);
  // index of split t's record of this row in its side's partial arrays
  auto record = [&](int t, const CombineSide** side) -> size_t {
    const CombineSide& sd = t < nA ? p.a : p.b;
    const int s = t < nA ? t : t - nA;
    const int z = (outer / sd.rows_outer) * p.Hkv + h;
    const int r = (outer % sd.rows_outer) * p.G + g;
    *side = &sd;
    return ((size_t)z * sd.nsplit + s) * sd.MP + r;
  };
  float4 o[4];
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int t = grp + NG * k;
    o[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (t < total) {
      const CombineSide* sd;
      const size_t i = record(t, &sd);
      o[k] = *reinterpret_cast<const float4*>(sd->part_o + i * kHD + lane * 4);
    }
  }
  for (int t = tid; t < total; t += NG * 32) {
    const CombineSide* sd;
    const size_t i = record(t, &sd);
    const float2 ml = *reinterpret_cast<const float2*>(sd->part_ml + i * 2);
    s_m[t] = ml.x;
    s_l[t] = ml.y;
  }
  __syncthreads();
  float M = -INFINITY;
  for (int t = 0; t < total; ++t) M = fmaxf(M, s_m[t]);
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  float lsum = 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const int t = grp + NG * k;
    if (t < total) {
      const float m = s_m[t];
      const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
      acc.x += w * o[k].x; acc.y += w * o[k].y; acc.z += w * o[k].z; acc.w += w * o[k].w;
      lsum += w * s_l[t];
    }
  }
  for (int t = grp + 4 * NG; t < total; t += NG) {        // rows with more than 4 NG splits: the rest, one by one
    const CombineSide* sd;
    const size_t i = record(t, &sd);
    const float4 v = *reinterpret_cast<const float4*>(sd->part_o + i * kHD + lane * 4);
    const float m = s_m[t];
    const float w = (m == -INFINITY) ? 0.f : exp2f(m - M);
    acc.x += w * v.x; acc.y += w * v.y; acc.z += w * v.z; acc.w += w * v.w;
    lsum += w * s_l[t];
  }
  s_red[grp][lane] = acc;
  if (lane == 0) s_lred[grp] = lsum;
  __syncthreads();
  if (tid >= 32) return;
  acc = s_red[0][lane];
  lsum = s_lred[0];
#pragma unroll
  for (int q = 1; q < NG; ++q) {
    const float4 v = s_red[q][lane];
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    lsum += s_lred[q];
  }
  if (blockIdx.x == 0) ATTN_M(1024, 2);
  const int d = lane * 4;
  if (p.out != nullptr) {
    uint2 pk;
    pk.x = pack2(acc.x / lsum, acc.y / lsum, p.bf16);
    pk.y = pack2(acc.z / lsum, acc.w / lsum, p.bf16);
    *reinterpret_cast<uint2*>(&p.out[(size_t)row * kHD + d]) = pk;
  } else {
    float* po = p.po + (size_t)row * p.o_stride + d;      // packed records start 8 bytes into the row: scalar stores
    po[0] = acc.x; po[1] = acc.y; po[2] = acc.z; po[3] = acc.w;
    if (lane == 0) {
      p.pm[(size_t)row * p.ml_stride] = M;
      p.pl[(size_t)row * p.ml_stride] = lsum;
    }
  }
}

int g_batch_invariant = 0;

// Launch of the combine pass as a programmatic dependent of the kernel enqueued just before it.
static int launch_combine(const CombineParams& c, int rows, cudaStream_t stream) {
  if (c.a.nsplit + (c.has_b ? c.b.nsplit : 0) > kMaxParts) return VMK_E_UNSUPPORTED;
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  // (batch-invariant mode: one fixed variant, so that a row's sum order does not depend on the row count)
  const bool few_rows = g_batch_invariant || rows <= 2048;
  cfg.gridDim = dim3(rows);
  cfg.blockDim = dim3(few_rows ? 256 : 128);
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_launch(few_rows ? cudaLaunchKernelEx(&cfg, combine_kernel<8>, c) : cudaLaunchKernelEx(&cfg, combine_kernel<4>, c));
}

// Merge of `parts` partials per row (used after an exchange between GPUs).
__global__ void __launch_bounds__(128) lse_merge_kernel(const float* __restrict__ m, const float* __restrict__ l,
                                                         const float* __restrict__ o, int parts, int rows, int D,
                                                         __half* __restrict__ out, int bf16) {
  const int row = blockIdx.x;
  float M = -INFINITY;
  for (int s = 0; s < parts; ++s) M = fmaxf(M, m[(size_t)s * rows + row]);
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float acc = 0.f, lsum = 0.f;
    for (int s = 0; s < parts; ++s) {
      const float ms = m[(size_t)s * rows + row];
      const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      acc += w * o[((size_t)s * rows + row) * D + d];
      lsum += w * l[(size_t)s * rows + row];
    }
    store16(&out[(size_t)row * D + d], acc / lsum, bf16);
  }
}

// The same merge over packed records: rec (parts, rows, 130) with (m, l, o[128]) per row, the layout in which
// partials arrive from other GPUs.  One CTA of 128 threads per row; thread d owns column d.
__global__ void __launch_bounds__(128) lse_merge_packed_kernel(const float* __restrict__ rec, int parts, int rows,
                                                                __half* __restrict__ out, int bf16) {
  constexpr int kRec = kHD + 2;
  const int row = blockIdx.x, d = threadIdx.x;
  const float* r0 = rec + (size_t)row * kRec;
  const size_t step = (size_t)rows * kRec;
  float M = -INFINITY;
  for (int s = 0; s < parts; ++s) M = fmaxf(M, r0[s * step]);
  float acc = 0.f, lsum = 0.f;
  for (int s = 0; s < parts; ++s) {
    const float ms = r0[s * step];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    acc += w * r0[s * step + 2 + d];
    lsum += w * r0[s * step + 1];
  }
  store16(&out[(size_t)row * kHD + d], acc / lsum, bf16);
}

// ------------------------------------------------------------------------------------------------
// planning
// ------------------------------------------------------------------------------------------------
int launch_attn_tc(const AttnParams& p, int n_cta, cudaStream_t stream);   // attn_tc.cu


static int g_attn_tc = 1;   // 1: row tiles of 128 run on tcgen05 (attn_tc.cu); 0: always the warp-level kernel
static int g_side_by_side = 1;   // 1: big prefix calls run their two kernels at the same time (see PrefixPlan)
constexpr int kTcRowsMin = 65;     // stacked rows from which the tensor-memory kernel is used
constexpr int kTcSplitCap = 32;

struct RolePlan {
  bool tc;                 // tcgen05 kernel (128-row tiles, 128-key blocks)
  int rt, ks;              // warp layout of the role's CTAs
  int row_tiles, MP;
  int nsplit, split_len;
  int n_cta;
  size_t off_o, off_ml;    // offsets into the workspace
};

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

static void pick_layout(int rows, int* rt, int* ks) {
  if (rows <= 16) { *rt = 1; *ks = 4; }
  else if (rows <= 32) { *rt = 2; *ks = 4; }
  else if (rows <= 64) { *rt = 4; *ks = 2; }
  else { *rt = 8; *ks = 1; }
}

// Splits the keys of each (group, row tile) so that about `target` CTAs exist, in multiples of 64 keys.
// Upper bound of the split count of the tcgen05 path; also sizes its share of the workspace, so that
// one workspace size serves every key range.
static int tc_split_cap(int units) {
  int cap = cdiv(2 * sm_count(), units > 0 ? units : 1);
  if (cap > kTcSplitCap) cap = kTcSplitCap;
  return cap < 1 ? 1 : cap;
}

// tcgen05 path: one CTA per SM, 256-row tiles, 128-key blocks.  The split count minimises
// waves x (blocks per CTA + a fixed per-CTA overhead of about three blocks), which avoids a mostly empty
// last wave.
// one_wave_on > 0: the CTAs must fit ONE wave on that many SMs (the rest of the GPU is left to a kernel that runs
// beside this one); the largest split count that does is taken.
static void plan_role_tc(RolePlan* r, int groups, int rows, int keys, int one_wave_on = 0) {
  constexpr int kTcBlock = 128;      // keys per block of the tensor-memory kernel
  r->tc = true;
  r->rt = 8; r->ks = 1;
  r->row_tiles = cdiv(rows, 256);
  r->MP = rows;                      // partial rows are indexed by the real row, no padding needed
  const int units = groups * r->row_tiles;
  const int blocks = cdiv(keys > 0 ? keys : 1, kTcBlock);
  const int sms = sm_count();
  const int cap = tc_split_cap(units);
  long long best_cost = -1;
  int best = 1;
  for (int ns = 1; ns <= cap && ns <= blocks; ++ns) {
    const int per = cdiv(blocks, ns);
    const int real = cdiv(blocks, per);
    if (one_wave_on > 0) {
      if (units * real <= one_wave_on || real == 1) best = real;      // ascending: ends at the largest that fits
      continue;
    }
    const long long cost = (long long)cdiv(units * real, sms) * (per + 3);
    if (best_cost < 0 || cost < best_cost) { best_cost = cost; best = real; }
  }
  r->split_len = cdiv(blocks, best) * kTcBlock;
  r->nsplit = cdiv(blocks * kTcBlock, r->split_len);
  r->n_cta = units * r->nsplit;
}

// Batch-invariant plan: the arithmetic of a row must not depend on what else is in the batch, so the kernel, the
// warp layout and the cut points of the key range are fixed: warp-level kernel, 16-row tiles with the 64 keys of a
// block over four warps, splits of 2048 keys (512 for the private suffixes).
static void plan_role_invariant(RolePlan* r, int groups, int rows, int keys, bool fixed_small) {
  r->tc = false;
  r->rt = 1; r->ks = 4;
  r->row_tiles = cdiv(rows, 16);
  r->MP = rows;
  r->split_len = fixed_small ? 512 : 2048;
  r->nsplit = cdiv(keys > 0 ? keys : 1, r->split_len);
  r->n_cta = groups * r->row_tiles * r->nsplit;
}

static void plan_role(RolePlan* r, int groups, int rows, int keys, int target, bool fixed_small, int one_wave_on = 0) {
  r->tc = false;
  if (g_batch_invariant) { plan_role_invariant(r, groups, rows, keys, fixed_small); return; }
  if (!fixed_small && g_attn_tc && rows >= kTcRowsMin) { plan_role_tc(r, groups, rows, keys, one_wave_on); return; }
  if (fixed_small) { r->rt = 1; r->ks = 4; } else pick_layout(rows, &r->rt, &r->ks);
  const int mt = r->rt * 16;
  r->row_tiles = cdiv(rows, mt);
  r->MP = rows;                      // partial rows are indexed by the real row, no padding needed
  const int units = groups * r->row_tiles;
  const int blocks = cdiv(keys > 0 ? keys : 1, kBK);
  int want = cdiv(target > 0 ? target : 1, units > 0 ? units : 1);
  // never more than 2048 keys per CTA: with many groups of unequal (ragged) lengths, short pieces balance the SMs,
  // and a piece's partial record (130 floats per row) is small beside the 1 MB of K and V it stands for
  if (!fixed_small && want < cdiv(blocks, 32)) want = cdiv(blocks, 32);
  if (want > blocks) want = blocks;
  if (want < 1) want = 1;
  r->split_len = cdiv(blocks, want) * kBK;
  r->nsplit = cdiv(blocks * kBK, r->split_len);
  r->n_cta = units * r->nsplit;
}

// Reserves the role's partial arrays.  They are sized for `cap` splits, an upper bound of nsplit that
// does not depend on the key range, so one workspace size serves full and partial (key_lo/key_hi) calls.
static size_t place(RolePlan* r, int groups, size_t off, int cap) {
  if (cap < r->nsplit) cap = r->nsplit;
  r->off_o = align_up(off, 256);
  r->off_ml = align_up(r->off_o + (size_t)groups * cap * r->MP * kHD * sizeof(float), 256);
  return r->off_ml + (size_t)groups * cap * r->MP * 2 * sizeof(float);
}

struct PrefixPlan {
  RolePlan a, b;
  bool has_a, has_b;       // shared-prefix role (keys [key_lo, key_hi) not empty), private-suffix role
  bool side_by_side;       // the tensor-bound prefix tiles and the HBM-bound suffix streams run at the same time
  size_t ws_bytes;
};

// From this many private suffixes (request x kv head) on, a call whose shared prefix runs on the tensor-memory
// kernel gives that kernel one wave on about two thirds of the SMs and streams the suffixes beside it on a second
// stream.  The rule looks at the number of suffixes, not at their length: the length bound S of a paged call is
// rounded up to whole pages, and the paged and the contiguous call must cut the work alike.
constexpr int kSideBySideGroups = 512;

static PrefixPlan plan_prefix(int N, int Hq, int Hkv, int P, int S, int key_lo, int key_hi, bool with_suffix) {
  PrefixPlan pl;
  const int G = Hq / Hkv;
  const int sms = sm_count();
  pl.has_a = key_hi > key_lo;
  pl.has_b = with_suffix && S > 0;
  // Suffix role: one group per (request, kv head), G rows; aim for chunks of at least 128 keys.
  int target_b = 0;
  if (pl.has_b) {
    const int groups_b = N * Hkv;
    int per = cdiv(2 * sms, groups_b);
    const int maxper = cdiv(S, 128);
    if (per > maxper) per = maxper;
    if (per < 1) per = 1;
    plan_role(&pl.b, groups_b, G, S, groups_b * per, true);
    target_b = pl.b.n_cta;
  } else {
    pl.b = RolePlan{};
  }
  size_t off = 0;
  pl.side_by_side = false;
  if (pl.has_a) {
    int target_a = 2 * sms - target_b;
    if (target_a < sms) target_a = sms;
    const bool big_suffix = pl.has_b && (long long)N * Hkv >= kSideBySideGroups;
    const bool tc_rows = !g_batch_invariant && g_attn_tc && N * G >= kTcRowsMin;
    pl.side_by_side = big_suffix && tc_rows && g_side_by_side;
    plan_role(&pl.a, Hkv, N * G, key_hi - key_lo, target_a, false, pl.side_by_side ? (2 * sms) / 3 : 0);
    off = place(&pl.a, Hkv, 0, pl.a.tc ? tc_split_cap(Hkv * pl.a.row_tiles) : cdiv(2 * sms, Hkv * pl.a.row_tiles));
  } else {
    pl.a = RolePlan{};
  }
  if (pl.has_b) off = place(&pl.b, N * Hkv, off, pl.b.nsplit);
  pl.ws_bytes = align_up(off, 256);
  return pl;
}

struct SpecPlan {
  RolePlan a;
  size_t ws_bytes;
};

static SpecPlan plan_spec(int B, int kd, int Hq, int Hkv, int key_lo, int key_hi) {
  SpecPlan pl;
  const int G = Hq / Hkv;
  plan_role(&pl.a, B * Hkv, kd * G, key_hi - key_lo, 2 * sm_count(), false);
  pl.ws_bytes = align_up(place(&pl.a, B * Hkv, 0, pl.a.tc ? tc_split_cap(B * Hkv * pl.a.row_tiles)
                                                               : cdiv(2 * sm_count(), B * Hkv * pl.a.row_tiles)), 256);
  return pl;
}

// ------------------------------------------------------------------------------------------------
// launch
// ------------------------------------------------------------------------------------------------
template <int RT, int KS, int STAGES, bool HAS_B, int MIN_CTAS, bool BF>
static int launch_attn_inst(const AttnParams& p, int n_cta, cudaStream_t stream) {
  constexpr int smem = attn_smem_bytes<(RT > 1 ? RT : 1), STAGES>();
  auto kern = attn_kernel<RT, KS, STAGES, HAS_B, MIN_CTAS, BF>;
  static bool configured = false;   // per instantiation; the attribute is per device function
  static int configured_dev = -1;
  int dev = 0;
  cudaGetDevice(&dev);
  if (!configured || configured_dev != dev) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return check_launch(e);
    configured = true;
    configured_dev = dev;
  }
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(n_cta);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return check_launch(cudaLaunchKernelEx(&cfg, kern, p));
}

template <bool HAS_B, bool BF>
static int launch_attn_dt(const AttnParams& p, int rt, int n_cta, cudaStream_t stream) {
  switch (rt) {
    case 1: return launch_attn_inst<1, 4, 3, HAS_B, 2, BF>(p, n_cta, stream);
    case 2: return launch_attn_inst<2, 4, 3, HAS_B, 2, BF>(p, n_cta, stream);
    case 4: return launch_attn_inst<4, 2, 4, HAS_B, 1, BF>(p, n_cta, stream);
    default: return launch_attn_inst<8, 1, 4, HAS_B, 1, BF>(p, n_cta, stream);
  }
}

template <bool HAS_B>
static int launch_attn(const AttnParams& p, int rt, int n_cta, cudaStream_t stream) {
  return p.bf16 ? launch_attn_dt<HAS_B, true>(p, rt, n_cta, stream) : launch_attn_dt<HAS_B, false>(p, rt, n_cta, stream);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

static void fill_role(AttnRole* r, const RolePlan& pl, uint8_t* ws) {
  r->row_tiles = pl.row_tiles;
  r->MP = pl.MP;
  r->nsplit = pl.nsplit;
  r->split_len = pl.split_len;
  r->n_cta = pl.n_cta;
  r->part_o = reinterpret_cast<float*>(ws + pl.off_o);
  r->part_ml = reinterpret_cast<float*>(ws + pl.off_ml);
}

// Where a call that returns partials instead of the final output puts them: three separate arrays
// (rows), (rows), (rows, 128), or one packed record of 130 floats (m, l, o[128]) per row, the form that
// travels between GPUs in a single exchange.
struct PartialOut {
  float* pm;
  float* pl;
  float* po;
  int ml_stride, o_stride;
  bool any() const { return pm && pl && po; }
};
static PartialOut partial_none() { return PartialOut{nullptr, nullptr, nullptr, 1, kHD}; }
static PartialOut partial_arrays(float* m, float* l, float* o) { return PartialOut{m, l, o, 1, kHD}; }
static PartialOut partial_packed(float* rec) {
  return PartialOut{rec, rec ? rec + 1 : nullptr, rec ? rec + 2 : nullptr, kHD + 2, kHD + 2};
}

// Pages of a paged cache: pool (pages, Hkv, page_size, D) addressed through table (groups, table_stride);
// pages == 0 means the caches are contiguous.
struct PageArgs {
  const int32_t* table;
  int pages, page_size, table_stride;
};

// Describes the role's K/V to TMA: a contiguous (groups, keys, 128) tensor, or the page pool.
static int role_tmaps(AttnRole* r, const void* k, const void* v, int keys, uint64_t groups, int Hkv, const PageArgs& pg) {
  if (pg.pages > 0) {
    if (!pg.table || pg.page_size < kBK || pg.page_size % kBK != 0 || pg.table_stride <= 0 ||
        (long long)pg.table_stride * pg.page_size < keys)
      return VMK_E_BADARG;
    int rc = make_tmap_3d(&r->tmK, k, kHD, pg.page_size, (uint64_t)pg.pages * Hkv, 64, kBK);
    if (rc) return rc;
    rc = make_tmap_3d(&r->tmV, v, kHD, pg.page_size, (uint64_t)pg.pages * Hkv, 64, kBK);
    if (rc) return rc;
    r->page_table = pg.table;
    r->page_size = pg.page_size;
    r->table_stride = pg.table_stride;
    r->page_groups = pg.pages * Hkv;
    return VMK_OK;
  }
  int rc = make_tmap_3d(&r->tmK, k, kHD, keys, groups, 64, kBK);
  if (rc) return rc;
  return make_tmap_3d(&r->tmV, v, kHD, keys, groups, 64, kBK);
}

// pg_a / pg_b: page tables of the shared prefix (one row) and of the private suffixes (one row per request);
// with pages > 0, kp/vp and ks/vs all point at the page pool.
// The library's second stream of a device and the two events that fork it from, and join it to, the caller's
// stream.  Created at the first call that needs them (no device memory involved); calls on one device share
// them, which is correct for any order of calls (every use is bracketed by its own fork and join) but makes the
// suffix kernels of concurrent calls queue behind one another.  Works under stream capture: the fork pulls the
// second stream into the capture and the join hands it back.
struct SideStream {
  cudaStream_t stream;
  cudaEvent_t fork, join;
};
static SideStream* side_stream() {
  static SideStream made[64];
  static bool ready[64] = {false};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!ready[dev]) {
    SideStream s;
    if (cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.fork, cudaEventDisableTiming) != cudaSuccess ||
        cudaEventCreateWithFlags(&s.join, cudaEventDisableTiming) != cudaSuccess) {
      cudaGetLastError();
      return nullptr;                                   // the call then runs its kernels one after the other
    }
    made[dev] = s;
    ready[dev] = true;
  }
  return &made[dev];
}

// q_heads: heads per request in q's memory (the distance between two requests' rows, in heads); Hq when the
// call covers every head, larger when q points at a slice of heads [h0, h0 + Hq) of a wider tensor.
static int prefix_impl(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                       const int32_t* slens, void* out, int N, int Hq, int Hkv, int D, int P, int S, int key_lo,
                       int key_hi, int with_suffix, PartialOut po, void* ws, size_t ws_bytes,
                       int32_t* status, cudaStream_t stream, PageArgs pg_a = PageArgs{nullptr, 0, 0, 0},
                       PageArgs pg_b = PageArgs{nullptr, 0, 0, 0}, int bf16 = 0, int q_heads = 0) {
  if (N <= 0 || Hq <= 0 || Hkv <= 0 || P <= 0 || S < 0) return VMK_E_BADARG;
  if (D != kHD || Hq % Hkv != 0 || Hq / Hkv > 16) return VMK_E_UNSUPPORTED;
  if ((long long)N * (Hq / Hkv) > (1 << 24)) return VMK_E_UNSUPPORTED;
  if (q_heads == 0) q_heads = Hq;
  if (q_heads < Hq) return VMK_E_BADARG;
  if (!q || (key_hi > key_lo && (!kp || !vp)) || (S > 0 && with_suffix && (!ks || !vs)) || (!out && !po.any()) || !ws)
    return VMK_E_BADARG;
  if (!aligned16(q) || !aligned16(kp) || !aligned16(vp) || !aligned16(ks) || !aligned16(vs) || !aligned16(out) ||
      (reinterpret_cast<uintptr_t>(ws) & 255))
    return VMK_E_BADARG;
  if (key_lo < 0 || key_hi > P || key_lo > key_hi) return VMK_E_BADARG;
  const int G = Hq / Hkv;
  const PrefixPlan pl = plan_prefix(N, Hq, Hkv, P, S, key_lo, key_hi, with_suffix != 0);
  if (!pl.has_a && !pl.has_b) return VMK_E_BADARG;      // no keys at all: every row would be empty
  if (ws_bytes < pl.ws_bytes) return VMK_E_WORKSPACE;
  if (pl.a.nsplit + (pl.has_b ? pl.b.nsplit : 0) > kMaxParts) return VMK_E_UNSUPPORTED;   // before any launch

  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.sc = kLog2e / sqrtf((float)D);
  p.status = status;
  p.bf16 = bf16;
  int rc = VMK_OK;
  if (pl.has_a) {
    rc = role_tmaps(&p.a, kp, vp, P, Hkv, Hkv, pg_a);
    if (rc) return rc;
    p.a.q = static_cast<const __half*>(q);
    p.a.n_groups = Hkv; p.a.Hkv = Hkv; p.a.G = G; p.a.Hq = q_heads;
    p.a.rows_outer = N;
    p.a.klen = P; p.a.key_lo = key_lo; p.a.key_hi = key_hi;
    p.a.mask_start = INT_MAX;
    fill_role(&p.a, pl.a, static_cast<uint8_t*>(ws));
  }
  if (pl.has_b) {
    rc = role_tmaps(&p.b, ks, vs, S, (uint64_t)N * Hkv, Hkv, pg_b);
    if (rc) return rc;
    p.b.q = static_cast<const __half*>(q);
    p.b.klens = slens;
    p.b.n_groups = N * Hkv; p.b.Hkv = Hkv; p.b.G = G; p.b.Hq = q_heads;
    p.b.rows_outer = 1;
    p.b.klen = S; p.b.key_lo = 0; p.b.key_hi = S;
    p.b.mask_start = INT_MAX;
    fill_role(&p.b, pl.b, static_cast<uint8_t*>(ws));
  }
  if (pl.has_a && pl.has_b) {
    if (pl.a.tc) {
      // shared prefix on the tensor-memory kernel, private suffixes on the warp-level kernel
      AttnParams ps = p;
      ps.a = p.b;
      SideStream* side = pl.side_by_side ? side_stream() : nullptr;
      if (side != nullptr) {
        // fork: the suffix streams go to the library's second stream and fill whatever SMs the prefix tiles leave
        if (cudaEventRecord(side->fork, stream) != cudaSuccess || cudaStreamWaitEvent(side->stream, side->fork, 0) != cudaSuccess)
          return check_launch(cudaGetLastError());
        rc = launch_attn_tc(p, pl.a.n_cta, stream);
        if (rc) return rc;
        rc = launch_attn<false>(ps, 1, pl.b.n_cta, side->stream);
        if (rc) return rc;
        if (cudaEventRecord(side->join, side->stream) != cudaSuccess || cudaStreamWaitEvent(stream, side->join, 0) != cudaSuccess)
          return check_launch(cudaGetLastError());
      } else {
        rc = launch_attn_tc(p, pl.a.n_cta, stream);
        if (rc) return rc;
        rc = launch_attn<false>(ps, 1, pl.b.n_cta, stream);
      }
    } else {
      rc = launch_attn<true>(p, pl.a.rt, pl.a.n_cta + pl.b.n_cta, stream);
    }
  } else if (pl.has_a) {
    rc = pl.a.tc ? launch_attn_tc(p, pl.a.n_cta, stream) : launch_attn<false>(p, pl.a.rt, pl.a.n_cta, stream);
  } else {
    AttnParams ps = p;
    ps.a = p.b;
    rc = launch_attn<false>(ps, 1, pl.b.n_cta, stream);
  }
  if (rc) return rc;

  CombineParams c;
  memset(&c, 0, sizeof(c));
  if (pl.has_a) c.a = CombineSide{p.a.part_o, p.a.part_ml, pl.a.nsplit, pl.a.MP, N};
  c.has_b = pl.has_b ? 1 : 0;
  if (pl.has_b) c.b = CombineSide{p.b.part_o, p.b.part_ml, pl.b.nsplit, pl.b.MP, 1};
  c.Hkv = Hkv; c.G = G; c.Hq = Hq;
  c.out = static_cast<__half*>(out);
  c.bf16 = bf16;
  c.pm = po.pm; c.pl = po.pl; c.po = po.po;
  c.ml_stride = po.ml_stride; c.o_stride = po.o_stride;
  return launch_combine(c, N * Hq, stream);
}

static int spec_impl(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words, void* out,
                     int B, int kd, int Hq, int Hkv, int D, int L, int key_lo, int key_hi, PartialOut po,
                     void* ws, size_t ws_bytes, int32_t* status, cudaStream_t stream,
                     PageArgs pg = PageArgs{nullptr, 0, 0, 0}, int bf16 = 0, const int32_t* klens = nullptr,
                     int mask_start = -1) {
  // mask_start: first position of k, v that is a draft (subject to `bits`); -1 = L - kd, the tensor ends with the
  // drafts.  A value >= L says the tensor is a slice of a longer cache whose drafts lie elsewhere: nothing is masked.
  if (mask_start < 0) mask_start = L - kd;
  if (mask_start < L && mask_start != L - kd) return VMK_E_BADARG;
  // klens (B): per-request cache lengths.  Only without a draft mask (bits == nullptr, kd == 1: plain decode),
  // because the mask is anchored at the common length L.
  if (klens != nullptr && (bits != nullptr || kd != 1)) return VMK_E_UNSUPPORTED;
  if (B <= 0 || kd <= 0 || Hq <= 0 || Hkv <= 0 || L <= 0 || bits_words <= 0) return VMK_E_BADARG;
  if (D != kHD || Hq % Hkv != 0 || Hq / Hkv > 16) return VMK_E_UNSUPPORTED;
  if ((mask_start < L && kd > L) || kd > VMK_SPEC_MAX_DRAFTS || kd > 32 * bits_words || bits_words > kMaxMaskWords)
    return VMK_E_UNSUPPORTED;
  if (!q || !k || !v || (!bits && !klens) || (!out && !po.any()) || !ws) return VMK_E_BADARG;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || (reinterpret_cast<uintptr_t>(bits) & 3) ||
      (reinterpret_cast<uintptr_t>(ws) & 255))
    return VMK_E_BADARG;
  if (key_lo < 0 || key_hi > L || key_lo > key_hi) return VMK_E_BADARG;
  const int G = Hq / Hkv;
  const SpecPlan pl = plan_spec(B, kd, Hq, Hkv, key_lo, key_hi);
  if (ws_bytes < pl.ws_bytes) return VMK_E_WORKSPACE;
  if (pl.a.nsplit > kMaxParts) return VMK_E_UNSUPPORTED;            // before any launch

  AttnParams p;
  memset(&p, 0, sizeof(p));
  p.sc = kLog2e / sqrtf((float)D);
  p.status = status;
  p.bf16 = bf16;
  int rc = role_tmaps(&p.a, k, v, L, (uint64_t)B * Hkv, Hkv, pg);
  if (rc) return rc;
  p.a.q = static_cast<const __half*>(q);
  p.a.out = static_cast<__half*>(out);
  p.a.bits = bits;
  p.a.bits_words = bits_words;
  p.a.n_groups = B * Hkv; p.a.Hkv = Hkv; p.a.G = G; p.a.Hq = Hq;
  p.a.rows_outer = kd;
  p.a.klen = L; p.a.key_lo = key_lo; p.a.key_hi = key_hi;
  p.a.mask_start = (bits && mask_start < L) ? mask_start : INT_MAX;
  p.a.klens = klens;
  fill_role(&p.a, pl.a, static_cast<uint8_t*>(ws));
  p.a.direct = (out != nullptr && pl.a.nsplit == 1 && key_hi > key_lo) ? 1 : 0;
  rc = pl.a.tc ? launch_attn_tc(p, pl.a.n_cta, stream) : launch_attn<false>(p, pl.a.rt, pl.a.n_cta, stream);
  if (rc || p.a.direct) return rc;

  CombineParams c;
  memset(&c, 0, sizeof(c));
  c.a = CombineSide{p.a.part_o, p.a.part_ml, pl.a.nsplit, pl.a.MP, kd};
  c.Hkv = Hkv; c.G = G; c.Hq = Hq;
  c.out = static_cast<__half*>(out);
  c.bf16 = bf16;
  c.pm = po.pm; c.pl = po.pl; c.po = po.po;
  c.ml_stride = po.ml_stride; c.o_stride = po.o_stride;
  return launch_combine(c, B * kd * Hq, stream);
}

}  // namespace vmk

// ------------------------------------------------------------------------------------------------
// C ABI
// ------------------------------------------------------------------------------------------------
using namespace vmk;

#ifdef VMK_ATTN_TIMING
extern "C" VMK_API int vmk_debug_attn_marks(long long* out) {
  cudaDeviceSynchronize();
  return (int)cudaMemcpyFromSymbol(out, g_attn_marks, sizeof(g_attn_marks));
}
#endif

// 1: results of a row (a request's output) are bit-identical whatever else is in the batch, for every op of the
// library, at the price of speed (fixed kernels, layouts and cut points instead of ones chosen for the batch).
extern "C" VMK_API int vmk_set_batch_invariant(int on) {
  g_batch_invariant = on ? 1 : 0;
  return VMK_OK;
}

// A/B switch: 1 = a prefix call with a large suffix volume runs its prefix tiles (one wave on two thirds of the
// SMs) and its suffix streams at the same time on two streams (default), 0 = one after the other.
extern "C" VMK_API int vmk_prefix_set_side_by_side(int on) {
  g_side_by_side = on ? 1 : 0;
  return VMK_OK;
}

// Test hook: 1 = row tiles of 128 use the tcgen05 kernel (default), 0 = warp-level kernel everywhere.
extern "C" VMK_API int vmk_attn_set_tc(int on) {
  g_attn_tc = on ? 1 : 0;
  return VMK_OK;
}

extern "C" size_t vmk_prefix_workspace_bytes(int N, int Hq, int Hkv, int D, int P, int S) {
  if (N <= 0 || Hq <= 0 || Hkv <= 0 || P <= 0 || S < 0 || D != kHD || Hq % Hkv != 0) return 0;
  const PrefixPlan pl = plan_prefix(N, Hq, Hkv, P, S, 0, P, true);
  if (pl.a.nsplit + (pl.has_b ? pl.b.nsplit : 0) > kMaxParts) return 0;       // the call would refuse this shape
  return pl.ws_bytes;
}

extern "C" int vmk_prefix_decode(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                                 const int32_t* slens, void* out, int N, int Hq, int Hkv, int D, int P, int S,
                                 void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!out) return VMK_E_BADARG;
  return prefix_impl(q, kp, vp, ks, vs, slens, out, N, Hq, Hkv, D, P, S, 0, P, 1, partial_none(), ws,
                     ws_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" int vmk_prefix_decode_paged(const void* q, const void* k_pages, const void* v_pages, int pages, int page_size,
                                       const int32_t* prefix_table, int prefix_pages, const int32_t* suffix_table,
                                       int suffix_stride, const int32_t* slens, void* out, int N, int Hq, int Hkv, int D,
                                       int P, int S, int bf16, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!out || pages <= 0 || !prefix_table || (S > 0 && (!suffix_table || !slens)) || (bf16 != 0 && bf16 != 1))
    return VMK_E_BADARG;
  return prefix_impl(q, k_pages, v_pages, k_pages, v_pages, slens, out, N, Hq, Hkv, D, P, S, 0, P, 1, partial_none(), ws, ws_bytes, status, static_cast<cudaStream_t>(stream),
                     PageArgs{prefix_table, pages, page_size, prefix_pages},
                     PageArgs{suffix_table, pages, page_size, suffix_stride}, bf16);
}

extern "C" int vmk_prefix_partial(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                                  const int32_t* slens, int N, int Hq, int Hkv, int D, int P, int S, int key_lo,
                                  int key_hi, int with_suffix, float* part_m, float* part_l, float* part_o, void* ws,
                                  size_t ws_bytes, int32_t* status, void* stream) {
  if (!part_m || !part_l || !part_o) return VMK_E_BADARG;
  return prefix_impl(q, kp, vp, ks, vs, slens, nullptr, N, Hq, Hkv, D, P, S, key_lo, key_hi, with_suffix,
                     partial_arrays(part_m, part_l, part_o), ws, ws_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" size_t vmk_spec_workspace_bytes(int B, int kd, int Hq, int Hkv, int D, int L) {
  if (B <= 0 || kd <= 0 || Hq <= 0 || Hkv <= 0 || L <= 0 || D != kHD || Hq % Hkv != 0) return 0;
  const SpecPlan pl = plan_spec(B, kd, Hq, Hkv, 0, L);
  if (pl.a.nsplit > kMaxParts) return 0;                                       // the call would refuse this shape
  return pl.ws_bytes;
}

extern "C" int vmk_spec_verify(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                               void* out, int B, int kd, int Hq, int Hkv, int D, int L, void* ws, size_t ws_bytes,
                               int32_t* status, void* stream) {
  if (!out) return VMK_E_BADARG;
  return spec_impl(q, k, v, bits, bits_words, out, B, kd, Hq, Hkv, D, L, 0, L, partial_none(), ws,
                   ws_bytes, status, static_cast<cudaStream_t>(stream));
}

extern "C" int vmk_spec_verify_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* page_table,
                                     int pages, int page_size, int table_stride, const uint32_t* bits, int bits_words,
                                     void* out, int B, int kd, int Hq, int Hkv, int D, int L, int bf16, void* ws,
                                     size_t ws_bytes, int32_t* status, void* stream) {
  if (!out || pages <= 0 || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  return spec_impl(q, k_pages, v_pages, bits, bits_words, out, B, kd, Hq, Hkv, D, L, 0, L, partial_none(), ws,
                   ws_bytes, status, static_cast<cudaStream_t>(stream), PageArgs{page_table, pages, page_size, table_stride},
                   bf16);
}

extern "C" int vmk_spec_partial(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                                int B, int kd, int Hq, int Hkv, int D, int L, int key_lo, int key_hi, float* part_m,
                                float* part_l, float* part_o, void* ws, size_t ws_bytes, int32_t* status,
                                void* stream) {
  if (!part_m || !part_l || !part_o) return VMK_E_BADARG;
  return spec_impl(q, k, v, bits, bits_words, nullptr, B, kd, Hq, Hkv, D, L, key_lo, key_hi,
                   partial_arrays(part_m, part_l, part_o), ws, ws_bytes, status, static_cast<cudaStream_t>(stream));
}

// ---- partials as packed records (m, l, o[128]) of 130 floats per row: what crosses between GPUs ------------
extern "C" int vmk_prefix_partial_packed(const void* q, int q_heads, const void* kp, const void* vp, const void* ks,
                                         const void* vs, const int32_t* slens, int N, int Hq, int Hkv, int D, int P,
                                         int S, int key_lo, int key_hi, int with_suffix, int bf16, float* records,
                                         void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!records || (reinterpret_cast<uintptr_t>(records) & 7) || (bf16 != 0 && bf16 != 1) || q_heads < Hq)
    return VMK_E_BADARG;
  return prefix_impl(q, kp, vp, ks, vs, slens, nullptr, N, Hq, Hkv, D, P, S, key_lo, key_hi, with_suffix,
                     partial_packed(records), ws, ws_bytes, status, static_cast<cudaStream_t>(stream),
                     PageArgs{nullptr, 0, 0, 0}, PageArgs{nullptr, 0, 0, 0}, bf16, q_heads);
}

extern "C" int vmk_spec_partial_packed(const void* q, const void* k, const void* v, const uint32_t* bits,
                                       int bits_words, int B, int kd, int Hq, int Hkv, int D, int L, int key_lo,
                                       int key_hi, int mask_start, int bf16, float* records, void* ws,
                                       size_t ws_bytes, int32_t* status, void* stream) {
  if (!records || (reinterpret_cast<uintptr_t>(records) & 7) || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  return spec_impl(q, k, v, bits, bits_words, nullptr, B, kd, Hq, Hkv, D, L, key_lo, key_hi, partial_packed(records),
                   ws, ws_bytes, status, static_cast<cudaStream_t>(stream), PageArgs{nullptr, 0, 0, 0}, bf16, nullptr,
                   mask_start);
}

// ------------------------------------------------------------------------------------------------
// vmk_spec_verify_noalloc: the same kernels, with the split partials in a buffer that is part of the
// library image instead of caller-provided scratch.
//
// g_spec_scratch is a file-scope device array: every GPU on which this module gets loaded (at the first use of
// one of its kernels or symbols, under the runtime's default lazy loading) reserves these bytes until the
// process exits.  In host code the name is only a handle; the device address comes from
// cudaGetSymbolAddress, taken once per device with that device current.  Every call on a device uses
// the same bytes, which still hold the previous call's partials: the kernels write each partial before
// the combine pass reads it, so nothing has to be cleared -- but two calls whose kernels overlap on the
// GPU (different streams) would overwrite each other's partials.
// ------------------------------------------------------------------------------------------------
static __device__ __align__(256) unsigned char g_spec_scratch[VMK_SPEC_NOALLOC_SCRATCH_BYTES];

static int spec_scratch_address(void** out) {
  static void* cached[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return VMK_E_LAUNCH;
  void* ptr = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (ptr == nullptr) {
    // first call on this device: resolve the array's device address (not to be done during stream capture)
    // (this is also what loads the module, and with it reserves the array, under lazy module loading)
    const cudaError_t e = cudaGetSymbolAddress(&ptr, g_spec_scratch);
    if (e == cudaErrorMemoryAllocation) {
      cudaGetLastError();                               // the failure is reported through the return code
      return VMK_E_NOMEM;
    }
    if (e != cudaSuccess || ptr == nullptr) return VMK_E_LAUNCH;
    __atomic_store_n(&cached[dev], ptr, __ATOMIC_RELEASE);
  }
  *out = ptr;
  return VMK_OK;
}

extern "C" int vmk_spec_verify_noalloc(const void* q, const void* k, const void* v, const uint32_t* bits,
                                       int bits_words, void* out, int B, int kd, int Hq, int Hkv, int D, int L,
                                       int32_t* status, void* stream) {
  if (!out) return VMK_E_BADARG;
  if (B <= 0 || kd <= 0 || Hq <= 0 || Hkv <= 0 || L <= 0 || bits_words <= 0) return VMK_E_BADARG;
  if (D != kHD || Hq % Hkv != 0 || Hq / Hkv > 16) return VMK_E_UNSUPPORTED;
  if (plan_spec(B, kd, Hq, Hkv, 0, L).ws_bytes > (size_t)VMK_SPEC_NOALLOC_SCRATCH_BYTES) return VMK_E_TOO_LARGE;
  void* ws = nullptr;
  const int rc = spec_scratch_address(&ws);
  if (rc) return rc;
  return spec_impl(q, k, v, bits, bits_words, out, B, kd, Hq, Hkv, D, L, 0, L, partial_none(), ws,
                   (size_t)VMK_SPEC_NOALLOC_SCRATCH_BYTES, status, static_cast<cudaStream_t>(stream));
}

extern "C" int vmk_lse_merge(const float* m, const float* l, const float* o, int parts, int rows, int D, void* out,
                             void* stream) {
  if (!m || !l || !o || !out || parts <= 0 || rows <= 0 || D <= 0) return VMK_E_BADARG;
  lse_merge_kernel<<<rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(m, l, o, parts, rows, D,
                                                                          static_cast<__half*>(out), 0);
  return check_launch(cudaGetLastError());
}

extern "C" int vmk_lse_merge_packed(const float* records, int parts, int rows, int D, int bf16, void* out,
                                    void* stream) {
  if (!records || !out || parts <= 0 || rows <= 0 || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  if (D != kHD) return VMK_E_UNSUPPORTED;
  lse_merge_packed_kernel<<<rows, 128, 0, static_cast<cudaStream_t>(stream)>>>(records, parts, rows,
                                                                                  static_cast<__half*>(out), bf16);
  return check_launch(cudaGetLastError());
}

// ---- plain single-token decode: one query per request over its own cache of lens[b] keys ---------------------
extern "C" size_t vmk_decode_workspace_bytes(int B, int Hq, int Hkv, int D, int L) {
  return vmk_spec_workspace_bytes(B, 1, Hq, Hkv, D, L);
}

extern "C" int vmk_decode(const void* q, const void* k, const void* v, const int32_t* lens, void* out, int B, int Hq,
                          int Hkv, int D, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!out || !lens || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  return spec_impl(q, k, v, nullptr, 1, out, B, 1, Hq, Hkv, D, L, 0, L, partial_none(), ws, ws_bytes, status,
                   static_cast<cudaStream_t>(stream), PageArgs{nullptr, 0, 0, 0}, bf16, lens);
}

extern "C" int vmk_decode_paged(const void* q, const void* k_pages, const void* v_pages, const int32_t* page_table,
                                int pages, int page_size, int table_stride, const int32_t* lens, void* out, int B,
                                int Hq, int Hkv, int D, int L, int bf16, void* ws, size_t ws_bytes, int32_t* status,
                                void* stream) {
  if (!out || !lens || pages <= 0 || (bf16 != 0 && bf16 != 1)) return VMK_E_BADARG;
  return spec_impl(q, k_pages, v_pages, nullptr, 1, out, B, 1, Hq, Hkv, D, L, 0, L, partial_none(), ws,
                   ws_bytes, status, static_cast<cudaStream_t>(stream),
                   PageArgs{page_table, pages, page_size, table_stride}, bf16, lens);
}

// ---- the same ops on bf16 tensors (q, K, V and out) --------------------------------------------------------
extern "C" int vmk_prefix_decode_bf16(const void* q, const void* kp, const void* vp, const void* ks, const void* vs,
                                      const int32_t* slens, void* out, int N, int Hq, int Hkv, int D, int P, int S,
                                      void* ws, size_t ws_bytes, int32_t* status, void* stream) {
  if (!out) return VMK_E_BADARG;
  return prefix_impl(q, kp, vp, ks, vs, slens, out, N, Hq, Hkv, D, P, S, 0, P, 1, partial_none(), ws,
                     ws_bytes, status, static_cast<cudaStream_t>(stream), PageArgs{nullptr, 0, 0, 0},
                     PageArgs{nullptr, 0, 0, 0}, 1);
}

extern "C" int vmk_spec_verify_bf16(const void* q, const void* k, const void* v, const uint32_t* bits, int bits_words,
                                    void* out, int B, int kd, int Hq, int Hkv, int D, int L, void* ws, size_t ws_bytes,
                                    int32_t* status, void* stream) {
  if (!out) return VMK_E_BADARG;
  return spec_impl(q, k, v, bits, bits_words, out, B, kd, Hq, Hkv, D, L, 0, L, partial_none(), ws,
                   ws_bytes, status, static_cast<cudaStream_t>(stream), PageArgs{nullptr, 0, 0, 0}, 1);
}
