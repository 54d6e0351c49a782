// Launch interface of the tcgen05 sparse-MLA stage (dsa stage 3), shared by dsa.cu and dsa_mla_tc.cu.
#pragma once

#include "common.cuh"

namespace vmk {

struct MlaTcParams {
  CUtensorMap tmKV;    // the latent rows as a 2-D tensor (576 columns, every row of every request or page), box
                       // (64 columns, 1 row), 128-byte swizzle: the source of the TMA row gather
  CUtensorMap tmQ;     // the queries as (576, 128, B), box (64, 64, 1), 128-byte swizzle: staged through the ring
  const __half* q;
  const __half* kv;
  const int32_t* idx;
  const int32_t* cnt;
  __half* out;
  float* part_o;       // (((cta * 2 + k) * 64 + column / 4) * 128 + head) * 4: k = 0 the CTA's first unit, 1 its last
  float* part_ml;      // ((cta * 2 + k) * 128 + head) * 2
  int B, L, ncta;
  int rows_total;      // rows of the tensor tmKV describes: B * L, or pages * page_size
  int gather_tma;      // 0: rows gathered by cp.async from four warps (default); 1: by TMA (tile::gather4)
  float sc;
  int32_t* status;
  int bf16;            // q, kv and out are bf16 instead of fp16
  const int32_t* page_table;   // paged cache: row l of request b is row l % page_size of page
                               // page_table[b * table_stride + l / page_size] of kv = (pages, page_size, 576); null = (B, L, 576)
  int page_size, table_stride, pages;
};

int mla_tc_launch(const MlaTcParams& p, float* workspace, cudaStream_t stream);
size_t mla_tc_workspace(int B);

// The same stage by clusters of two CTAs per request that share the score product (dsa_mla_pair.cu).  Uses q, kv,
// idx, cnt, out, tmQ and the paging fields; part_o is then (((cluster * 2 + k) * 128 + column / 4) * 128 + head) * 4.
int mla_pair_launch(const MlaTcParams& p, float* workspace, cudaStream_t stream);
size_t mla_pair_workspace(int B);

// Tiled tensor map over a 16-bit tensor viewed as (rows, width) with `width` contiguous, box (64, 1), 128-byte
// swizzle: rows are fetched four at a time by cp.async.bulk.tensor ... tile::gather4.  Returns 0 or a VMK_E_* code.
int make_tmap_rows(CUtensorMap* tm, const void* base, uint64_t width, uint64_t rows);

}  // namespace vmk
