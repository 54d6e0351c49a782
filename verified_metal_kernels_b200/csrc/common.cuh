// Shared device/host helpers for the sm_100a kernels: PTX wrappers (mbarrier, TMA, ldmatrix, mma,
// tcgen05), tensor-map construction and the status codes of the C ABI.
#pragma once

#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/vmk_b200.h"

namespace vmk {

constexpr float kLog2e = 1.4426950408889634f;
constexpr uint32_t kSpinLimit = 1u << 22;   // bound on every mbarrier wait; exceeded => status word set

// Bits of the device status word (written with atomicOr; 0 means clean).
constexpr int kStatusTimeout = 1;     // a bounded wait ran out
constexpr int kStatusBadIndex = 2;    // an index outside its tensor was clamped

// ------------------------------------------------------------------------------------------------
// shared-memory addresses, mbarrier
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init() {
  asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// Orders generic-proxy shared-memory accesses against async-proxy (TMA / tcgen05) accesses.
__device__ __forceinline__ void fence_proxy_async() {
  asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
               : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}

// Bounded wait.  Returns false when the limit ran out; the caller records kStatusTimeout and winds down.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  for (uint32_t i = 0; i < kSpinLimit; ++i) {
    if (mbar_try_wait(bar, parity)) return true;
  }
  return false;
}

__device__ __forceinline__ void report(int32_t* status, int bit) {
  if (status != nullptr) atomicOr(status, bit);
}

// ------------------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), never with cluster multicast
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tm) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(tm) : "memory");
}

// The innermost coordinate x must make x * element_size a multiple of 16 bytes; every caller passes
// 0 or a multiple of 64 fp16 elements.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* tm, int x, int y, int z, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z)
      : "memory");
}

// Prefetch of one box into L2 (no shared memory, no barrier): a hint that starts the HBM read early.
__device__ __forceinline__ void tma_prefetch_3d(const CUtensorMap* tm, int x, int y, int z) {
  asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global.tile [%0, {%1, %2, %3}];" ::"l"(tm), "r"(x), "r"(y), "r"(z)
               : "memory");
}

// Programmatic dependent launch.  pdl_wait: block until every grid this one depends on has completed and its
// writes are visible (returns at once when the launch was an ordinary one).  pdl_release: allow the grid
// launched after this one with programmatic stream serialisation to start being scheduled.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* dst, const CUtensorMap* tm, int x, int y, uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Row gather: four rows y0..y3 of a 2-D tensor (box (64 x 16-bit, 1)), columns [x, x + 64), land as four
// consecutive 128-byte rows at dst (512-byte aligned, swizzled by address like any other TMA tile); a row
// coordinate outside the tensor is filled with zeros.  x * 2 must be a multiple of 16 bytes: callers pass
// multiples of 64.  No cluster multicast.
__device__ __forceinline__ void tma_gather4(void* dst, const CUtensorMap* tm, int x, int y0, int y1, int y2, int y3,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes"
      " [%0], [%1, {%3, %4, %5, %6, %7}], [%2];"
      ::"r"(smem_u32(dst)), "l"(tm), "r"(smem_u32(bar)), "r"(x), "r"(y0), "r"(y1), "r"(y2), "r"(y3)
      : "memory");
}

// ------------------------------------------------------------------------------------------------
// cp.async (16-byte, zero-fill when src_bytes == 0), ldmatrix, mma.sync
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(dst)), "l"(src), "r"(src_bytes)
               : "memory");
}
// This thread's arrival on `bar` happens when all its cp.async copies so far have landed (the arrival is one of the
// barrier's expected ones: .noinc).
__device__ __forceinline__ void cp_async_arrive_noinc(uint64_t* bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}

// D(16x8,f32) += A(16x16,f16,row) * B(16x8,f16,col)
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// The same with bf16 operands.
__device__ __forceinline__ void mma_16816_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}

// Two fp32 -> one 32-bit word of bf16 (round to nearest even), low element first.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// One fp32 -> the 16 bits of an fp16 or bf16 value, stored through a __half* (the library's type for "16 bits").
__device__ __forceinline__ void store16(__half* dst, float x, int bf16) {
  *reinterpret_cast<uint16_t*>(dst) = (uint16_t)(bf16 ? pack_bf16x2(x, 0.f) : pack_half2(x, 0.f));
}

// The 16-bit type of a call's tensors: fp16 (the reference's) or bf16.
__device__ __forceinline__ uint32_t pack2(float lo, float hi, int bf16) {
  return bf16 ? pack_bf16x2(lo, hi) : pack_half2(lo, hi);
}

// Byte offset of the 16-byte chunk `chunk` (0..7) of row `row` inside a [rows][128 B] tile written by
// TMA with CU_TENSOR_MAP_SWIZZLE_128B (tile base 1024-byte aligned): chunk index XOR (row mod 8).
__device__ __forceinline__ uint32_t swz128(uint32_t row, uint32_t chunk) {
  return row * 128u + ((chunk ^ (row & 7u)) << 4);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Order-preserving 32-bit key of an fp32 score (larger score = larger key); NaN ranks last and the two
// zeros share a key.  Used by the dsa indexer's fused histogram and by the top-k select.
__device__ __forceinline__ uint32_t score_key(float x) {
  if (x != x) return 0u;
  const uint32_t u = __float_as_uint(x + 0.0f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
constexpr int kSelBins = 2048;        // first radix level: the top 11 bits of the key
constexpr int kSelShift = 21;

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
// Tiled tensor map over an fp16 tensor viewed as (groups, rows, width) with `width` contiguous:
// box = (box_w, box_rows, 1), 128-byte swizzle, out-of-range elements read as zero.
// Returns 0 or a VMK_E_* code.
int make_tmap_3d(CUtensorMap* tm, const void* base, uint64_t width, uint64_t rows, uint64_t groups,
                 uint32_t box_w, uint32_t box_rows);
int make_tmap_3d_u8(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t groups, uint32_t box_rows);

int sm_count();

// 1: every planner cuts the work the same way whatever the batch holds (vmk_set_batch_invariant); defined in attn.cu
extern int g_batch_invariant;
int check_launch(cudaError_t e);

inline int cdiv(int a, int b) { return (a + b - 1) / b; }

}  // namespace vmk
