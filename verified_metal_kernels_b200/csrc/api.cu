// Library-wide host helpers: version, error strings, tensor-map encoding through the driver entry
// point (so the library does not link against libcuda), cached device properties.
#include <cudaTypedefs.h>

#include "common.cuh"
#include "dsa_mla_tc.cuh"

namespace vmk {

int check_launch(cudaError_t e) { return e == cudaSuccess ? VMK_OK : VMK_E_LAUNCH; }

int sm_count() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

static PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
  static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
  }
  return fn;
}

int make_tmap_3d(CUtensorMap* tm, const void* base, uint64_t width, uint64_t rows, uint64_t groups, uint32_t box_w,
                 uint32_t box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return VMK_E_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (width * 2) % 16 != 0 || box_w * 2 != 128 || box_rows > 256)
    return VMK_E_BADARG;
  cuuint64_t dims[3] = {width, rows, groups};
  cuuint64_t strides[2] = {width * 2, width * 2 * rows};
  cuuint32_t box[3] = {box_w, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VMK_OK : VMK_E_DRIVER;
}

int make_tmap_rows(CUtensorMap* tm, const void* base, uint64_t width, uint64_t rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return VMK_E_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || (width * 2) % 16 != 0 || rows == 0 || rows > 0x7fffffffull)
    return VMK_E_BADARG;
  cuuint64_t dims[2] = {width, rows};
  cuuint64_t strides[1] = {width * 2};
  cuuint32_t box[2] = {64, 1};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VMK_OK : VMK_E_DRIVER;
}

// The same for a tensor of bytes (fp8): (groups, rows, 128) with one 128-byte swizzled row per tensor row.
int make_tmap_3d_u8(CUtensorMap* tm, const void* base, uint64_t rows, uint64_t groups, uint32_t box_rows) {
  auto fn = encode_fn();
  if (fn == nullptr) return VMK_E_DRIVER;
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0 || box_rows > 256) return VMK_E_BADARG;
  cuuint64_t dims[3] = {128, rows, groups};
  cuuint64_t strides[2] = {128, 128 * rows};
  cuuint32_t box[3] = {128, box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? VMK_OK : VMK_E_DRIVER;
}

}  // namespace vmk

extern "C" int vmk_version(void) { return 100; }

extern "C" const char* vmk_error_string(int code) {
  switch (code) {
    case VMK_OK: return "ok";
    case VMK_E_BADARG: return "bad argument (null or misaligned pointer, or a non-positive dimension)";
    case VMK_E_UNSUPPORTED: return "shape not supported by the sm_100a kernels";
    case VMK_E_WORKSPACE: return "workspace smaller than vmk_<op>_workspace_bytes()";
    case VMK_E_LAUNCH: return "CUDA launch failed";
    case VMK_E_DRIVER: return "tensor-map encoding failed or the driver entry point is missing";
    case VMK_E_TOO_LARGE: return "the problem needs more scratch than the library's built-in static buffer holds";
    case VMK_E_NOMEM: return "no device memory left for the library's static device buffers (load them before the host claims the rest)";
    default: return "unknown error code";
  }
}
