// `dsa` stage 1 on the 5th-generation tensor cores (tcgen05 + TMEM).  Placeholder until the kernel
// lands: the entry reports the variant as unsupported so that callers fall back to nothing silently.
#include "common.cuh"

namespace vmk {

int indexer_tc_launch(const CUtensorMap&, const CUtensorMap&, const float*, const int32_t*, float*, int, int, int32_t*,
                      cudaStream_t) {
  return VMK_E_UNSUPPORTED;
}

}  // namespace vmk
