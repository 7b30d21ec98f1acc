#include "common.cuh"
using namespace bsir;
extern "C" int32_t bsir_matmul_w4a16(int64_t, int64_t, int64_t, int64_t, const void *, int64_t, const int32_t *,
                                     const void *, const int32_t *, void *, int64_t, void *) {
  return fail(BSIR_ERR_UNSUPPORTED, "matmul_w4a16: not built yet");
}
