#include "common.cuh"
using namespace bsir;
extern "C" int64_t bsir_matmul_w8a8_workspace_bytes(int64_t, int64_t, int64_t, int32_t) { return 0; }
extern "C" int32_t bsir_matmul_w8a8(int64_t, int64_t, int64_t, const int8_t *, int64_t, const int8_t *, int64_t,
                                    int32_t, const float *, const float *, int32_t, void *, int64_t, int32_t *,
                                    void *, int64_t, void *) {
  return fail(BSIR_ERR_UNSUPPORTED, "matmul_w8a8: not built yet");
}
