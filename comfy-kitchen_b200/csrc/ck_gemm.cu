// placeholder until the tcgen05 GEMMs land
#include "ck_common.cuh"
extern "C" int ck_scaled_mm_nvfp4(const void*, const void*, const void*, const void*, const float*, const float*,
                                  const float*, const void*, int, void*, int, int64_t, int64_t, int64_t, void*) {
  return ck::fail(CK_ERR_UNSUPPORTED, "scaled_mm_nvfp4: not built yet");
}
extern "C" int ck_scaled_mm_mxfp8(const void*, const void*, const void*, const void*, const void*, int, void*, int,
                                  int64_t, int64_t, int64_t, void*) {
  return ck::fail(CK_ERR_UNSUPPORTED, "scaled_mm_mxfp8: not built yet");
}
