// Library-wide pieces of the C ABI: error reporting, version, compiled-in tables.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "luts.inc"

namespace b200 {

static const int32_t h_inv_sqrt_lut[1024] = {B200_LUT_kInvSqrtLut};
static const int32_t h_exp2_silu_lut[1024] = {B200_LUT_kExp2SiluLut};
static const int32_t h_exp2_attn_lut[1024] = {B200_LUT_kExp2AttnLut};

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

bool pdl_enabled() {
  static const int on = [] {
    const char* v = getenv("B200_PDL");
    return (v != nullptr && v[0] == '0') ? 0 : 1;
  }();
  return on != 0;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return B200_E_CUDA;
  }
  return B200_OK;
}

}  // namespace b200

extern "C" int b200_version(void) { return 100; }

extern "C" const char* b200_last_error_string(void) { return b200::g_err; }

extern "C" int b200_get_lut(int which, int32_t* out_host_1024) {
  B200_REQUIRE(out_host_1024, B200_E_NULL, "get_lut: null pointer");
  const int32_t* src = which == 0   ? b200::h_inv_sqrt_lut
                       : which == 1 ? b200::h_exp2_silu_lut
                       : which == 2 ? b200::h_exp2_attn_lut
                                    : nullptr;
  B200_REQUIRE(src, B200_E_SHAPE, "get_lut: which=%d (0, 1 or 2)", which);
  memcpy(out_host_1024, src, 1024 * sizeof(int32_t));
  return B200_OK;
}
