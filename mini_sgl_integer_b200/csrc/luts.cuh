// Device copies of the three look-up tables (values in luts.inc, dumped from the reference).
#pragma once
#include <stdint.h>

#include "luts.inc"

namespace b200 {
static __device__ const int32_t g_inv_sqrt_lut[1024] = {B200_LUT_kInvSqrtLut};
static __device__ const int32_t g_exp2_silu_lut[1024] = {B200_LUT_kExp2SiluLut};
static __device__ const int32_t g_exp2_attn_lut[1024] = {B200_LUT_kExp2AttnLut};
}  // namespace b200
