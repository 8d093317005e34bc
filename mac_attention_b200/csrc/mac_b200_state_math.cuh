// Device helpers shared by the prefill-side kernels: streaming 16-byte
// loads/stores, LSE element access in the
// three element types the reference accepts, bf16 pair packing, and the scalar
// part of the LSE downdate.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "mac_b200_common.h"

namespace mac_b200 {

__device__ __forceinline__ uint4 ld_stream16(const void* p) {
  uint4 v;
  asm volatile("ld.global.cs.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
  asm volatile("st.global.cs.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

__device__ __forceinline__ float load_lse(const void* p, int dt, int64_t i) {
  if (dt == MAC_B200_LSE_F32) return static_cast<const float*>(p)[i];
  if (dt == MAC_B200_LSE_F16) return __half2float(static_cast<const __half*>(p)[i]);
  return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
}
__device__ __forceinline__ void store_lse(void* p, int dt, int64_t i, float v) {
  if (dt == MAC_B200_LSE_F32) static_cast<float*>(p)[i] = v;
  else if (dt == MAC_B200_LSE_F16) static_cast<__half*>(p)[i] = __float2half_rn(v);
  else static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
__device__ __forceinline__ float lo_f(uint32_t p) { return __uint_as_float(p << 16); }
__device__ __forceinline__ float hi_f(uint32_t p) { return __uint_as_float(p & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// The three scalars of a row (mac_merge_downdate_cache.cu:152-176).
__device__ __forceinline__ void downdate_scalars(float l1, float l2, float& ret_lse, float& t,
                                                 float& scale) {
  const float diff = l2 - l1;
  const float em1 = expm1f(diff);
  const bool last_block = fabsf(em1) <= 1e-7f;
  const bool invalid = (diff > 0.0f) && !last_block;
  if (last_block) {
    ret_lse = -INFINITY; t = 0.f; scale = 0.f;
  } else if (invalid) {
    ret_lse = l1; t = 0.f; scale = 1.f;
  } else {
    const float one_minus = 1.f - expf(diff);
    ret_lse = l1 + logf(fmaxf(one_minus + 1e-7f, 1e-30f));
    t = expf(diff);
    scale = expf(l1 - ret_lse);
  }
}


}  // namespace mac_b200
