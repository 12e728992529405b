// Four consecutive elements at once (16 bytes of float32, 8 bytes of bfloat16), as float32.
#pragma once

#include "common.cuh"

namespace somi {

struct F4 { float v[4]; };
__device__ __forceinline__ F4 load4(const float* p) {
    const float4 t = *reinterpret_cast<const float4*>(p);
    return F4{{t.x, t.y, t.z, t.w}};
}
__device__ __forceinline__ F4 load4(const __nv_bfloat16* p) {
    const uint2 t = *reinterpret_cast<const uint2*>(p);
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&t.x);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&t.y);
    return F4{{__low2float(a), __high2float(a), __low2float(b), __high2float(b)}};
}
__device__ __forceinline__ void store4(float* p, const F4& f) {
    *reinterpret_cast<float4*>(p) = make_float4(f.v[0], f.v[1], f.v[2], f.v[3]);
}
__device__ __forceinline__ void store4(__nv_bfloat16* p, const F4& f) {
    __nv_bfloat162 a = __floats2bfloat162_rn(f.v[0], f.v[1]);
    __nv_bfloat162 b = __floats2bfloat162_rn(f.v[2], f.v[3]);
    uint2 t;
    t.x = *reinterpret_cast<uint32_t*>(&a);
    t.y = *reinterpret_cast<uint32_t*>(&b);
    *reinterpret_cast<uint2*>(p) = t;
}
__device__ __forceinline__ F4 load4_any(const void* p, int dtype, size_t i) {
    return dtype == SOMI_F32 ? load4(reinterpret_cast<const float*>(p) + i)
                             : load4(reinterpret_cast<const __nv_bfloat16*>(p) + i);
}

}  // namespace somi
