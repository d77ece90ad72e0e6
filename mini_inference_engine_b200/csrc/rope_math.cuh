// The rotate-half rotation of eight pairs at once (bfloat16, 16-byte pieces): lo holds dimensions j .. j+7 of a
// head, hi the dimensions half a rotary width further; cs / sn point at the cosines and sines of pair j of the
// token's position (float32).  out_lo = lo cos - hi sin, out_hi = hi cos + lo sin, rounded to bfloat16 once
// (inference_engine/model.py:56-69).
#pragma once
#include <cuda_bf16.h>

__device__ __forceinline__ void rotate8(const uint4& lo, const uint4& hi, const float* cs, const float* sn, uint4& out_lo, uint4& out_hi) {
    const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&lo);
    const __nv_bfloat162* b = reinterpret_cast<const __nv_bfloat162*>(&hi);
    __nv_bfloat162* oa = reinterpret_cast<__nv_bfloat162*>(&out_lo);
    __nv_bfloat162* ob = reinterpret_cast<__nv_bfloat162*>(&out_hi);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 x = __bfloat1622float2(a[j]), y = __bfloat1622float2(b[j]);
        const float c0 = cs[2 * j], c1 = cs[2 * j + 1], s0 = sn[2 * j], s1 = sn[2 * j + 1];
        oa[j] = __floats2bfloat162_rn(x.x * c0 - y.x * s0, x.y * c1 - y.y * s1);
        ob[j] = __floats2bfloat162_rn(y.x * c0 + x.x * s0, y.y * c1 + x.y * s1);
    }
}
