// Quantisation of one 128-value chunk of an activation row into the formats the GEMV consumers
// read (reference: glm53/gfx950/kernel.py:1440-1466 quant_scaled / quant_mxfp8).  Shared by the
// activation staging, the expert activation and the sparse-MLA merge.
#pragma once
#include "mono_common.cuh"

namespace mono {

// position inside a group of 8 values of the MXFP4-ordered activation plane
__device__ __forceinline__ int mx_perm8(int i) { return (i & 1) ? 4 + (i >> 1) : (i >> 1); }

__device__ __forceinline__ void quant_chunk128(const float* x /* smem, 128 values */, int fmt, int lane, int chunk,
                                               uint8_t* plane0, uint8_t* plane1, float* scale_f32, uint8_t* scale_e8) {
    // lane owns values 4*lane .. 4*lane+3
    float v[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) v[i] = x[4 * lane + i];
    if (fmt == MONO_ACT_A8 || fmt == MONO_ACT_HILO) {
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
        amax = warp_max(amax);
        if (fmt == MONO_ACT_A8) {
            const float scale = amax > 0.f ? amax / 448.f : 1.f;
            const float inv = amax > 0.f ? 448.f / amax : 1.f;
            uint32_t w = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) w |= (uint32_t)f32_to_e4m3(v[i] * inv) << (8 * i);
            reinterpret_cast<uint32_t*>(plane0 + chunk * 128)[lane] = w;
            if (lane == 0) scale_f32[chunk] = scale;
        } else {
            const int code = code_ceil(fmaxf(amax, 7.888609052210118e-31f /* 2^-100 */) / 448.f);
            const float sc = exp2_code(code), inv = exp2_code(254 - code);
            uint32_t wh = 0, wl = 0;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float s = v[i] * inv;
                const uint8_t h = f32_to_e4m3(s);
                const uint8_t l = f32_to_e4m3(s - e4m3_to_f32(h));
                wh |= (uint32_t)h << (8 * i);
                wl |= (uint32_t)l << (8 * i);
            }
            reinterpret_cast<uint32_t*>(plane0 + chunk * 128)[lane] = wh;
            reinterpret_cast<uint32_t*>(plane1 + chunk * 128)[lane] = wl;
            if (lane == 0) scale_f32[chunk] = sc;
        }
    } else if (fmt == MONO_ACT_MX8 || fmt == MONO_ACT_MX8N) {
        // four groups of 32: lanes 8q .. 8q+7 own group q
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 4; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        int code = code_ceil(fmaxf(amax, 1e-10f) * (1.0f / 448.0f));
        code = min(max(code, 1), 254);
        const float inv = exp2_code(254 - code);
        // values 4*lane+i sit in group-of-8 number lane/2 at in-group index (lane&1)*4+i
        uint8_t* dst = plane0 + chunk * 128 + (lane >> 1) * 8;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int k8 = (lane & 1) * 4 + i;  // index inside the group of 8
            dst[fmt == MONO_ACT_MX8 ? mx_perm8(k8) : k8] = f32_to_e4m3(v[i] * inv);
        }
        if ((lane & 7) == 0) scale_e8[chunk * 4 + (lane >> 3)] = (uint8_t)code;
    } else if (fmt == MONO_ACT_NVF4) {
        // eight blocks of 16: lanes 4q .. 4q+3 own block q; the scale is an E4M3 byte, never zero
        float amax = fmaxf(fmaxf(fabsf(v[0]), fabsf(v[1])), fmaxf(fabsf(v[2]), fabsf(v[3])));
#pragma unroll
        for (int o = 2; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
        const uint8_t sb = f32_to_e4m3(__fdiv_rn(fmaxf(amax, 0.01171875f /* 6 * 2^-9 */), 6.0f));
        const float sc = e4m3_to_f32(sb);
        uint32_t w = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) w |= f32_to_e2m1(__fdiv_rn(v[i], sc)) << (4 * i);
        reinterpret_cast<uint16_t*>(plane0 + chunk * 64)[lane] = (uint16_t)w;
        if ((lane & 3) == 0) scale_e8[chunk * 8 + (lane >> 2)] = sb;
    } else {  // MONO_ACT_BF16
        __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
        uint2 w = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
        reinterpret_cast<uint2*>(plane0 + chunk * 256)[lane] = w;
    }
}

}  // namespace mono
