// Declarations shared by the two convolution kernels (tcgen05 implicit GEMM and the direct
// fallback) and the C-ABI dispatch: packed weights, resolved problem geometry, and the fused
// epilogue arithmetic, which must be the same in both kernels.
#pragma once
#include "common.cuh"

struct exb_conv_weights {
    int dtype;        // EXB_F16 or EXB_I8
    int Cout, Cin, kh, kw, group;
    int cout_pad;     // rows of the packed matrix (Cout rounded up to 16)
    int cin_pad;      // channels per tap in the packed matrix (== x's physical channel count / group)
    void* d_w;        // [cout_pad][kh][kw][cin_pad], K-major rows
    float* d_scale;   // [cout_pad] epilogue multiplier (fp16: 1; int8: 1/(wscale*act_scale))
    float* d_bias;    // [cout_pad] zeros when the layer has no bias
    int device;
};

namespace exb {

// Problem geometry after validation (all strides physical).
struct ConvGeom {
    int N, H, W, Cin, Cout, cin_stride, cout_stride;
    int kh, kw, sh, sw, pt, pl, OH, OW, group;
    int in_dtype, out_dtype, out2_dtype, has_res, act;
    float out_scale, out2_scale;
};

struct EpiParams {
    const float* scale;
    const float* bias;
    const __half* residual;
    void* y;
    void* y2;
    int out_dtype, out2_dtype, act;
    float out_scale, out2_scale;
    int cout_stride;
};

// v = act(acc * scale + bias + residual)
template <bool kInt8>
__device__ __forceinline__ float epi_value(uint32_t raw, float scale, float bias) {
    const float a = kInt8 ? (float)(int)raw : __uint_as_float(raw);
    return fmaf(a, scale, bias);
}

__device__ __forceinline__ void epi_store_scalar(void* y, int dtype, int64_t off, float v, float qscale,
                                                 uint32_t raw) {
    switch (dtype) {
    case EXB_F16: static_cast<__half*>(y)[off] = __float2half_rn(v); break;
    case EXB_I8: static_cast<int8_t*>(y)[off] = (int8_t)quant_rne(v * qscale); break;
    case EXB_F32: static_cast<float*>(y)[off] = v; break;
    case EXB_I32: static_cast<int32_t*>(y)[off] = (int32_t)raw; break;
    default: break;
    }
}

// Four floats -> four int8 (round half to even, saturate), packed little-endian in 32 bits.
__device__ __forceinline__ uint32_t quant_pack4(float a, float b, float c, float d, float qscale) {
    const int q0 = __float2int_rn(a * qscale), q1 = __float2int_rn(b * qscale);
    const int q2 = __float2int_rn(c * qscale), q3 = __float2int_rn(d * qscale);
    uint32_t r;
    // cvt.pack.sat.s8.s32.b32 d, a, b, c:  d = (c << 16) | (sat8(a) << 8) | sat8(b)
    asm("{\n\t.reg .b32 t;\n\t"
        "cvt.pack.sat.s8.s32.b32 t, %4, %3, 0;\n\t"
        "cvt.pack.sat.s8.s32.b32 %0, %2, %1, t;\n\t}"
        : "=r"(r)
        : "r"(q0), "r"(q1), "r"(q2), "r"(q3));
    return r;
}

// 16 consecutive channels starting at element offset `off` (16-byte aligned for every dtype).
__device__ __forceinline__ void epi_store_vec16(void* y, int dtype, int64_t off, const float (&v)[16],
                                                float qscale, const uint32_t (&raw)[16]) {
    if (dtype == EXB_I8) {
        uint4 o;
        o.x = quant_pack4(v[0], v[1], v[2], v[3], qscale);
        o.y = quant_pack4(v[4], v[5], v[6], v[7], qscale);
        o.z = quant_pack4(v[8], v[9], v[10], v[11], qscale);
        o.w = quant_pack4(v[12], v[13], v[14], v[15], qscale);
        *reinterpret_cast<uint4*>(static_cast<int8_t*>(y) + off) = o;
    } else if (dtype == EXB_F16) {
        uint4 o[2];
        __half2* h = reinterpret_cast<__half2*>(o);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        uint4* dst = reinterpret_cast<uint4*>(static_cast<__half*>(y) + off);
        dst[0] = o[0];
        dst[1] = o[1];
    } else if (dtype == EXB_F32) {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(y) + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    } else {
        uint4* dst = reinterpret_cast<uint4*>(static_cast<int32_t*>(y) + off);
#pragma unroll
        for (int i = 0; i < 4; ++i) dst[i] = make_uint4(raw[4 * i], raw[4 * i + 1], raw[4 * i + 2], raw[4 * i + 3]);
    }
}

// Activation over a register vector with the selector hoisted out of the element loop.
__device__ __forceinline__ void act_vec16(float (&v)[16], int act) {
    if (act == EXB_ACT_RELU) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
    } else if (act != EXB_ACT_NONE) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = apply_act(v[i], act);
    }
}

int conv_direct_launch(exb_ctx* ctx, const ConvGeom& g, const void* x, const exb_conv_weights* w,
                       const void* residual, void* y, void* y2, cudaStream_t st);
int conv_tc_launch(exb_ctx* ctx, const ConvGeom& g, const void* x, const exb_conv_weights* w,
                   const void* residual, void* y, void* y2, cudaStream_t st);
// True when the tcgen05 kernel can run this geometry.
bool conv_tc_eligible(const ConvGeom& g);

}  // namespace exb
