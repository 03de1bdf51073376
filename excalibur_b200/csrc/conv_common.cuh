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
    int kw_pack;      // taps per kernel row in the packed matrix: kw, or the fold width F (>= kw)
    int s_shift;      // column of tap s = 0 inside a packed kernel row (0 unless folded)
    void* d_w;        // [cout_pad][kh][kw_pack][cin_pad], K-major rows
    float* d_scale;   // [cout_pad] epilogue multiplier (fp16: 1; int8: 1/(wscale*act_scale))
    float* d_bias;    // [cout_pad] zeros when the layer has no bias
    float* d_slope;   // [cout_pad + kSlopeSlack] PReLU slopes (zero beyond Cout), or null
    float* h_scale;   // host copies of d_scale / d_bias: narrow layers pass them to the kernel as launch parameters
    float* h_bias;
    int device;
};

namespace exb {

// The epilogue reads 16 slopes at any channel offset below the output's channel stride.
constexpr int kSlopeSlack = 1024;

// Problem geometry after validation (all strides physical).
struct ConvGeom {
    int N, H, W, Cin, Cout, cin_stride, cout_stride;
    int kh, kw, sh, sw, pt, pl, OH, OW, group;
    int in_dtype, out_dtype, out2_dtype, has_res, act;
    float out_scale, out2_scale;
    int w_pitch, w_pad;   // physical pixels per input row and zero pixels left of pixel 0 (dense: W, 0)
    int pool;             // 1: 3x3/2 pad-1 max pooling fused into the epilogue; y is [N][PH][PW][cout_stride]
    int PH, PW;
    int y_pitch;                    // elements between output pixels of y (== cout_stride unless y is a slice of a wider tensor)
};

// "Folded" K layout for convolutions with very few input channels (a stem): one K row of an
// output pixel is the contiguous run of F input pixels x cin_stride channels that covers all kw
// taps of one kernel row, so a kernel row is one K block instead of kw tiny ones.  It needs
// physically zero-padded input rows, a W stride that keeps TMA's 16-byte alignment, and weights
// packed [Cout][kh][F][cin_stride] with the taps placed at column `shift`.
struct FoldPlan {
    bool on;
    int F;          // input pixels per K row
    int shift;      // extra zero-weight columns on the left (pl_eff - pad_l)
    int pl_eff;     // left reach of a K row in pixels (>= pad_l)
    int kb_bytes;   // bytes of a K row: 32, 64 or 128
};
inline FoldPlan conv_fold_plan(const ConvGeom& g) {
    FoldPlan f = {false, 0, 0, 0, 0};
    const int px = g.cin_stride * (g.in_dtype == EXB_I8 ? 1 : 2);
    if (g.w_pad <= 0 || g.group != 1 || px >= 32) return f;
    if ((g.sw * px) % 16 != 0 || g.sh != g.sw || (g.sh != 1 && g.sh != 2)) return f;
    int pl_eff = g.pl;
    while (pl_eff <= g.w_pad && ((g.w_pad - pl_eff) * px) % 16 != 0) ++pl_eff;
    if (pl_eff > g.w_pad) return f;
    const int shift = pl_eff - g.pl;
    for (int kb = 32; kb <= 128; kb *= 2) {
        if (kb % px) continue;
        const int F = kb / px;
        if (F < g.kw + shift) continue;
        if ((g.OW - 1) * g.sw - pl_eff + F + g.w_pad > g.w_pitch) return f;   // right padding too short
        f.on = true; f.F = F; f.shift = shift; f.pl_eff = pl_eff; f.kb_bytes = kb;
        return f;
    }
    return f;
}

struct EpiParams {
    const float* scale;
    const float* bias;
    const float* slope;   // EXB_ACT_PRELU only
    const __half* residual;
    void* y;
    void* y2;
    int out_dtype, out2_dtype, act;
    float out_scale, out2_scale;
    int cout_stride;
    int y_pitch;     // elements between output pixels of y / y2
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

// 256-bit global accesses (sm_100): one instruction per 32-byte pixel segment instead of two.
__device__ __forceinline__ void st_global_256(void* p, const uint32_t (&o)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                 "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
}
__device__ __forceinline__ void ld_global_nc_256(const void* p, uint32_t (&o)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                 : "l"(p));
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
        uint32_t o[8];
        __half2* h = reinterpret_cast<__half2*>(o);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        st_global_256(static_cast<__half*>(y) + off, o);   // 32 bytes, 32-byte aligned
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

// 8 consecutive channels starting at element offset `off` (8-byte aligned for every dtype): fp16, int8 or fp32.
__device__ __forceinline__ void epi_store_vec8(void* y, int dtype, int64_t off, const float (&v)[8], float qscale) {
    if (dtype == EXB_I8) {
        uint2 o;
        o.x = quant_pack4(v[0], v[1], v[2], v[3], qscale);
        o.y = quant_pack4(v[4], v[5], v[6], v[7], qscale);
        *reinterpret_cast<uint2*>(static_cast<int8_t*>(y) + off) = o;
    } else if (dtype == EXB_F16) {
        uint4 o;
        __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(static_cast<__half*>(y) + off) = o;
    } else {
        float4* dst = reinterpret_cast<float4*>(static_cast<float*>(y) + off);
        dst[0] = make_float4(v[0], v[1], v[2], v[3]);
        dst[1] = make_float4(v[4], v[5], v[6], v[7]);
    }
}

// Activation over a register vector with the selector hoisted out of the element loop (one uniform
// branch per chunk instead of a switch per element).
__device__ __forceinline__ void prelu_vec16(float (&v)[16], const float* slope) {
    const float4* s4 = reinterpret_cast<const float4*>(slope);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float4 s = __ldg(s4 + i);
        v[4 * i + 0] = v[4 * i + 0] >= 0.f ? v[4 * i + 0] : v[4 * i + 0] * s.x;
        v[4 * i + 1] = v[4 * i + 1] >= 0.f ? v[4 * i + 1] : v[4 * i + 1] * s.y;
        v[4 * i + 2] = v[4 * i + 2] >= 0.f ? v[4 * i + 2] : v[4 * i + 2] * s.z;
        v[4 * i + 3] = v[4 * i + 3] >= 0.f ? v[4 * i + 3] : v[4 * i + 3] * s.w;
    }
}

__device__ __forceinline__ void act_vec16(float (&v)[16], int act) {
    if (act == EXB_ACT_NONE) return;
    if (act == EXB_ACT_RELU) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = fmaxf(v[i], 0.f);
    } else if (act == EXB_ACT_RELU6) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = fminf(fmaxf(v[i], 0.f), 6.f);
    } else if (act == EXB_ACT_SILU) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = v[i] * sigmoid_fast(v[i]);
    } else if (act == EXB_ACT_HARDSWISH) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = v[i] * fminf(fmaxf(fmaf(v[i], 1.f / 6.f, 0.5f), 0.f), 1.f);
    } else if (act == EXB_ACT_SIGMOID) {
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = sigmoid_fast(v[i]);
    } else {
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
// True when the tcgen05 kernel can also apply the 3x3/2 max pooling in its epilogue.
bool conv_tc_pool_fusable(const ConvGeom& g);

}  // namespace exb
