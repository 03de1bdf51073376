// C-ABI front of the dense convolution: descriptor validation, weight packing and the choice
// between the tcgen05 implicit-GEMM kernel and the direct kernel.
#include "conv_common.cuh"

#include <math.h>
#include <string.h>

#include <vector>

namespace exb {
namespace {

int resolve(const exb_conv_desc* d, ConvGeom& g) {
    EXB_REQUIRE(d != nullptr, "null convolution descriptor");
    EXB_REQUIRE(d->N >= 0 && d->H > 0 && d->W > 0 && d->Cin > 0 && d->Cout > 0, "bad convolution shape");
    EXB_REQUIRE(d->kh > 0 && d->kw > 0 && d->stride_h > 0 && d->stride_w > 0, "bad convolution window / stride");
    EXB_REQUIRE(d->pad_t >= 0 && d->pad_b >= 0 && d->pad_l >= 0 && d->pad_r >= 0, "negative pad");
    EXB_REQUIRE(d->group >= 1 && d->Cin % d->group == 0 && d->Cout % d->group == 0,
                "group %d does not divide Cin %d / Cout %d", d->group, d->Cin, d->Cout);
    if (d->dilation != 1 && d->dilation != 0)
        return fail(EXB_ERR_UNSUPPORTED, "dilation %d is not implemented", d->dilation);
    if (d->in_dtype != EXB_F16 && d->in_dtype != EXB_I8)
        return fail(EXB_ERR_UNSUPPORTED, "convolution input dtype %d (EXB_F16 or EXB_I8 expected)", d->in_dtype);
    if (d->out_dtype != EXB_F16 && d->out_dtype != EXB_I8 && d->out_dtype != EXB_F32 &&
        !(d->out_dtype == EXB_I32 && d->in_dtype == EXB_I8))
        return fail(EXB_ERR_UNSUPPORTED, "convolution output dtype %d", d->out_dtype);
    if (d->out2_dtype != -1 && d->out2_dtype != EXB_F16 && d->out2_dtype != EXB_I8)
        return fail(EXB_ERR_UNSUPPORTED, "convolution second output dtype %d", d->out2_dtype);
    if (d->res_dtype != -1 && d->res_dtype != EXB_F16)
        return fail(EXB_ERR_UNSUPPORTED, "convolution residual dtype %d (EXB_F16 expected)", d->res_dtype);
    if (!act_supported(d->act) && d->act != EXB_ACT_PRELU)
        return fail(EXB_ERR_UNSUPPORTED, "activation type %d is not implemented", d->act);
    if (d->act == EXB_ACT_PRELU && d->fuse_pool)
        return fail(EXB_ERR_UNSUPPORTED, "fuse_pool needs an activation with non-negative results, not EXB_ACT_PRELU");
    g.N = d->N; g.H = d->H; g.W = d->W; g.Cin = d->Cin; g.Cout = d->Cout;
    g.cin_stride = d->cin_stride ? d->cin_stride : d->Cin;
    g.cout_stride = d->cout_stride ? d->cout_stride : d->Cout;
    EXB_REQUIRE(g.cin_stride >= g.Cin && g.cout_stride >= g.Cout, "channel stride smaller than channel count");
    EXB_REQUIRE(d->group == 1 || g.cin_stride == g.Cin, "grouped convolution needs unpadded input channels");
    g.kh = d->kh; g.kw = d->kw; g.sh = d->stride_h; g.sw = d->stride_w; g.pt = d->pad_t; g.pl = d->pad_l;
    g.OH = (d->H + d->pad_t + d->pad_b - d->kh) / d->stride_h + 1;
    g.OW = (d->W + d->pad_l + d->pad_r - d->kw) / d->stride_w + 1;
    EXB_REQUIRE(g.OH > 0 && g.OW > 0 && d->H + d->pad_t + d->pad_b >= d->kh && d->W + d->pad_l + d->pad_r >= d->kw,
                "convolution window larger than the padded input");
    g.group = d->group;
    g.in_dtype = d->in_dtype; g.out_dtype = d->out_dtype; g.out2_dtype = d->out2_dtype;
    g.has_res = d->res_dtype != -1;
    g.act = d->act; g.out_scale = d->out_scale; g.out2_scale = d->out2_scale;
    EXB_REQUIRE(d->x_w_pad >= 0 && (d->x_w_pitch == 0 || d->x_w_pitch >= d->W + d->x_w_pad),
                "bad input row padding (x_w_pad %d, x_w_pitch %d, W %d)", d->x_w_pad, d->x_w_pitch, d->W);
    g.w_pitch = d->x_w_pitch ? d->x_w_pitch : d->W;
    g.w_pad = d->x_w_pitch ? d->x_w_pad : 0;
    EXB_REQUIRE(d->fuse_pool == 0 || d->fuse_pool == 1, "fuse_pool must be 0 or 1");
    g.pool = d->fuse_pool;
    g.PH = (g.OH - 1) / 2 + 1;     // (OH + 2*1 - 3) / 2 + 1, floor mode
    g.PW = (g.OW - 1) / 2 + 1;
    g.y_pitch = d->y_pitch ? d->y_pitch : g.cout_stride;
    if (g.y_pitch != g.cout_stride) {
        EXB_REQUIRE(g.y_pitch > g.cout_stride && g.y_pitch % 16 == 0 && g.cout_stride % 16 == 0,
                    "y_pitch %d needs to be a multiple of 16 above cout_stride %d, itself a multiple of 16", g.y_pitch, g.cout_stride);
        if (g.out_dtype != EXB_F16 || g.out2_dtype != -1 || g.has_res || g.pool)
            return fail(EXB_ERR_UNSUPPORTED, "y_pitch is implemented for one fp16 output without residual or pooling");
    }
    return EXB_OK;
}

uint16_t f32_to_f16_bits(float f) {
    return __half_as_ushort(__float2half_rn(f));  // round to nearest even
}

int pack_common(exb_ctx* ctx, const ConvGeom& g, int dtype, const void* hw, size_t wbytes,
                const std::vector<float>& scale, const std::vector<float>& bias, int cout_pad, int cin_pad,
                int kw_pack, int s_shift, exb_conv_weights** out) {
    exb_conv_weights* w = new exb_conv_weights();
    memset(w, 0, sizeof(*w));
    w->dtype = dtype; w->Cout = g.Cout; w->Cin = g.Cin; w->kh = g.kh; w->kw = g.kw; w->group = g.group;
    w->cout_pad = cout_pad; w->cin_pad = cin_pad; w->kw_pack = kw_pack; w->s_shift = s_shift; w->device = ctx->device;
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc(&w->d_w, wbytes);
    if (e == cudaSuccess) e = cudaMalloc(&w->d_scale, sizeof(float) * cout_pad);
    if (e == cudaSuccess) e = cudaMalloc(&w->d_bias, sizeof(float) * cout_pad);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_w, hw, wbytes, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_scale, scale.data(), sizeof(float) * cout_pad, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_bias, bias.data(), sizeof(float) * cout_pad, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) {
        exb_conv_weights_destroy(w);
        return fail(EXB_ERR_CUDA, "conv weight upload: %s", cudaGetErrorString(e));
    }
    w->h_scale = new float[cout_pad];
    w->h_bias = new float[cout_pad];
    memcpy(w->h_scale, scale.data(), sizeof(float) * cout_pad);
    memcpy(w->h_bias, bias.data(), sizeof(float) * cout_pad);
    *out = w;
    return EXB_OK;
}

// OIHW [Cout][cin_g][kh][kw] -> [cout_pad][kh][kw_pack][cin_pad] (zero filled), tap s at column s + s_shift
template <typename TSrc, typename TDst, typename F>
void repack(const TSrc* src, std::vector<TDst>& dst, const ConvGeom& g, int cin_g, int cin_pad, int kw_pack,
            int s_shift, F cvt) {
    for (int o = 0; o < g.Cout; ++o)
        for (int c = 0; c < cin_g; ++c)
            for (int r = 0; r < g.kh; ++r)
                for (int s = 0; s < g.kw; ++s)
                    dst[(((size_t)o * g.kh + r) * kw_pack + s + s_shift) * cin_pad + c] =
                        cvt(src[(((size_t)o * cin_g + c) * g.kh + r) * g.kw + s]);
}

}  // namespace
}  // namespace exb

using namespace exb;

extern "C" int exb_conv_out_dims(const exb_conv_desc* d, int* OH, int* OW) {
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    EXB_REQUIRE(OH && OW, "null output pointer");
    *OH = g.pool ? g.PH : g.OH;
    *OW = g.pool ? g.PW : g.OW;
    return EXB_OK;
}

extern "C" int exb_conv2d_pool_fusable(const exb_conv_desc* d) {
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    return (d->impl != 1 && conv_tc_eligible(g) && conv_tc_pool_fusable(g)) ? 1 : 0;
}

extern "C" int exb_conv2d_uses_tensor_cores(const exb_conv_desc* d) {
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    return (d->impl != 1 && conv_tc_eligible(g)) ? 1 : 0;
}

extern "C" int exb_conv_weights_pack_f16(exb_ctx* ctx, const exb_conv_desc* d, const float* w_oihw,
                                         const float* bias, exb_conv_weights** out) {
    EXB_REQUIRE(ctx && out && w_oihw, "exb_conv_weights_pack_f16: null argument");
    *out = nullptr;
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    if (g.in_dtype != EXB_F16) return fail(EXB_ERR_BAD_ARG, "exb_conv_weights_pack_f16 needs in_dtype EXB_F16");
    const int cin_g = g.Cin / g.group;
    const int cin_pad = g.group == 1 ? g.cin_stride : cin_g;
    const int cout_pad = (g.cout_stride + 15) / 16 * 16;  // covers the padding channels of y too
    const FoldPlan fold = conv_fold_plan(g);
    const int kw_pack = fold.on ? fold.F : g.kw, s_shift = fold.on ? fold.shift : 0;
    std::vector<uint16_t> packed((size_t)cout_pad * g.kh * kw_pack * cin_pad, 0);
    repack(w_oihw, packed, g, cin_g, cin_pad, kw_pack, s_shift, f32_to_f16_bits);
    std::vector<float> scale(cout_pad, 0.f), b(cout_pad, 0.f);
    for (int o = 0; o < g.Cout; ++o) {
        scale[o] = 1.0f;
        if (bias) b[o] = bias[o];
    }
    return pack_common(ctx, g, EXB_F16, packed.data(), packed.size() * 2, scale, b, cout_pad, cin_pad, kw_pack, s_shift, out);
}

extern "C" int exb_conv_weights_pack_i8(exb_ctx* ctx, const exb_conv_desc* d, const int8_t* w_oihw,
                                        const float* bias, const float* wscale, int n_wscale, float act_scale,
                                        exb_conv_weights** out) {
    EXB_REQUIRE(ctx && out && w_oihw && wscale, "exb_conv_weights_pack_i8: null argument");
    *out = nullptr;
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    if (g.in_dtype != EXB_I8) return fail(EXB_ERR_BAD_ARG, "exb_conv_weights_pack_i8 needs in_dtype EXB_I8");
    EXB_REQUIRE(n_wscale == 1 || n_wscale == g.Cout, "weight scale table has %d entries, expected 1 or %d", n_wscale, g.Cout);
    const int cin_g = g.Cin / g.group;
    const int cin_pad = g.group == 1 ? g.cin_stride : cin_g;
    const int cout_pad = (g.cout_stride + 15) / 16 * 16;  // covers the padding channels of y too
    const FoldPlan fold = conv_fold_plan(g);
    const int kw_pack = fold.on ? fold.F : g.kw, s_shift = fold.on ? fold.shift : 0;
    std::vector<int8_t> packed((size_t)cout_pad * g.kh * kw_pack * cin_pad, 0);
    repack(w_oihw, packed, g, cin_g, cin_pad, kw_pack, s_shift, [](int8_t v) { return v; });
    std::vector<float> scale(cout_pad, 0.f), b(cout_pad, 0.f);
    for (int o = 0; o < g.Cout; ++o) {
        const float ws = n_wscale == 1 ? wscale[0] : wscale[o];
        // the reference's dequantise multiplier, formed in fp32 in the same order
        scale[o] = (fabsf(ws) <= 1e-6) ? 0.f : (1.0f / (ws * act_scale));
        if (bias) b[o] = bias[o];
    }
    return pack_common(ctx, g, EXB_I8, packed.data(), packed.size(), scale, b, cout_pad, cin_pad, kw_pack, s_shift, out);
}

extern "C" int exb_conv_weights_destroy(exb_conv_weights* w) {
    if (!w) return EXB_OK;
    if (w->d_w) cudaFree(w->d_w);
    if (w->d_scale) cudaFree(w->d_scale);
    if (w->d_bias) cudaFree(w->d_bias);
    if (w->d_slope) cudaFree(w->d_slope);
    delete[] w->h_scale;
    delete[] w->h_bias;
    delete w;
    return EXB_OK;
}

extern "C" int exb_conv2d_fwd(exb_ctx* ctx, const exb_conv_desc* d, const void* x, const exb_conv_weights* w,
                              const void* residual, void* y, void* y2, void* stream) {
    EXB_REQUIRE(ctx && w, "exb_conv2d_fwd: null argument");
    ConvGeom g;
    if (int rc = resolve(d, g)) return rc;
    const int cin_pad = g.group == 1 ? g.cin_stride : g.Cin / g.group;
    EXB_REQUIRE(w->dtype == g.in_dtype && w->Cout == g.Cout && w->Cin == g.Cin && w->kh == g.kh && w->kw == g.kw &&
                    w->group == g.group && w->cin_pad == cin_pad,
                "exb_conv2d_fwd: packed weights do not match the descriptor");
    {
        const FoldPlan fold = conv_fold_plan(g);
        EXB_REQUIRE(w->kw_pack == (fold.on ? fold.F : g.kw) && w->s_shift == (fold.on ? fold.shift : 0),
                    "exb_conv2d_fwd: weights were packed for a different input row layout");
    }
    EXB_REQUIRE(w->device == ctx->device, "exb_conv2d_fwd: weights live on device %d, context on %d", w->device, ctx->device);
    if (g.act == EXB_ACT_PRELU) {
        EXB_REQUIRE(w->d_slope != nullptr, "exb_conv2d_fwd: EXB_ACT_PRELU without slopes (exb_conv_weights_set_slopes)");
        EXB_REQUIRE(g.cout_stride <= w->cout_pad + kSlopeSlack - 16, "exb_conv2d_fwd: output channel stride %d too wide for PReLU",
                    g.cout_stride);
    }
    if (g.N == 0) return EXB_OK;
    EXB_REQUIRE(x && y && aligned16(x) && aligned16(y), "exb_conv2d_fwd: null or misaligned x / y");
    EXB_REQUIRE(!g.has_res || (residual && aligned16(residual)), "exb_conv2d_fwd: null or misaligned residual");
    EXB_REQUIRE(g.out2_dtype == -1 || (y2 && aligned16(y2)), "exb_conv2d_fwd: null or misaligned second output");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (g.pool && !(d->impl != 1 && conv_tc_eligible(g) && conv_tc_pool_fusable(g)))
        return fail(EXB_ERR_UNSUPPORTED, "fuse_pool is not available for this convolution (see exb_conv2d_pool_fusable)");
    if (g.y_pitch != g.cout_stride && !(d->impl != 1 && conv_tc_eligible(g)))
        return fail(EXB_ERR_UNSUPPORTED, "y_pitch needs the tensor-core kernel");
    if (d->impl != 1 && conv_tc_eligible(g)) return conv_tc_launch(ctx, g, x, w, residual, y, y2, st);
    return conv_direct_launch(ctx, g, x, w, residual, y, y2, st);
}

extern "C" int exb_conv_weights_set_slopes(exb_ctx* ctx, exb_conv_weights* w, const float* slopes, int n) {
    EXB_REQUIRE(ctx != nullptr && w != nullptr && slopes != nullptr, "exb_conv_weights_set_slopes: null argument");
    EXB_REQUIRE(n == 1 || n == w->Cout, "exb_conv_weights_set_slopes: %d slopes for %d output channels", n, w->Cout);
    const size_t len = (size_t)w->cout_pad + kSlopeSlack;
    std::vector<float> h(len, 0.f);
    for (int c = 0; c < w->Cout; ++c) h[c] = slopes[n == 1 ? 0 : c];
    cudaError_t e = cudaSetDevice(w->device);
    if (e == cudaSuccess && !w->d_slope) e = cudaMalloc(&w->d_slope, sizeof(float) * len);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_slope, h.data(), sizeof(float) * len, cudaMemcpyHostToDevice);
    if (e != cudaSuccess) return fail(EXB_ERR_CUDA, "exb_conv_weights_set_slopes: %s", cudaGetErrorString(e));
    return EXB_OK;
}
