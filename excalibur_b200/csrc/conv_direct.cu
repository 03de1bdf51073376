// Direct convolution: one thread per (output pixel, output channel).  It covers what the
// tensor-core kernel does not (grouped convolution, strides above 2, channel counts that do
// not meet the TMA alignment rules) and serves as an on-device cross-check of the tensor-core
// kernel at sizes a CPU oracle cannot reach.  Same fused epilogue as the tensor-core kernel.
#include "conv_common.cuh"

#include <type_traits>

namespace exb {
namespace {

struct DirectParams {
    int N, H, W, cin_stride, OH, OW, Cout;
    int kh, kw, sh, sw, pt, pl;
    int cin_g;    // input channels per group actually multiplied
    int cout_g;   // output channels per group
    int w_cin;    // channels per tap in the packed weight rows
    int kw_pack, s_shift;   // packed taps per kernel row / column of tap 0
    int w_pitch, w_pad;     // physical input row pitch and left padding (pixels)
    int has_res;
    EpiParams e;
};

template <bool kInt8>
__global__ void __launch_bounds__(256) conv_direct_kernel(const void* __restrict__ xv, const void* __restrict__ wv,
                                                          DirectParams p) {
    typedef typename std::conditional<kInt8, int8_t, __half>::type T;
    const T* x = static_cast<const T*>(xv);
    const T* w = static_cast<const T*>(wv);
    const int64_t total = (int64_t)p.N * p.OH * p.OW * p.Cout;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int co = (int)(idx % p.Cout);
        int64_t pix = idx / p.Cout;
        const int ow = (int)(pix % p.OW);
        const int oh = (int)((pix / p.OW) % p.OH);
        const int n = (int)(pix / ((int64_t)p.OW * p.OH));
        const int g = co / p.cout_g;
        int iacc = 0;
        float facc = 0.f;
        for (int r = 0; r < p.kh; ++r) {
            const int ih = oh * p.sh - p.pt + r;
            if (ih < 0 || ih >= p.H) continue;
            for (int s = 0; s < p.kw; ++s) {
                const int iw = ow * p.sw - p.pl + s;
                if (iw < 0 || iw >= p.W) continue;
                const T* xp = x + (((int64_t)n * p.H + ih) * p.w_pitch + iw + p.w_pad) * p.cin_stride + g * p.cin_g;
                const T* wp = w + (((int64_t)co * p.kh + r) * p.kw_pack + s + p.s_shift) * p.w_cin;
                for (int c = 0; c < p.cin_g; ++c) {
                    if (kInt8) iacc += (int)xp[c] * (int)wp[c];
                    else facc = fmaf(__half2float(xp[c]), __half2float(wp[c]), facc);
                }
            }
        }
        const uint32_t raw = kInt8 ? (uint32_t)iacc : __float_as_uint(facc);
        float v = epi_value<kInt8>(raw, p.e.scale[co], p.e.bias[co]);
        const int64_t off = pix * p.e.cout_stride + co;
        if (p.has_res) v += __half2float(p.e.residual[off]);
        if (p.e.act == EXB_ACT_PRELU) v = v >= 0.f ? v : v * p.e.slope[co];
        else v = apply_act(v, p.e.act);
        epi_store_scalar(p.e.y, p.e.out_dtype, off, v, p.e.out_scale, raw);
        if (p.e.out2_dtype >= 0) epi_store_scalar(p.e.y2, p.e.out2_dtype, off, v, p.e.out2_scale, raw);
    }
}

// Zero the padding channels [Cout, cout_stride) of an NHWC output so consumers never read
// uninitialised memory.
__global__ void zero_pad_channels_kernel(void* y, int esize, int64_t pixels, int Cout, int cout_stride) {
    const int padc = cout_stride - Cout;
    const int64_t total = pixels * padc;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t pix = i / padc;
        const int c = Cout + (int)(i % padc);
        char* dst = static_cast<char*>(y) + (pix * cout_stride + c) * esize;
        for (int b = 0; b < esize; ++b) dst[b] = 0;
    }
}

}  // namespace

int conv_direct_launch(exb_ctx* ctx, const ConvGeom& g, const void* x, const exb_conv_weights* w,
                       const void* residual, void* y, void* y2, cudaStream_t st) {
    DirectParams p;
    p.N = g.N; p.H = g.H; p.W = g.W; p.cin_stride = g.cin_stride; p.OH = g.OH; p.OW = g.OW; p.Cout = g.Cout;
    p.kh = g.kh; p.kw = g.kw; p.sh = g.sh; p.sw = g.sw; p.pt = g.pt; p.pl = g.pl;
    p.cin_g = g.Cin / g.group;
    p.cout_g = g.Cout / g.group;
    p.w_cin = w->cin_pad;
    p.kw_pack = w->kw_pack; p.s_shift = w->s_shift;
    p.w_pitch = g.w_pitch; p.w_pad = g.w_pad;
    p.has_res = g.has_res;
    p.e.scale = w->d_scale; p.e.bias = w->d_bias; p.e.slope = w->d_slope; p.e.residual = static_cast<const __half*>(residual);
    p.e.y = y; p.e.y2 = y2; p.e.out_dtype = g.out_dtype; p.e.out2_dtype = g.out2_dtype; p.e.act = g.act;
    p.e.out_scale = g.out_scale; p.e.out2_scale = g.out2_scale; p.e.cout_stride = g.cout_stride;
    const int64_t total = (int64_t)g.N * g.OH * g.OW * g.Cout;
    const int grid = stream_grid(ctx, total, 256, 16);
    if (g.in_dtype == EXB_I8) conv_direct_kernel<true><<<grid, 256, 0, st>>>(x, w->d_w, p);
    else conv_direct_kernel<false><<<grid, 256, 0, st>>>(x, w->d_w, p);
    if (int rc = after_launch("conv_direct_kernel")) return rc;
    if (g.cout_stride > g.Cout) {
        const int64_t pixels = (int64_t)g.N * g.OH * g.OW;
        const int zgrid = stream_grid(ctx, pixels * (g.cout_stride - g.Cout), 256);
        zero_pad_channels_kernel<<<zgrid, 256, 0, st>>>(y, (int)dtype_size(g.out_dtype), pixels, g.Cout, g.cout_stride);
        if (g.out2_dtype >= 0)
            zero_pad_channels_kernel<<<zgrid, 256, 0, st>>>(y2, (int)dtype_size(g.out2_dtype), pixels, g.Cout, g.cout_stride);
        return after_launch("zero_pad_channels_kernel");
    }
    return EXB_OK;
}

}  // namespace exb
