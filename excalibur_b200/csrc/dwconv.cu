// Depthwise convolution on NHWC tensors, fp32 math on fp16 or int8 activations.
// A thread owns 8 consecutive channels of a strip of TW output pixels along W: every input
// vector of the strip is loaded once per kernel row and reused by all taps that touch it, and
// each weight vector is loaded once per strip.  Weights are kept tap-major [kh*kw][C] in fp32
// so consecutive threads read consecutive channels.
#include <type_traits>

#include "common.cuh"

struct exb_dw_weights {
    float* d_w;     // [kh*kw][cs]
    float* d_bias;  // [cs] (zeros when the layer has no bias)
    float* d_slope; // [cs] PReLU slopes, or null
    int C, cs, kh, kw;
    int device;
};

namespace exb {
namespace {

constexpr int V = 8;  // channels per thread

struct DwParams {
    int N, H, W, cs, OH, OW;
    int kh, kw, sh, sw, pt, pl;
    int act;
    float in_scale, out_scale;
    const float* slope;   // EXB_ACT_PRELU only: [cs]
};

__device__ __forceinline__ void load8(const __half* p, float (&v)[V], float) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void load8(const int8_t* p, float (&v)[V], float scale) {
    alignas(8) int8_t b[8];
    *reinterpret_cast<uint2*>(b) = *reinterpret_cast<const uint2*>(p);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = (float)b[i] * scale;
}
__device__ __forceinline__ void store8(__half* p, const float (&v)[V], float) {
    uint4 r;
    __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
}
__device__ __forceinline__ void store8(int8_t* p, const float (&v)[V], float scale) {
    uint2 r;
    r.x = quant_pack4(v[0], v[1], v[2], v[3], scale);
    r.y = quant_pack4(v[4], v[5], v[6], v[7], scale);
    *reinterpret_cast<uint2*>(p) = r;
}
__device__ __forceinline__ void loadw(const float* p, float (&v)[V]);
// Activation of the 8 channels starting at c0.
__device__ __forceinline__ void dw_act(float (&v)[V], const DwParams& p, int c0) {
    if (p.act == EXB_ACT_PRELU) {
        float s[V];
        loadw(p.slope + c0, s);
#pragma unroll
        for (int k = 0; k < V; ++k) v[k] = v[k] >= 0.f ? v[k] : v[k] * s[k];
    } else {
        apply_act_vec(v, p.act);
    }
}
__device__ __forceinline__ void loadw(const float* p, float (&v)[V]) {
    float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename TIn, typename TOut, int K, int S, int TW>
__global__ void __launch_bounds__(128) dw_strip_kernel(const TIn* __restrict__ x, const float* __restrict__ w,
                                                       const float* __restrict__ bias, TOut* __restrict__ y,
                                                       DwParams p) {
    constexpr int IN_W = (TW - 1) * S + K;
    const int cvecs = p.cs / V;
    const int owb = (p.OW + TW - 1) / TW;
    const int64_t total = (int64_t)p.N * p.OH * owb * cvecs;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int cv = (int)(idx % cvecs);
        int64_t t = idx / cvecs;
        const int ob = (int)(t % owb); t /= owb;
        const int oh = (int)(t % p.OH);
        const int n = (int)(t / p.OH);
        const int ow0 = ob * TW;
        float acc[TW][V];
        {
            float b[V];
            loadw(bias + cv * V, b);
#pragma unroll
            for (int j = 0; j < TW; ++j)
#pragma unroll
                for (int k = 0; k < V; ++k) acc[j][k] = b[k];
        }
#pragma unroll
        for (int r = 0; r < K; ++r) {
            const int ih = oh * S - p.pt + r;
            if (ih < 0 || ih >= p.H) continue;
            float in[IN_W][V];
#pragma unroll
            for (int j = 0; j < IN_W; ++j) {
                const int iw = ow0 * S - p.pl + j;
                if (iw >= 0 && iw < p.W) {
                    load8(x + (((int64_t)n * p.H + ih) * p.W + iw) * p.cs + cv * V, in[j], p.in_scale);
                } else {
#pragma unroll
                    for (int k = 0; k < V; ++k) in[j][k] = 0.f;
                }
            }
#pragma unroll
            for (int s = 0; s < K; ++s) {
                float wv[V];
                loadw(w + (int64_t)(r * K + s) * p.cs + cv * V, wv);
#pragma unroll
                for (int j = 0; j < TW; ++j)
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[j][k] = fmaf(in[j * S + s][k], wv[k], acc[j][k]);
            }
        }
#pragma unroll
        for (int j = 0; j < TW; ++j) {
            const int ow = ow0 + j;
            if (ow < p.OW) {
                dw_act(acc[j], p, cv * V);
                store8(y + (((int64_t)n * p.OH + oh) * p.OW + ow) * p.cs + cv * V, acc[j], p.out_scale);
            }
        }
    }
}

// 3x3 fp16 -> fp16, rolling window: a thread owns 8 channels x TW output columns and walks R output
// rows downwards, keeping the last input rows in registers (raw fp16 vectors), so every input row
// is loaded once per thread instead of once per output row; weights and bias sit in shared memory.
// Over-fetch is (R+2)/R vertically and ((TW-1)*S+3)/(TW*S) horizontally, all of it served by L1/L2.
// Four CTAs per SM (128 registers per thread, a few dozen bytes spilled): the kernel is bound by the latency of its
// loads, and 16 warps per SM instead of the 12 that 160 registers allowed put a third more bytes in flight
// (0.17 -> 0.13 ms on 32 channels @112, 0.20 -> 0.15 ms on 96 channels @112 stride 2); five CTAs spill too much.
__device__ __forceinline__ void cvt8(const uint4& r, float (&v)[V]) {
    const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}

template <typename TOut, int S, int TW, int R>
__global__ void __launch_bounds__(128, 4) dw3x3_roll_f16_kernel(const __half* __restrict__ x, const float* __restrict__ w,
                                                             const float* __restrict__ bias, TOut* __restrict__ y,
                                                             DwParams p) {
    constexpr int IN_W = (TW - 1) * S + 3;
    extern __shared__ float s_w[];   // [9][cs] taps, then [cs] bias
    for (int i = threadIdx.x; i < 9 * p.cs; i += blockDim.x) s_w[i] = w[i];
    for (int i = threadIdx.x; i < p.cs; i += blockDim.x) s_w[9 * p.cs + i] = bias[i];
    __syncthreads();
    const int cvecs = p.cs / V;
    const int owb = (p.OW + TW - 1) / TW, ohb = (p.OH + R - 1) / R;
    const int64_t total = (int64_t)p.N * ohb * owb * cvecs;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int cv = (int)(idx % cvecs);
        int64_t t = idx / cvecs;
        const int ob = (int)(t % owb); t /= owb;
        const int rb = (int)(t % ohb);
        const int n = (int)(t / ohb);
        const int ow0 = ob * TW, oh0 = rb * R;
        const int iw0 = ow0 * S - p.pl;
        const __half* xin = x + (int64_t)n * p.H * p.W * p.cs + cv * V;
        auto load_row = [&](int ih, uint4 (&row)[IN_W]) {
            const bool rok = ih >= 0 && ih < p.H;
#pragma unroll
            for (int j = 0; j < IN_W; ++j) {
                const int iw = iw0 + j;
                row[j] = (rok && iw >= 0 && iw < p.W)
                             ? *reinterpret_cast<const uint4*>(xin + ((int64_t)ih * p.W + iw) * p.cs)
                             : zero;
            }
        };
        uint4 r0[IN_W], r1[IN_W], r2[IN_W];
        if (S == 1) {
            load_row(oh0 - p.pt, r0);
            load_row(oh0 - p.pt + 1, r1);
        } else {
            load_row(oh0 * 2 - p.pt, r0);
        }
        const float* wb = s_w + cv * V;
#pragma unroll 1
        for (int orow = 0; orow < R; ++orow) {
            const int oh = oh0 + orow;
            if (oh >= p.OH) break;
            if (S == 1) {
                load_row(oh - p.pt + 2, r2);
            } else {
                load_row(oh * 2 - p.pt + 1, r1);
                load_row(oh * 2 - p.pt + 2, r2);
            }
            float acc[TW][V];
            {
                float b[V];
                loadw(wb + 9 * p.cs, b);
#pragma unroll
                for (int j = 0; j < TW; ++j)
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[j][k] = b[k];
            }
#pragma unroll
            for (int r = 0; r < 3; ++r) {
                float wv[3][V];
#pragma unroll
                for (int sx = 0; sx < 3; ++sx) loadw(wb + (r * 3 + sx) * p.cs, wv[sx]);
#pragma unroll
                for (int j = 0; j < IN_W; ++j) {
                    float f[V];
                    cvt8(r == 0 ? r0[j] : (r == 1 ? r1[j] : r2[j]), f);
#pragma unroll
                    for (int tcol = 0; tcol < TW; ++tcol) {
                        const int sx = j - tcol * S;
                        if (sx >= 0 && sx < 3) {
#pragma unroll
                            for (int k = 0; k < V; ++k) acc[tcol][k] = fmaf(f[k], wv[sx][k], acc[tcol][k]);
                        }
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < TW; ++j) {
                const int ow = ow0 + j;
                if (ow < p.OW) {
                    dw_act(acc[j], p, cv * V);
                    store8(y + (((int64_t)n * p.OH + oh) * p.OW + ow) * p.cs + cv * V, acc[j], p.out_scale);
                }
            }
            // the window moves down by S rows
#pragma unroll
            for (int j = 0; j < IN_W; ++j) {
                if (S == 1) {
                    r0[j] = r1[j];
                    r1[j] = r2[j];
                } else {
                    r0[j] = r2[j];
                }
            }
        }
    }
}

// Any window / stride: one output pixel x 8 channels per thread.
template <typename TIn, typename TOut>
__global__ void __launch_bounds__(128) dw_generic_kernel(const TIn* __restrict__ x, const float* __restrict__ w,
                                                         const float* __restrict__ bias, TOut* __restrict__ y,
                                                         DwParams p) {
    const int cvecs = p.cs / V;
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cvecs;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int cv = (int)(idx % cvecs);
        int64_t t = idx / cvecs;
        const int ow = (int)(t % p.OW); t /= p.OW;
        const int oh = (int)(t % p.OH);
        const int n = (int)(t / p.OH);
        float acc[V];
        loadw(bias + cv * V, acc);
        for (int r = 0; r < p.kh; ++r) {
            const int ih = oh * p.sh - p.pt + r;
            if (ih < 0 || ih >= p.H) continue;
            for (int s = 0; s < p.kw; ++s) {
                const int iw = ow * p.sw - p.pl + s;
                if (iw < 0 || iw >= p.W) continue;
                float in[V], wv[V];
                load8(x + (((int64_t)n * p.H + ih) * p.W + iw) * p.cs + cv * V, in, p.in_scale);
                loadw(w + (int64_t)(r * p.kw + s) * p.cs + cv * V, wv);
#pragma unroll
                for (int k = 0; k < V; ++k) acc[k] = fmaf(in[k], wv[k], acc[k]);
            }
        }
        dw_act(acc, p, cv * V);
        store8(y + (((int64_t)n * p.OH + oh) * p.OW + ow) * p.cs + cv * V, acc, p.out_scale);
    }
}

template <typename TIn, typename TOut>
int launch(exb_ctx* ctx, const DwParams& p, const void* x, const exb_dw_weights* w, void* y, cudaStream_t st) {
    const TIn* xi = static_cast<const TIn*>(x);
    TOut* yo = static_cast<TOut*>(y);
    const int cvecs = p.cs / V;
    constexpr int TW = 4;
    if constexpr (std::is_same<TIn, __half>::value) {      // fp16 or int8 (quantised in the store) output
        const size_t smem = (size_t)10 * p.cs * sizeof(float);
        if (p.kh == 3 && p.kw == 3 && p.sh == p.sw && (p.sh == 1 || p.sh == 2) && smem <= 48 * 1024) {
            constexpr int R = 8;
            if (p.sh == 1) {
                const int64_t total = (int64_t)p.N * ((p.OH + R - 1) / R) * ((p.OW + 3) / 4) * cvecs;
                const int grid = stream_grid(ctx, total, 128, 4);
                dw3x3_roll_f16_kernel<TOut, 1, 4, R><<<grid, 128, smem, st>>>(xi, w->d_w, w->d_bias, yo, p);
            } else {
                const int64_t total = (int64_t)p.N * ((p.OH + R - 1) / R) * ((p.OW + 1) / 2) * cvecs;
                const int grid = stream_grid(ctx, total, 128, 4);
                dw3x3_roll_f16_kernel<TOut, 2, 2, R><<<grid, 128, smem, st>>>(xi, w->d_w, w->d_bias, yo, p);
            }
            return after_launch("dw3x3_roll_f16_kernel");
        }
    }
    if (p.kh == 3 && p.kw == 3 && p.sh == p.sw && (p.sh == 1 || p.sh == 2)) {
        const int64_t total = (int64_t)p.N * p.OH * ((p.OW + TW - 1) / TW) * cvecs;
        const int grid = stream_grid(ctx, total, 128, 16);
        if (p.sh == 1) dw_strip_kernel<TIn, TOut, 3, 1, TW><<<grid, 128, 0, st>>>(xi, w->d_w, w->d_bias, yo, p);
        else dw_strip_kernel<TIn, TOut, 3, 2, TW><<<grid, 128, 0, st>>>(xi, w->d_w, w->d_bias, yo, p);
        return after_launch("dw_strip_kernel");
    }
    const int64_t total = (int64_t)p.N * p.OH * p.OW * cvecs;
    const int grid = stream_grid(ctx, total, 128, 16);
    dw_generic_kernel<TIn, TOut><<<grid, 128, 0, st>>>(xi, w->d_w, w->d_bias, yo, p);
    return after_launch("dw_generic_kernel");
}

int check_desc(const exb_dwconv_desc* d, int& cs, int& OH, int& OW) {
    EXB_REQUIRE(d != nullptr, "null depthwise descriptor");
    EXB_REQUIRE(d->N >= 0 && d->H > 0 && d->W > 0 && d->C > 0, "bad depthwise input shape");
    EXB_REQUIRE(d->kh > 0 && d->kw > 0 && d->stride_h > 0 && d->stride_w > 0, "bad depthwise window / stride");
    EXB_REQUIRE(d->pad_t >= 0 && d->pad_b >= 0 && d->pad_l >= 0 && d->pad_r >= 0, "negative pad");
    cs = d->c_stride ? d->c_stride : d->C;
    EXB_REQUIRE(cs >= d->C, "c_stride %d < C %d", cs, d->C);
    if (cs % V != 0) return fail(EXB_ERR_UNSUPPORTED, "depthwise conv needs the physical channel count (%d) to be a multiple of %d", cs, V);
    OH = (d->H + d->pad_t + d->pad_b - d->kh) / d->stride_h + 1;
    OW = (d->W + d->pad_l + d->pad_r - d->kw) / d->stride_w + 1;
    EXB_REQUIRE(OH > 0 && OW > 0, "depthwise window larger than the padded input");
    if (!act_supported(d->act) && d->act != EXB_ACT_PRELU)
        return fail(EXB_ERR_UNSUPPORTED, "activation type %d is not implemented", d->act);
    return EXB_OK;
}

}  // namespace
}  // namespace exb

using namespace exb;

extern "C" int exb_dw_weights_pack(exb_ctx* ctx, const exb_dwconv_desc* d, const float* w, const float* bias,
                                   exb_dw_weights** out) {
    EXB_REQUIRE(ctx && out && w, "exb_dw_weights_pack: null argument");
    *out = nullptr;
    int cs, OH, OW;
    if (int rc = check_desc(d, cs, OH, OW)) return rc;
    const int taps = d->kh * d->kw;
    float* hw = new float[(size_t)taps * cs]();
    float* hb = new float[cs]();
    for (int c = 0; c < d->C; ++c) {
        for (int t = 0; t < taps; ++t) hw[(size_t)t * cs + c] = w[(size_t)c * taps + t];
        if (bias) hb[c] = bias[c];
    }
    exb_dw_weights* pw = new exb_dw_weights();
    pw->C = d->C; pw->cs = cs; pw->kh = d->kh; pw->kw = d->kw; pw->device = ctx->device;
    pw->d_w = nullptr; pw->d_bias = nullptr; pw->d_slope = nullptr;
    cudaError_t e = cudaSetDevice(ctx->device);
    if (e == cudaSuccess) e = cudaMalloc(&pw->d_w, sizeof(float) * taps * cs);
    if (e == cudaSuccess) e = cudaMalloc(&pw->d_bias, sizeof(float) * cs);
    if (e == cudaSuccess) e = cudaMemcpy(pw->d_w, hw, sizeof(float) * taps * cs, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaMemcpy(pw->d_bias, hb, sizeof(float) * cs, cudaMemcpyHostToDevice);
    delete[] hw;
    delete[] hb;
    if (e != cudaSuccess) {
        exb_dw_weights_destroy(pw);
        return fail(EXB_ERR_CUDA, "exb_dw_weights_pack: %s", cudaGetErrorString(e));
    }
    *out = pw;
    return EXB_OK;
}

extern "C" int exb_dw_weights_destroy(exb_dw_weights* w) {
    if (!w) return EXB_OK;
    if (w->d_w) cudaFree(w->d_w);
    if (w->d_bias) cudaFree(w->d_bias);
    if (w->d_slope) cudaFree(w->d_slope);
    delete w;
    return EXB_OK;
}

extern "C" int exb_dwconv2d_fwd(exb_ctx* ctx, const exb_dwconv_desc* d, const void* x, const exb_dw_weights* w,
                                void* y, void* stream) {
    EXB_REQUIRE(ctx && w, "exb_dwconv2d_fwd: null argument");
    int cs, OH, OW;
    if (int rc = check_desc(d, cs, OH, OW)) return rc;
    EXB_REQUIRE(w->C == d->C && w->cs == cs && w->kh == d->kh && w->kw == d->kw,
                "exb_dwconv2d_fwd: packed weights do not match the descriptor");
    if (d->N == 0) return EXB_OK;
    EXB_REQUIRE(x && y && aligned16(x) && aligned16(y), "exb_dwconv2d_fwd: null or misaligned buffer");
    DwParams p;
    p.N = d->N; p.H = d->H; p.W = d->W; p.cs = cs; p.OH = OH; p.OW = OW;
    p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w; p.pt = d->pad_t; p.pl = d->pad_l;
    p.act = d->act; p.in_scale = d->in_scale; p.out_scale = d->out_scale;
    p.slope = w->d_slope;
    EXB_REQUIRE(p.act != EXB_ACT_PRELU || p.slope != nullptr, "exb_dwconv2d_fwd: EXB_ACT_PRELU without slopes (exb_dw_weights_set_slopes)");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (d->in_dtype == EXB_F16 && d->out_dtype == EXB_F16) return launch<__half, __half>(ctx, p, x, w, y, st);
    if (d->in_dtype == EXB_I8 && d->out_dtype == EXB_I8) return launch<int8_t, int8_t>(ctx, p, x, w, y, st);
    if (d->in_dtype == EXB_I8 && d->out_dtype == EXB_F16) return launch<int8_t, __half>(ctx, p, x, w, y, st);
    if (d->in_dtype == EXB_F16 && d->out_dtype == EXB_I8) return launch<__half, int8_t>(ctx, p, x, w, y, st);
    return fail(EXB_ERR_UNSUPPORTED, "depthwise conv dtypes in=%d out=%d", d->in_dtype, d->out_dtype);
}

extern "C" int exb_dw_weights_set_slopes(exb_ctx* ctx, exb_dw_weights* w, const float* slopes, int n) {
    EXB_REQUIRE(ctx != nullptr && w != nullptr && slopes != nullptr, "exb_dw_weights_set_slopes: null argument");
    EXB_REQUIRE(n == 1 || n == w->C, "exb_dw_weights_set_slopes: %d slopes for %d channels", n, w->C);
    float* h = new float[w->cs]();
    for (int c = 0; c < w->C; ++c) h[c] = slopes[n == 1 ? 0 : c];
    cudaError_t e = cudaSetDevice(w->device);
    if (e == cudaSuccess && !w->d_slope) e = cudaMalloc(&w->d_slope, sizeof(float) * w->cs);
    if (e == cudaSuccess) e = cudaMemcpy(w->d_slope, h, sizeof(float) * w->cs, cudaMemcpyHostToDevice);
    delete[] h;
    if (e != cudaSuccess) return fail(EXB_ERR_CUDA, "exb_dw_weights_set_slopes: %s", cudaGetErrorString(e));
    return EXB_OK;
}
