// Max / average / global pooling on NHWC tensors.  One thread produces one 16-byte channel
// vector of one output pixel (8 fp16, 16 int8 or 4 fp32 channels), so a warp reads and writes
// whole contiguous pixel rows.  Global pooling splits the map across the warps of a CTA and
// combines the partial sums through shared memory.
#include "common.cuh"

#include <float.h>

#include <type_traits>

namespace exb {
namespace {

struct PoolParams {
    int N, H, W, C, cs;  // cs = physical channels
    int PH, PW;
    int type, kh, kw, sh, sw, pt, pb, pl, pr;
    int count_include_pad;
    float out2_scale;
};

template <typename T> struct PV;
template <> struct PV<__half> {
    static constexpr int N = 8;
    __device__ static void load(const __half* p, float (&v)[8]) {
        uint4 r = *reinterpret_cast<const uint4*>(p);
        const __half2* h = reinterpret_cast<const __half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) { float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    __device__ static void store(__half* p, const float (&v)[8]) {
        uint4 r;
        __half2* h = reinterpret_cast<__half2*>(&r);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4*>(p) = r;
    }
};
template <> struct PV<float> {
    static constexpr int N = 4;
    __device__ static void load(const float* p, float (&v)[4]) {
        float4 r = *reinterpret_cast<const float4*>(p);
        v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
    }
    __device__ static void store(float* p, const float (&v)[4]) {
        *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
    }
};
template <> struct PV<int8_t> {
    static constexpr int N = 16;
    __device__ static void load(const int8_t* p, float (&v)[16]) {
        alignas(16) int8_t b[16];
        *reinterpret_cast<uint4*>(b) = *reinterpret_cast<const uint4*>(p);
#pragma unroll
        for (int i = 0; i < 16; ++i) v[i] = (float)b[i];
    }
    __device__ static void store(int8_t* p, const float (&v)[16]) {
        alignas(16) int8_t b[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) b[i] = (int8_t)(int)v[i];
        *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(b);
    }
};

// Second output: int8 copy of V consecutive channels, q = sat8(rne(v * scale)).
template <int V>
__device__ __forceinline__ void store_q8(int8_t* p, const float (&v)[V], float scale) {
    alignas(16) int8_t b[V];
#pragma unroll
    for (int i = 0; i < V; ++i) b[i] = (int8_t)quant_rne(v[i] * scale);
    if (V == 8) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(b);
    else if (V == 4) *reinterpret_cast<uint32_t*>(p) = *reinterpret_cast<const uint32_t*>(b);
    else *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(b);
}

template <typename T, bool kOut2>
__global__ void __launch_bounds__(256) pool_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                   int8_t* __restrict__ y2, PoolParams p) {
    constexpr int V = PV<T>::N;
    const int cvecs = p.cs / V;
    const int64_t total = (int64_t)p.N * p.PH * p.PW * cvecs;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += stride) {
        const int cv = (int)(idx % cvecs);
        int64_t t = idx / cvecs;
        const int pw = (int)(t % p.PW); t /= p.PW;
        const int ph = (int)(t % p.PH);
        const int n = (int)(t / p.PH);
        int hs = ph * p.sh - p.pt, ws = pw * p.sw - p.pl;
        float acc[V];
        if (p.type == 0) {
            const int he = min(hs + p.kh, p.H), we = min(ws + p.kw, p.W);
            hs = max(hs, 0); ws = max(ws, 0);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = -FLT_MAX;
            for (int h = hs; h < he; ++h)
                for (int w = ws; w < we; ++w) {
                    float v[V];
                    PV<T>::load(x + (((int64_t)n * p.H + h) * p.W + w) * p.cs + cv * V, v);
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] = fmaxf(acc[k], v[k]);
                }
        } else {
            int he = min(hs + p.kh, p.H + p.pb), we = min(ws + p.kw, p.W + p.pr);
            int pool_size = (he - hs) * (we - ws);
            hs = max(hs, 0); ws = max(ws, 0);
            he = min(he, p.H); we = min(we, p.W);
            if (p.count_include_pad == 0) pool_size = (he - hs) * (we - ws);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = 0.f;
            for (int h = hs; h < he; ++h)
                for (int w = ws; w < we; ++w) {
                    float v[V];
                    PV<T>::load(x + (((int64_t)n * p.H + h) * p.W + w) * p.cs + cv * V, v);
#pragma unroll
                    for (int k = 0; k < V; ++k) acc[k] += v[k];
                }
            const float div = (float)pool_size;
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = acc[k] / div;
        }
        const int64_t o = (((int64_t)n * p.PH + ph) * p.PW + pw) * p.cs + cv * V;
        PV<T>::store(y + o, acc);
        if (kOut2) store_q8<V>(y2 + o, acc, p.out2_scale);
    }
}

// Global pooling: grid = (ceil(cvecs/32), N), block = 8 warps.  Lane = channel vector (coalesced),
// warp w reduces pixels w, w+8, ...; partials are combined through shared memory.
template <typename T, bool kOut2>
__global__ void __launch_bounds__(256) global_pool_kernel(const T* __restrict__ x, T* __restrict__ y,
                                                          int8_t* __restrict__ y2, PoolParams p) {
    constexpr int V = PV<T>::N;
    __shared__ float part[8][32][V + 1];
    const int cvecs = p.cs / V;
    const int cv = blockIdx.x * 32 + (threadIdx.x & 31);
    const int warp = threadIdx.x >> 5;
    const int n = blockIdx.y;
    const int HW = p.H * p.W;
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = p.type == 0 ? -FLT_MAX : 0.f;
    if (cv < cvecs) {
        for (int i = warp; i < HW; i += 8) {
            float v[V];
            PV<T>::load(x + ((int64_t)n * HW + i) * p.cs + cv * V, v);
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = p.type == 0 ? fmaxf(acc[k], v[k]) : acc[k] + v[k];
        }
    }
#pragma unroll
    for (int k = 0; k < V; ++k) part[warp][threadIdx.x & 31][k] = acc[k];
    __syncthreads();
    if (warp == 0 && cv < cvecs) {
        for (int w = 1; w < 8; ++w)
#pragma unroll
            for (int k = 0; k < V; ++k) {
                float o = part[w][threadIdx.x][k];
                acc[k] = p.type == 0 ? fmaxf(acc[k], o) : acc[k] + o;
            }
        if (p.type == 1) {
            const float div = (float)HW;
#pragma unroll
            for (int k = 0; k < V; ++k) acc[k] = acc[k] / div;
        }
        const int64_t o = (int64_t)n * p.cs + cv * V;
        PV<T>::store(y + o, acc);
        if (kOut2) store_q8<V>(y2 + o, acc, p.out2_scale);
    }
}

// 3x3 / stride 2 max pooling of fp16 NHWC data (the ResNet stem pool): a thread produces a 2x2
// block of outputs for 16 channels.  The 5x5 input patch is read once with 32-byte loads (25
// loads for 4 outputs instead of 36), maxima are taken on packed half2 values, and the optional
// int8 copy is quantised from the same registers.
__device__ __forceinline__ void ld256(const void* p, uint32_t (&o)[8]) {
    asm volatile("ld.global.nc.v8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(o[0]), "=r"(o[1]), "=r"(o[2]), "=r"(o[3]), "=r"(o[4]), "=r"(o[5]), "=r"(o[6]), "=r"(o[7])
                 : "l"(p));
}
__device__ __forceinline__ void st256(void* p, const uint32_t (&o)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(o[0]), "r"(o[1]), "r"(o[2]),
                 "r"(o[3]), "r"(o[4]), "r"(o[5]), "r"(o[6]), "r"(o[7])
                 : "memory");
}
__device__ __forceinline__ uint32_t hmax2_u32(uint32_t a, uint32_t b) {
    __half2 r = __hmax2(*reinterpret_cast<__half2*>(&a), *reinterpret_cast<__half2*>(&b));
    return *reinterpret_cast<uint32_t*>(&r);
}

template <bool kOut2>
__global__ void __launch_bounds__(128) maxpool3x3s2_f16_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                               int8_t* __restrict__ y2, PoolParams p) {
    const int cv16 = p.cs / 16;
    const int bw = (p.PW + 1) / 2, bh = (p.PH + 1) / 2;
    const int64_t total = (int64_t)p.N * bh * bw * cv16;
    const uint32_t NEG = 0xFC00FC00u;   // (-inf, -inf): max pooling ignores the padding
    for (int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (int64_t)gridDim.x * blockDim.x) {
        const int cv = (int)(idx % cv16);
        int64_t t = idx / cv16;
        const int bx = (int)(t % bw); t /= bw;
        const int by = (int)(t % bh);
        const int n = (int)(t / bh);
        const int ph0 = by * 2, pw0 = bx * 2;
        const int h0 = ph0 * 2 - p.pt, w0 = pw0 * 2 - p.pl;
        uint32_t acc[2][2][8];
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b)
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[a][b][k] = NEG;
#pragma unroll
        for (int r = 0; r < 5; ++r) {
            const int h = h0 + r;
            if (h < 0 || h >= p.H) continue;
            uint32_t hm0[8], hm1[8];   // horizontal maxima of this input row for the two output columns
#pragma unroll
            for (int k = 0; k < 8; ++k) hm0[k] = hm1[k] = NEG;
#pragma unroll
            for (int c = 0; c < 5; ++c) {
                const int w = w0 + c;
                if (w < 0 || w >= p.W) continue;
                uint32_t v[8];
                ld256(x + (((int64_t)n * p.H + h) * p.W + w) * p.cs + cv * 16, v);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    if (c <= 2) hm0[k] = hmax2_u32(hm0[k], v[k]);
                    if (c >= 2) hm1[k] = hmax2_u32(hm1[k], v[k]);
                }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                if (r <= 2) { acc[0][0][k] = hmax2_u32(acc[0][0][k], hm0[k]); acc[0][1][k] = hmax2_u32(acc[0][1][k], hm1[k]); }
                if (r >= 2) { acc[1][0][k] = hmax2_u32(acc[1][0][k], hm0[k]); acc[1][1][k] = hmax2_u32(acc[1][1][k], hm1[k]); }
            }
        }
#pragma unroll
        for (int a = 0; a < 2; ++a)
#pragma unroll
            for (int b = 0; b < 2; ++b) {
                const int ph = ph0 + a, pw = pw0 + b;
                if (ph >= p.PH || pw >= p.PW) continue;
                const int64_t o = (((int64_t)n * p.PH + ph) * p.PW + pw) * p.cs + cv * 16;
                st256(y + o, acc[a][b]);
                if (kOut2) {
                    alignas(16) int8_t q[16];
#pragma unroll
                    for (int k = 0; k < 8; ++k) {
                        const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&acc[a][b][k]));
                        q[2 * k] = (int8_t)quant_rne(f.x * p.out2_scale);
                        q[2 * k + 1] = (int8_t)quant_rne(f.y * p.out2_scale);
                    }
                    *reinterpret_cast<uint4*>(y2 + o) = *reinterpret_cast<const uint4*>(q);
                }
            }
    }
}

int pool_dim(int in, int pa, int pb, int k, int s, int pad_mode) {
    // static_cast<int>(ceil|floor(static_cast<float>(in + pa + pb - k) / s)) + 1
    float q = (float)(in + pa + pb - k) / (float)s;
    return (int)(pad_mode == 0 ? ceilf(q) : floorf(q)) + 1;
}

template <typename T>
int launch(exb_ctx* ctx, const exb_pool_desc* d, const PoolParams& p, const void* x, void* y, void* y2,
           cudaStream_t st) {
    constexpr int V = PV<T>::N;
    if (p.cs % V != 0)
        return fail(EXB_ERR_UNSUPPORTED, "pooling needs the physical channel count (%d) to be a multiple of %d for this dtype", p.cs, V);
    const bool out2 = d->out2_dtype == EXB_I8;
    if (d->global_pool) {
        EXB_REQUIRE(p.N <= 65535, "batch %d exceeds the grid limit of global pooling", p.N);
        dim3 grid((p.cs / V + 31) / 32, p.N);
        if (out2) global_pool_kernel<T, true><<<grid, 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), static_cast<int8_t*>(y2), p);
        else global_pool_kernel<T, false><<<grid, 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), nullptr, p);
        return after_launch("global_pool_kernel");
    }
    if (std::is_same<T, __half>::value && p.type == 0 && p.kh == 3 && p.kw == 3 && p.sh == 2 && p.sw == 2 &&
        p.cs % 16 == 0 && p.pt <= 1 && p.pl <= 1) {
        const int64_t work = (int64_t)p.N * ((p.PH + 1) / 2) * ((p.PW + 1) / 2) * (p.cs / 16);
        const int g2 = stream_grid(ctx, work, 128, 16);
        if (out2) maxpool3x3s2_f16_kernel<true><<<g2, 128, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), static_cast<int8_t*>(y2), p);
        else maxpool3x3s2_f16_kernel<false><<<g2, 128, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), nullptr, p);
        return after_launch("maxpool3x3s2_f16_kernel");
    }
    const int64_t total = (int64_t)p.N * p.PH * p.PW * (p.cs / V);
    const int grid = stream_grid(ctx, total, 256);
    if (out2) pool_kernel<T, true><<<grid, 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), static_cast<int8_t*>(y2), p);
    else pool_kernel<T, false><<<grid, 256, 0, st>>>(static_cast<const T*>(x), static_cast<T*>(y), nullptr, p);
    return after_launch("pool_kernel");
}

int fill_params(const exb_pool_desc* d, PoolParams& p) {
    EXB_REQUIRE(d != nullptr, "null pooling descriptor");
    EXB_REQUIRE(d->N >= 0 && d->H > 0 && d->W > 0 && d->C > 0, "bad pooling input shape");
    EXB_REQUIRE(d->type == 0 || d->type == 1, "unknown pooling method %d", d->type);
    EXB_REQUIRE(d->pad_mode == 0 || d->pad_mode == 1, "pad_mode %d is not implemented", d->pad_mode);
    p.N = d->N; p.H = d->H; p.W = d->W; p.C = d->C;
    p.cs = d->c_stride ? d->c_stride : d->C;
    EXB_REQUIRE(p.cs >= p.C, "c_stride %d < C %d", p.cs, p.C);
    p.type = d->type;
    if (d->global_pool) {
        p.kh = d->H; p.kw = d->W; p.sh = p.sw = 1; p.pt = p.pb = p.pl = p.pr = 0;
    } else {
        p.kh = d->kh; p.kw = d->kw; p.sh = d->stride_h; p.sw = d->stride_w;
        p.pt = d->pad_t; p.pb = d->pad_b; p.pl = d->pad_l; p.pr = d->pad_r;
    }
    EXB_REQUIRE(p.kh > 0 && p.kw > 0 && p.sh > 0 && p.sw > 0, "bad pooling window / stride");
    EXB_REQUIRE(p.pt >= 0 && p.pb >= 0 && p.pl >= 0 && p.pr >= 0, "negative pooling pad");
    p.PH = pool_dim(p.H, p.pt, p.pb, p.kh, p.sh, d->pad_mode);
    p.PW = pool_dim(p.W, p.pl, p.pr, p.kw, p.sw, d->pad_mode);
    EXB_REQUIRE(p.PH > 0 && p.PW > 0, "pooling window larger than the padded input");
    p.count_include_pad = d->count_include_pad;
    p.out2_scale = d->out2_scale;
    return EXB_OK;
}

}  // namespace
}  // namespace exb

using namespace exb;

extern "C" int exb_pool_out_dims(const exb_pool_desc* d, int* PH, int* PW) {
    PoolParams p;
    if (int rc = fill_params(d, p)) return rc;
    EXB_REQUIRE(PH && PW, "null output pointer");
    *PH = p.PH;
    *PW = p.PW;
    return EXB_OK;
}

extern "C" int exb_pool2d_fwd(exb_ctx* ctx, const exb_pool_desc* d, const void* x, void* y, void* y2,
                              void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    PoolParams p;
    if (int rc = fill_params(d, p)) return rc;
    if (p.N == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_pool2d_fwd: null buffer");
    EXB_REQUIRE(aligned16(x) && aligned16(y), "exb_pool2d_fwd: buffers must be 16-byte aligned");
    if (d->out2_dtype != -1) {
        if (d->out2_dtype != EXB_I8) return fail(EXB_ERR_UNSUPPORTED, "pooling second output must be EXB_I8");
        EXB_REQUIRE(y2 && aligned16(y2), "exb_pool2d_fwd: second output null or misaligned");
    }
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (d->dtype) {
    case EXB_F16: return launch<__half>(ctx, d, p, x, y, y2, st);
    case EXB_F32: return launch<float>(ctx, d, p, x, y, y2, st);
    case EXB_I8:
        if (d->type != 0) return fail(EXB_ERR_UNSUPPORTED, "int8 pooling supports max only");
        if (d->out2_dtype != -1) return fail(EXB_ERR_UNSUPPORTED, "int8 pooling has no second output");
        return launch<int8_t>(ctx, d, p, x, y, y2, st);
    default: return fail(EXB_ERR_UNSUPPORTED, "pooling dtype %d", d->dtype);
    }
}
