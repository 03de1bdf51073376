// API-edge converts between the reference's NCHW fp32 tensors and the NHWC fp16 / int8
// buffers the kernels use.  Both directions go through a shared-memory transpose tile so
// that global reads and writes are both coalesced (reads along W, writes along C or back).
#include <algorithm>

#include "common.cuh"

namespace exb {
namespace {

constexpr int kTile = 32;  // 32 (hw) x 32 (c) transpose tile, 32x8 threads

template <typename Out> __device__ __forceinline__ Out cvt_out(float v, float scale, int rounding);
template <> __device__ __forceinline__ __half cvt_out<__half>(float v, float, int) { return __float2half_rn(v); }
template <> __device__ __forceinline__ int8_t cvt_out<int8_t>(float v, float scale, int rounding) {
    return (int8_t)(rounding ? quant_rne(v * scale) : quant_half_away(v * scale));
}
template <> __device__ __forceinline__ float cvt_out<float>(float v, float, int) { return v; }

// x: [N][C][HW] fp32  ->  y: [N][HW][c_stride] Out, channels >= C written as zero.
template <typename Out>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const float* __restrict__ x, Out* __restrict__ y,
                                                           int C, int HW, int c_stride, float scale, int rounding) {
    __shared__ float tile[kTile][kTile + 1];
    const int n = blockIdx.z;
    const int hw0 = blockIdx.x * kTile, c0 = blockIdx.y * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
    for (int j = ty; j < kTile; j += 8) {
        int c = c0 + j, hw = hw0 + tx;
        tile[j][tx] = (c < C && hw < HW) ? x[((int64_t)n * C + c) * HW + hw] : 0.f;
    }
    __syncthreads();
    for (int j = ty; j < kTile; j += 8) {
        int hw = hw0 + j, c = c0 + tx;
        if (hw < HW && c < c_stride)
            y[((int64_t)n * HW + hw) * c_stride + c] = cvt_out<Out>(tile[tx][j], scale, rounding);
    }
}

template <typename In> __device__ __forceinline__ float cvt_in(In v, float scale);
template <> __device__ __forceinline__ float cvt_in<__half>(__half v, float) { return __half2float(v); }
template <> __device__ __forceinline__ float cvt_in<int8_t>(int8_t v, float scale) { return (float)v * scale; }
template <> __device__ __forceinline__ float cvt_in<float>(float v, float) { return v; }

// x: [N][HW][c_stride] In  ->  y: [N][C][HW] fp32.
template <typename In>
__global__ void __launch_bounds__(256) nhwc_to_nchw_kernel(const In* __restrict__ x, float* __restrict__ y,
                                                           int C, int HW, int c_stride, float scale) {
    __shared__ float tile[kTile][kTile + 1];
    const int n = blockIdx.z;
    const int hw0 = blockIdx.x * kTile, c0 = blockIdx.y * kTile;
    const int tx = threadIdx.x, ty = threadIdx.y;
    for (int j = ty; j < kTile; j += 8) {
        int hw = hw0 + j, c = c0 + tx;
        tile[j][tx] = (hw < HW && c < C) ? cvt_in<In>(x[((int64_t)n * HW + hw) * c_stride + c], scale) : 0.f;
    }
    __syncthreads();
    for (int j = ty; j < kTile; j += 8) {
        int c = c0 + j, hw = hw0 + tx;
        if (c < C && hw < HW) y[((int64_t)n * C + c) * HW + hw] = tile[tx][j];
    }
}

// Few channels (C <= 8, detection heads and masks): one thread per pixel reads its C values and writes
// them to the C planes; consecutive threads write consecutive addresses of every plane.
template <typename In>
__global__ void __launch_bounds__(256) nhwc_to_nchw_fewc_kernel(const In* __restrict__ x, float* __restrict__ y, int N,
                                                                int C, int HW, int c_stride, float scale) {
    const int64_t total = (int64_t)N * HW;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / HW, hw = i - n * HW;
        const In* px = x + i * c_stride;
        for (int c = 0; c < C; ++c) y[(n * C + c) * HW + hw] = cvt_in<In>(px[c], scale);
    }
}

// Few-channel images (C <= 8): one thread per output pixel slot.  Reads are coalesced along W in
// each of the C planes, the write is one 8- or 16-byte vector per pixel; padding pixels and
// channels are written as zero.
template <typename Out, int CS>
__global__ void __launch_bounds__(256) nchw_to_nhwc_padded_kernel(const float* __restrict__ x, Out* __restrict__ y,
                                                                  int N, int C, int H, int W, int w_pad, int w_pitch,
                                                                  float scale, int rounding) {
    const int64_t total = (int64_t)N * H * w_pitch;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int wp = (int)(i % w_pitch);
        const int64_t nh = i / w_pitch;
        const int h = (int)(nh % H);
        const int n = (int)(nh / H);
        const int w = wp - w_pad;
        alignas(16) Out v[CS];
#pragma unroll
        for (int c = 0; c < CS; ++c) {
            float f = 0.f;
            if (c < C && w >= 0 && w < W) f = x[(((int64_t)n * C + c) * H + h) * W + w];
            v[c] = cvt_out<Out>(f, scale, rounding);
        }
        Out* dst = y + i * CS;
        if (sizeof(Out) * CS == 16) *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(v);
        else if (sizeof(Out) * CS == 8) *reinterpret_cast<uint2*>(dst) = *reinterpret_cast<const uint2*>(v);
        else if (sizeof(Out) * CS == 4) *reinterpret_cast<uint32_t*>(dst) = *reinterpret_cast<const uint32_t*>(v);
        else {
#pragma unroll
            for (int c = 0; c < CS; ++c) dst[c] = v[c];
        }
    }
}

// Few-channel image (C <= 4) into a dense channel-last tensor of CS physical channels: one thread per pixel, C
// coalesced plane loads, optional y = x * mul[c] + add[c] (input normalisation, same fma as the stand-alone
// pass), conversion, CS * sizeof(Out) / 16 vector stores with the padding channels zero.
template <typename Out, int CS>
__global__ void __launch_bounds__(256) image_to_nhwc_kernel(const float* __restrict__ x, Out* __restrict__ y, int N, int C,
                                                            int64_t HW, const float* __restrict__ mul,
                                                            const float* __restrict__ add, float scale, int rounding) {
    const int64_t total = (int64_t)N * HW;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t n = i / HW, hw = i - n * HW;
        alignas(16) Out v[CS];
#pragma unroll
        for (int c = 0; c < CS; ++c) v[c] = cvt_out<Out>(0.f, scale, rounding);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (c < C) {
                float f = x[(n * C + c) * HW + hw];
                if (mul) f = fmaf(f, mul[c], add[c]);
                v[c] = cvt_out<Out>(f, scale, rounding);
            }
        }
        uint4* dst = reinterpret_cast<uint4*>(y + i * CS);
#pragma unroll
        for (int k = 0; k < (int)(CS * sizeof(Out) / 16); ++k) dst[k] = reinterpret_cast<const uint4*>(v)[k];
    }
}

// The same conversion for fp16 NHWC4 when W, w_pad and w_pitch are multiples of 4: one thread per
// four consecutive row slots, a 16-byte load from each plane and one 32-byte store; rows are
// addressed by blockIdx.y so no division is left in the loop.
// kNorm: y = x * mul[c] + add[c] first (input normalisation), an instantiation of its own.
template <bool kNorm>
__global__ void __launch_bounds__(256) nchw_to_nhwc4_f16_quad_kernel(const float* __restrict__ x, __half* __restrict__ y,
                                                                     int C, int H, int W, int w_pad, int w_pitch,
                                                                     int64_t rows, const float* __restrict__ mul,
                                                                     const float* __restrict__ add) {
    const int quads = w_pitch >> 2;
    const int64_t plane = (int64_t)H * W;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += (int64_t)gridDim.x * blockDim.y) {
        const int64_t n = row / H;
        const int h = (int)(row - n * H);
        const float* src = x + (n * C * H + h) * (int64_t)W;
        for (int q = threadIdx.x; q < quads; q += blockDim.x) {
            const int w = 4 * q - w_pad;
            float4 v[3];
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                v[c] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (c < C && w >= 0 && w < W) {
                    v[c] = *reinterpret_cast<const float4*>(src + c * plane + w);
                    if (kNorm) {
                        const float m = mul[c], a = add[c];
                        v[c] = make_float4(fmaf(v[c].x, m, a), fmaf(v[c].y, m, a), fmaf(v[c].z, m, a), fmaf(v[c].w, m, a));
                    }
                }
            }
            uint32_t o[8];
#define EXB_PACK(j, m)                                                            \
            {                                                                         \
                __half2 lo = __floats2half2_rn(v[0].m, v[1].m), hi = __floats2half2_rn(v[2].m, 0.f); \
                o[2 * j] = *reinterpret_cast<uint32_t*>(&lo);                         \
                o[2 * j + 1] = *reinterpret_cast<uint32_t*>(&hi);                     \
            }
            EXB_PACK(0, x) EXB_PACK(1, y) EXB_PACK(2, z) EXB_PACK(3, w)
#undef EXB_PACK
            uint4* dst = reinterpret_cast<uint4*>(y + (row * w_pitch + 4 * q) * 4);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
}

// The same from fp16 planes (an input converted to half precision on the host): 8-byte plane loads, pure
// byte shuffles, the same 32-byte store.
__global__ void __launch_bounds__(256) nchw_f16_to_nhwc4_f16_quad_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                                         int C, int H, int W, int w_pad, int w_pitch,
                                                                         int64_t rows) {
    const int quads = w_pitch >> 2;
    const int64_t plane = (int64_t)H * W;
    for (int64_t row = (int64_t)blockIdx.x * blockDim.y + threadIdx.y; row < rows; row += (int64_t)gridDim.x * blockDim.y) {
        const int64_t n = row / H;
        const int h = (int)(row - n * H);
        const __half* src = x + (n * C * H + h) * (int64_t)W;
        for (int q = threadIdx.x; q < quads; q += blockDim.x) {
            const int w = 4 * q - w_pad;
            uint2 v[3];
#pragma unroll
            for (int c = 0; c < 3; ++c) {
                v[c] = make_uint2(0u, 0u);
                if (c < C && w >= 0 && w < W) v[c] = *reinterpret_cast<const uint2*>(src + c * plane + w);
            }
            // pixel j of the quad: halves (c0, c1, c2, 0); pixel 0/1 sit in .x, 2/3 in .y of each plane's load
            uint32_t o[8];
            o[0] = __byte_perm(v[0].x, v[1].x, 0x5410); o[1] = v[2].x & 0xffffu;
            o[2] = __byte_perm(v[0].x, v[1].x, 0x7632); o[3] = v[2].x >> 16;
            o[4] = __byte_perm(v[0].y, v[1].y, 0x5410); o[5] = v[2].y & 0xffffu;
            o[6] = __byte_perm(v[0].y, v[1].y, 0x7632); o[7] = v[2].y >> 16;
            uint4* dst = reinterpret_cast<uint4*>(y + (row * w_pitch + 4 * q) * 4);
            dst[0] = make_uint4(o[0], o[1], o[2], o[3]);
            dst[1] = make_uint4(o[4], o[5], o[6], o[7]);
        }
    }
}

int check_dims(const exb_ctx* ctx, const void* a, const void* b, int N, int C, int H, int W, int c_stride) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && C > 0 && H > 0 && W > 0, "bad tensor shape %dx%dx%dx%d", N, C, H, W);
    EXB_REQUIRE(c_stride >= C, "c_stride %d < C %d", c_stride, C);
    EXB_REQUIRE(N == 0 || (a && b), "null buffer");
    EXB_REQUIRE(N <= 65535, "batch %d exceeds the grid limit of this kernel", N);
    return EXB_OK;
}

}  // namespace
}  // namespace exb

using namespace exb;

extern "C" int exb_nchw_f32_to_nhwc(exb_ctx* ctx, const float* x, void* y, int dtype, int N, int C, int H,
                                    int W, int c_stride, float scale, int rounding, void* stream) {
    if (c_stride == 0) c_stride = C;
    if (int rc = check_dims(ctx, x, y, N, C, H, W, c_stride)) return rc;
    if (N == 0) return EXB_OK;
    const int HW = H * W;
    dim3 grid((HW + kTile - 1) / kTile, (c_stride + kTile - 1) / kTile, N), block(kTile, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (dtype) {
    case EXB_F16: nchw_to_nhwc_kernel<__half><<<grid, block, 0, st>>>(x, static_cast<__half*>(y), C, HW, c_stride, scale, rounding); break;
    case EXB_I8: nchw_to_nhwc_kernel<int8_t><<<grid, block, 0, st>>>(x, static_cast<int8_t*>(y), C, HW, c_stride, scale, rounding); break;
    case EXB_F32: nchw_to_nhwc_kernel<float><<<grid, block, 0, st>>>(x, static_cast<float*>(y), C, HW, c_stride, scale, rounding); break;
    default: return fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f32_to_nhwc: dtype %d", dtype);
    }
    return after_launch("nchw_to_nhwc_kernel");
}

extern "C" int exb_nhwc_to_nchw_f32(exb_ctx* ctx, const void* x, int dtype, float* y, int N, int C, int H,
                                    int W, int c_stride, float scale, void* stream) {
    if (c_stride == 0) c_stride = C;
    if (int rc = check_dims(ctx, x, y, N, C, H, W, c_stride)) return rc;
    if (N == 0) return EXB_OK;
    const int HW = H * W;
    dim3 grid((HW + kTile - 1) / kTile, (C + kTile - 1) / kTile, N), block(kTile, 8);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (C <= 8) {
        const int g = stream_grid(ctx, (int64_t)N * HW, 256);
        switch (dtype) {
        case EXB_F16: nhwc_to_nchw_fewc_kernel<__half><<<g, 256, 0, st>>>(static_cast<const __half*>(x), y, N, C, HW, c_stride, scale); break;
        case EXB_I8: nhwc_to_nchw_fewc_kernel<int8_t><<<g, 256, 0, st>>>(static_cast<const int8_t*>(x), y, N, C, HW, c_stride, scale); break;
        case EXB_F32: nhwc_to_nchw_fewc_kernel<float><<<g, 256, 0, st>>>(static_cast<const float*>(x), y, N, C, HW, c_stride, scale); break;
        default: return fail(EXB_ERR_UNSUPPORTED, "exb_nhwc_to_nchw_f32: dtype %d", dtype);
        }
        return after_launch("nhwc_to_nchw_fewc_kernel");
    }
    switch (dtype) {
    case EXB_F16: nhwc_to_nchw_kernel<__half><<<grid, block, 0, st>>>(static_cast<const __half*>(x), y, C, HW, c_stride, scale); break;
    case EXB_I8: nhwc_to_nchw_kernel<int8_t><<<grid, block, 0, st>>>(static_cast<const int8_t*>(x), y, C, HW, c_stride, scale); break;
    case EXB_F32: nhwc_to_nchw_kernel<float><<<grid, block, 0, st>>>(static_cast<const float*>(x), y, C, HW, c_stride, scale); break;
    default: return fail(EXB_ERR_UNSUPPORTED, "exb_nhwc_to_nchw_f32: dtype %d", dtype);
    }
    return after_launch("nhwc_to_nchw_kernel");
}

extern "C" int exb_nchw_f32_to_nhwc_padded(exb_ctx* ctx, const float* x, void* y, int dtype, int N, int C, int H,
                                           int W, int c_stride, int w_pad, int w_pitch, float scale, int rounding,
                                           void* stream) {
    if (c_stride == 0) c_stride = C;
    if (int rc = check_dims(ctx, x, y, N, C, H, W, c_stride)) return rc;
    EXB_REQUIRE(w_pad >= 0 && w_pitch >= W + w_pad, "bad row padding (w_pad %d, w_pitch %d, W %d)", w_pad, w_pitch, W);
    if (c_stride != 4 && c_stride != 8)
        return fail(EXB_ERR_UNSUPPORTED, "padded ingest supports c_stride 4 or 8, got %d", c_stride);
    if (N == 0) return EXB_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == EXB_F16 && c_stride == 4 && C <= 3 && (W & 3) == 0 && (w_pad & 3) == 0 && (w_pitch & 3) == 0 &&
        aligned16(x) && aligned16(y)) {
        const int64_t rows = (int64_t)N * H;
        const dim3 block(64, 4);
        const int grid = (int)std::min<int64_t>((rows + 3) / 4, (int64_t)ctx->sm_count * 32);
        nchw_to_nhwc4_f16_quad_kernel<false><<<grid, block, 0, st>>>(x, static_cast<__half*>(y), C, H, W, w_pad, w_pitch, rows,
                                                                     nullptr, nullptr);
        return after_launch("nchw_to_nhwc4_f16_quad_kernel");
    }
    const int grid = stream_grid(ctx, (int64_t)N * H * w_pitch, 256, 16);
#define EXB_LAUNCH(T, CS) nchw_to_nhwc_padded_kernel<T, CS><<<grid, 256, 0, st>>>(x, static_cast<T*>(y), N, C, H, W, w_pad, w_pitch, scale, rounding)
    if (dtype == EXB_F16) { if (c_stride == 4) EXB_LAUNCH(__half, 4); else EXB_LAUNCH(__half, 8); }
    else if (dtype == EXB_I8) { if (c_stride == 4) EXB_LAUNCH(int8_t, 4); else EXB_LAUNCH(int8_t, 8); }
    else return fail(EXB_ERR_UNSUPPORTED, "padded ingest supports EXB_F16 and EXB_I8 output");
#undef EXB_LAUNCH
    return after_launch("nchw_to_nhwc_padded_kernel");
}

// Input normalisation fused into the ingest: y = convert(x * mul[c] + add[c]).
extern "C" int exb_image_f32_to_nhwc_norm(exb_ctx* ctx, const float* x, void* y, int dtype, int N, int C, int H, int W,
                                          int c_stride, const float* mul, const float* add, float scale, int rounding,
                                          void* stream) {
    if (int rc = check_dims(ctx, x, y, N, C, H, W, c_stride)) return rc;
    EXB_REQUIRE((mul == nullptr) == (add == nullptr), "exb_image_f32_to_nhwc_norm: mul and add come together");
    if (C > 4) return fail(EXB_ERR_UNSUPPORTED, "exb_image_f32_to_nhwc_norm takes images of up to 4 channels, got %d", C);
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(aligned16(y), "exb_image_f32_to_nhwc_norm: misaligned output");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t HW = (int64_t)H * W;
    const int grid = stream_grid(ctx, (int64_t)N * HW, 256, 16);
    if (dtype == EXB_F16 && c_stride == 16)
        image_to_nhwc_kernel<__half, 16><<<grid, 256, 0, st>>>(x, static_cast<__half*>(y), N, C, HW, mul, add, scale, rounding);
    else if (dtype == EXB_F16 && c_stride == 8)
        image_to_nhwc_kernel<__half, 8><<<grid, 256, 0, st>>>(x, static_cast<__half*>(y), N, C, HW, mul, add, scale, rounding);
    else if (dtype == EXB_I8 && c_stride == 32)
        image_to_nhwc_kernel<int8_t, 32><<<grid, 256, 0, st>>>(x, static_cast<int8_t*>(y), N, C, HW, mul, add, scale, rounding);
    else if (dtype == EXB_I8 && c_stride == 16)
        image_to_nhwc_kernel<int8_t, 16><<<grid, 256, 0, st>>>(x, static_cast<int8_t*>(y), N, C, HW, mul, add, scale, rounding);
    else
        return fail(EXB_ERR_UNSUPPORTED, "exb_image_f32_to_nhwc_norm: dtype %d with channel stride %d", dtype, c_stride);
    return after_launch("image_to_nhwc_kernel");
}

extern "C" int exb_nchw_f32_to_nhwc4_padded_norm(exb_ctx* ctx, const float* x, void* y, int N, int C, int H, int W, int w_pad,
                                                 int w_pitch, const float* mul, const float* add, void* stream) {
    if (int rc = check_dims(ctx, x, y, N, C, H, W, 4)) return rc;
    EXB_REQUIRE(w_pad >= 0 && w_pitch >= W + w_pad, "bad row padding (w_pad %d, w_pitch %d, W %d)", w_pad, w_pitch, W);
    EXB_REQUIRE(mul != nullptr && add != nullptr, "exb_nchw_f32_to_nhwc4_padded_norm: null coefficients");
    if (C > 3 || (W & 3) || (w_pad & 3) || (w_pitch & 3))
        return fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f32_to_nhwc4_padded_norm needs C <= 3 and W, w_pad, w_pitch multiples of 4");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(aligned16(x) && aligned16(y), "exb_nchw_f32_to_nhwc4_padded_norm: misaligned buffer");
    const int64_t rows = (int64_t)N * H;
    const dim3 block(64, 4);
    const int grid = (int)std::min<int64_t>((rows + 3) / 4, (int64_t)ctx->sm_count * 32);
    nchw_to_nhwc4_f16_quad_kernel<true><<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(x, static_cast<__half*>(y), C, H, W,
                                                                                                w_pad, w_pitch, rows, mul, add);
    return after_launch("nchw_to_nhwc4_f16_quad_kernel");
}

extern "C" int exb_nchw_f16_to_nhwc4_padded(exb_ctx* ctx, const void* x, void* y, int N, int C, int H, int W, int w_pad,
                                            int w_pitch, void* stream) {
    if (int rc = check_dims(ctx, x, y, N, C, H, W, 4)) return rc;
    EXB_REQUIRE(w_pad >= 0 && w_pitch >= W + w_pad, "bad row padding (w_pad %d, w_pitch %d, W %d)", w_pad, w_pitch, W);
    if (C > 3 || (W & 3) || (w_pad & 3) || (w_pitch & 3))
        return fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f16_to_nhwc4_padded needs C <= 3 and W, w_pad, w_pitch multiples of 4");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE((reinterpret_cast<uintptr_t>(x) & 7u) == 0 && aligned16(y), "exb_nchw_f16_to_nhwc4_padded: misaligned buffer");
    const int64_t rows = (int64_t)N * H;
    const dim3 block(64, 4);
    const int grid = (int)std::min<int64_t>((rows + 3) / 4, (int64_t)ctx->sm_count * 32);
    nchw_f16_to_nhwc4_f16_quad_kernel<<<grid, block, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), static_cast<__half*>(y), C, H, W, w_pad, w_pitch, rows);
    return after_launch("nchw_f16_to_nhwc4_f16_quad_kernel");
}

namespace exb {
namespace {
// Network input -> Focus in one pass: fp32 NCHW image, optional per-channel affine (input normalisation),
// space-to-depth 2x2 and conversion to channel-last fp16.  One thread per output pixel: two float2 loads per
// input plane (rows 2i and 2i+1, columns 2j and 2j+1), CS / 8 16-byte stores.  4*C <= CS.
// C is a template parameter so that the output vector is indexed statically and stays in registers.
template <int CS, int C>
__global__ void __launch_bounds__(256) focus_ingest_kernel(const float* __restrict__ x, __half* __restrict__ y, int N,
                                                           int H, int W, const float* __restrict__ mul,
                                                           const float* __restrict__ add) {
    const int OH = H / 2, OW = W / 2;
    const int64_t total = (int64_t)N * OH * OW;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int oj = (int)(i % OW);
        const int64_t t = i / OW;
        const int oi = (int)(t % OH);
        const int n = (int)(t / OH);
        alignas(16) __half out[CS];
#pragma unroll
        for (int k = 0; k < CS; ++k) out[k] = __float2half_rn(0.f);
#pragma unroll
        for (int c = 0; c < C; ++c) {
            const float* p0 = x + (((int64_t)n * C + c) * H + 2 * oi) * W + 2 * oj;
            const float2 top = *reinterpret_cast<const float2*>(p0);
            const float2 bot = *reinterpret_cast<const float2*>(p0 + W);
            const float m = mul ? mul[c] : 1.f, a = add ? add[c] : 0.f;
            // group g reads row 2i + g%2, column 2j + g/2
            out[0 * C + c] = __float2half_rn(fmaf(top.x, m, a));
            out[1 * C + c] = __float2half_rn(fmaf(bot.x, m, a));
            out[2 * C + c] = __float2half_rn(fmaf(top.y, m, a));
            out[3 * C + c] = __float2half_rn(fmaf(bot.y, m, a));
        }
        uint4* dst = reinterpret_cast<uint4*>(y + i * CS);
#pragma unroll
        for (int k = 0; k < CS / 8; ++k) dst[k] = reinterpret_cast<const uint4*>(out)[k];
    }
}
}  // namespace
}  // namespace exb

extern "C" int exb_nchw_f32_focus_to_nhwc_f16(exb_ctx* ctx, const float* x, void* y, int N, int C, int H, int W,
                                              int c_stride, const float* mul, const float* add, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && C > 0 && H > 0 && W > 0, "exb_nchw_f32_focus_to_nhwc_f16: bad shape");
    if (H % 2 || W % 2) return exb::fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f32_focus_to_nhwc_f16 needs even H and W, got %d x %d", H, W);
    if ((c_stride != 16 && c_stride != 32) || 4 * C > c_stride)
        return exb::fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f32_focus_to_nhwc_f16: channel stride %d for %d input channels", c_stride, C);
    EXB_REQUIRE((mul == nullptr) == (add == nullptr), "exb_nchw_f32_focus_to_nhwc_f16: mul and add come together");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(x && y && exb::aligned16(y) && (reinterpret_cast<uintptr_t>(x) & 7u) == 0,
                "exb_nchw_f32_focus_to_nhwc_f16: null or misaligned buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = exb::stream_grid(ctx, (int64_t)N * (H / 2) * (W / 2), 256);
    __half* yh = static_cast<__half*>(y);
#define EXB_FOCUS(CS, CC) exb::focus_ingest_kernel<CS, CC><<<grid, 256, 0, st>>>(x, yh, N, H, W, mul, add)
    if (c_stride == 16) {
        if (C == 1) EXB_FOCUS(16, 1); else if (C == 2) EXB_FOCUS(16, 2); else if (C == 3) EXB_FOCUS(16, 3); else EXB_FOCUS(16, 4);
    } else {
        switch (C) {
        case 1: EXB_FOCUS(32, 1); break;
        case 2: EXB_FOCUS(32, 2); break;
        case 3: EXB_FOCUS(32, 3); break;
        case 4: EXB_FOCUS(32, 4); break;
        default: return exb::fail(EXB_ERR_UNSUPPORTED, "exb_nchw_f32_focus_to_nhwc_f16: %d input channels (1..4 are implemented)", C);
        }
    }
#undef EXB_FOCUS
    return exb::after_launch("exb_nchw_f32_focus_to_nhwc_f16");
}
