// Graph-glue kernels around the convolution trunk: channel concatenation, nearest-neighbour
// resize and the per-channel affine map (BatchNorm at inference, input normalisation).  All three
// are single-pass, bandwidth-bound copies; 16-byte vectors where strides allow, scalars otherwise.
#include "common.cuh"

namespace exb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxConcatInputs = 8;

struct ConcatArgs {
    const void* x[kMaxConcatInputs];
    int64_t width[kMaxConcatInputs];     // valid elements per row of input i
    int64_t stride[kMaxConcatInputs];    // physical elements per row of input i
    int64_t offset[kMaxConcatInputs + 1];  // first output column of input i; [n_in] = total width
    int n_in;
};

// y[r][offset_i + k] = x_i[r][k].  Unit = 1 << unit_shift bytes moved per thread step (16 when every
// width, stride and offset is a multiple of 16 bytes, else one element).
template <typename U>
__global__ void __launch_bounds__(kThreads) concat_rows_kernel(ConcatArgs a, U* y, int64_t y_stride, int64_t rows) {
    const int64_t total = a.offset[a.n_in];
    const int64_t work = rows * total;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int64_t r = i / total, c = i - r * total;
        int k = 0;
#pragma unroll
        for (int j = 1; j < kMaxConcatInputs; ++j)
            if (j < a.n_in && c >= a.offset[j]) k = j;
        y[r * y_stride + c] = static_cast<const U*>(a.x[k])[r * a.stride[k] + (c - a.offset[k])];
    }
}

// Nearest resize, channel-last: one thread per 16-byte (or one-element) slice of an output pixel.
template <typename U>
__global__ void __launch_bounds__(kThreads) interp_nearest_nhwc_kernel(const U* x, U* y, int N, int H, int W, int cs,
                                                                       int OH, int OW, float hs, float ws) {
    const int64_t work = (int64_t)N * OH * OW * cs;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int c = (int)(i % cs);
        int64_t p = i / cs;
        const int ox = (int)(p % OW);
        p /= OW;
        const int oy = (int)(p % OH);
        const int n = (int)(p / OH);
        const int iy = min((int)(oy * hs), H - 1), ix = min((int)(ox * ws), W - 1);
        y[i] = x[(((int64_t)n * H + iy) * W + ix) * cs + c];
    }
}

__global__ void __launch_bounds__(kThreads) interp_nearest_nchw_kernel(const float* x, float* y, int planes, int H, int W,
                                                                       int OH, int OW, float hs, float ws) {
    const int64_t work = (int64_t)planes * OH * OW;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int ox = (int)(i % OW);
        int64_t p = i / OW;
        const int oy = (int)(p % OH);
        const int64_t pl = p / OH;
        const int iy = min((int)(oy * hs), H - 1), ix = min((int)(ox * ws), W - 1);
        y[i] = x[(pl * H + iy) * W + ix];
    }
}

// Space-to-depth 2x2: output channel g*C + c of pixel (i, j) is input channel c of pixel
// (2i + g%2, 2j + g/2).  One thread per output element; the input is a few-channel image.
template <typename T>
__global__ void __launch_bounds__(kThreads) focus_kernel(const T* __restrict__ x, T* __restrict__ y, int N, int C, int H,
                                                         int W, int in_stride, int out_stride, int channel_last) {
    const int OH = H / 2, OW = W / 2, OC = 4 * C;
    const int ocs = channel_last ? out_stride : OC;
    const int64_t work = (int64_t)N * OH * OW * ocs;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        int n, pc, oi, oj;
        int64_t t = i;
        if (channel_last) {
            pc = (int)(t % ocs); t /= ocs;
            oj = (int)(t % OW); t /= OW;
            oi = (int)(t % OH);
            n = (int)(t / OH);
        } else {
            oj = (int)(t % OW); t /= OW;
            oi = (int)(t % OH); t /= OH;
            pc = (int)(t % OC);
            n = (int)(t / OC);
        }
        T v = T(0);
        if (pc < OC) {
            const int g = pc / C, c = pc - g * C;
            const int ih = 2 * oi + (g & 1), iw = 2 * oj + (g >> 1);
            v = channel_last ? x[(((int64_t)n * H + ih) * W + iw) * in_stride + c]
                             : x[(((int64_t)n * C + c) * H + ih) * W + iw];
        }
        y[i] = v;
    }
}

__device__ __forceinline__ float bin_apply(int op, float a, float b) {
    return op == 0 ? a + b : (op == 1 ? a - b : (op == 2 ? a * b : a / b));
}
__device__ __forceinline__ float ld1(const __half* p) { return __half2float(*p); }
__device__ __forceinline__ float ld1(const float* p) { return *p; }
__device__ __forceinline__ void st1(__half* p, float v) { *p = __float2half_rn(v); }
__device__ __forceinline__ void st1(float* p, float v) { *p = v; }

// y = act(x * mul[c] + add[c]).  channel-last: c = i % cs (padding channels c >= C are written 0);
// planar: c = (i / inner) % C.
template <typename T>
__global__ void __launch_bounds__(kThreads) channel_affine_kernel(const T* x, T* y, const float* mul, const float* add,
                                                                  int64_t count, int C, int cs, int64_t inner,
                                                                  int channel_last, int act, const float* slope,
                                                                  int n_slope) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
        const int c = channel_last ? (int)(i % cs) : (int)((i / inner) % C);
        float v = 0.f;
        if (c < C) {
            v = fmaf(ld1(x + i), mul[c], add[c]);
            if (slope) v = v >= 0.f ? v : v * slope[n_slope == 1 ? 0 : c];
            else v = apply_act(v, act);
        }
        st1(y + i, v);
    }
}


// Channel-last fp16, 8 channels (16 bytes) per thread step: y = f(x * mul[c] + add[c]) with f the activation
// `act`, or the PReLU with `slope` when that is not null; mul == null means no affine map (plain PReLU).
// cs is a multiple of 8; padding channels are written 0.  When the grid stride is a multiple of the vectors
// per pixel (the launcher arranges that), a thread keeps its channel slice for the whole loop and the per-
// channel parameters are loaded once.
__global__ void __launch_bounds__(kThreads) channel_affine_nhwc_f16x8_kernel(const uint4* x, uint4* y, const float* mul,
                                                                             const float* add, const float* slope,
                                                                             int n_slope, int act, int64_t nvec, int C,
                                                                             int cs8) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    const bool fixed = step % cs8 == 0;
    float m[8], a[8], sl[8];
    auto load_params = [&](int c0) {
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const int c = c0 + k;
            const bool in = c < C;
            m[k] = in ? (mul ? mul[c] : 1.f) : 0.f;
            a[k] = in && mul ? add[c] : 0.f;
            sl[k] = in && slope ? slope[n_slope == 1 ? 0 : c] : 0.f;
        }
    };
    const int64_t first = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    auto one = [&](uint4 raw, int c0) -> uint4 {
        __half2* h = reinterpret_cast<__half2*>(&raw);
        float v[8];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 f = __half22float2(h[k]);
            v[2 * k] = f.x;
            v[2 * k + 1] = f.y;
        }
#pragma unroll
        for (int k = 0; k < 8; ++k) v[k] = fmaf(v[k], m[k], a[k]);       // padding channels: m = a = 0
        if (slope) {
#pragma unroll
            for (int k = 0; k < 8; ++k) v[k] = v[k] >= 0.f ? v[k] : v[k] * sl[k];
        } else {
            apply_act_vec(v, act);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c0 + k >= C) v[k] = 0.f;
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) h[k] = __floats2half2_rn(v[2 * k], v[2 * k + 1]);
        return raw;
    };
    int64_t i = first;
    if (fixed) {
        const int c0 = (int)(first % cs8) * 8;
        load_params(c0);
        // four independent 16-byte loads in flight per thread
        for (; i + 3 * step < nvec; i += 4 * step) {
            uint4 r[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) r[u] = x[i + u * step];
#pragma unroll
            for (int u = 0; u < 4; ++u) y[i + u * step] = one(r[u], c0);
        }
        for (; i < nvec; i += step) y[i] = one(x[i], c0);
        return;
    }
    for (; i < nvec; i += step) {
        const int c0 = (int)(i % cs8) * 8;
        load_params(c0);
        y[i] = one(x[i], c0);
    }
}

// The per-channel gate on channel-last fp16: y = a op b[n][c] (or b op a), 8 channels per thread step.
__global__ void __launch_bounds__(kThreads) binary_bcast_nhwc_f16x8_kernel(const uint4* a, const uint4* b, uint4* y, int64_t nvec,
                                                                           int C, int cs8, int64_t vec_per_image, int op,
                                                                           int b_batch, int b_first) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += step) {
        const int cv = (int)(i % cs8);
        const int64_t n = i / vec_per_image;
        uint4 ra = a[i];
        const uint4 rb = b[(n % b_batch) * cs8 + cv];
        __half2* ha = reinterpret_cast<__half2*>(&ra);
        const __half2* hb = reinterpret_cast<const __half2*>(&rb);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float2 fa = __half22float2(ha[k]), fb = __half22float2(hb[k]);
            float2 r;
            r.x = b_first ? bin_apply(op, fb.x, fa.x) : bin_apply(op, fa.x, fb.x);
            r.y = b_first ? bin_apply(op, fb.y, fa.y) : bin_apply(op, fa.y, fb.y);
            if (cv * 8 + 2 * k >= C) r.x = 0.f;
            if (cv * 8 + 2 * k + 1 >= C) r.y = 0.f;
            ha[k] = __floats2half2_rn(r.x, r.y);
        }
        y[i] = ra;
    }
}

// y = x >= 0 ? x : x * slope[c] (PReLU; one shared slope when n_slope == 1, which is also LeakyReLU).
// Indexing as channel_affine_kernel; padding channels of a channel-last tensor are written 0.
template <typename T>
__global__ void __launch_bounds__(kThreads) prelu_kernel(const T* x, T* y, const float* slope, int n_slope, int64_t count,
                                                         int C, int cs, int64_t inner, int channel_last) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
        const int c = channel_last ? (int)(i % cs) : (int)((i / inner) % C);
        float v = 0.f;
        if (c < C) {
            v = ld1(x + i);
            v = v >= 0.f ? v : v * slope[n_slope == 1 ? 0 : c];
        }
        st1(y + i, v);
    }
}

// Depth-to-space: y[n][h*rh + a][w*rw + b][c] = x[n][h][w][(a*rw + b)*C + c]; channels c >= C of y are 0.
// One thread per output element (U = one element of the tensor's type).
template <typename U>
__global__ void __launch_bounds__(kThreads) depth_to_space_kernel(const U* __restrict__ x, U* __restrict__ y, int N, int H,
                                                                  int W, int rh, int rw, int C, int xs, int ys) {
    const int OH = H * rh, OW = W * rw;
    const int64_t work = (int64_t)N * OH * OW * ys;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int c = (int)(i % ys);
        int64_t p = i / ys;
        const int ox = (int)(p % OW);
        p /= OW;
        const int oy = (int)(p % OH);
        const int n = (int)(p / OH);
        U v = U(0);
        if (c < C) {
            const int h = oy / rh, a = oy - h * rh, w = ox / rw, b = ox - w * rw;
            v = x[(((int64_t)n * H + h) * W + w) * xs + (a * rw + b) * C + c];
        }
        y[i] = v;
    }
}

// The same with one 16-byte vector of 8 fp16 channels per thread step; C, xs and ys are multiples of 8 when
// kGather is false (one aligned load), otherwise the 8 values are gathered one by one (C not a multiple of 8).
template <bool kGather>
__global__ void __launch_bounds__(kThreads) depth_to_space_f16x8_kernel(const __half* __restrict__ x, uint4* __restrict__ y,
                                                                        int N, int H, int W, int rh, int rw, int C, int xs,
                                                                        int ys8) {
    const int OH = H * rh, OW = W * rw;
    const int64_t work = (int64_t)N * OH * OW * ys8;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int c0 = (int)(i % ys8) * 8;
        int64_t p = i / ys8;
        const int ox = (int)(p % OW);
        p /= OW;
        const int oy = (int)(p % OH);
        const int n = (int)(p / OH);
        const int h = oy / rh, a = oy - h * rh, w = ox / rw, b = ox - w * rw;
        const __half* src = x + (((int64_t)n * H + h) * W + w) * xs + (a * rw + b) * C;
        uint4 v = make_uint4(0u, 0u, 0u, 0u);
        if (!kGather) {
            if (c0 < C) v = *reinterpret_cast<const uint4*>(src + c0);
        } else {
            __half* e = reinterpret_cast<__half*>(&v);
#pragma unroll
            for (int k = 0; k < 8; ++k)
                if (c0 + k < C) e[k] = src[c0 + k];
        }
        y[i] = v;
    }
}

// y[p][w][h] = x[p][h][w] for every plane p; 32x32 tiles through shared memory.
__global__ void __launch_bounds__(256) transpose_planes_f32_kernel(const float* __restrict__ x, float* __restrict__ y,
                                                                   int H, int W) {
    __shared__ float tile[32][33];
    const int64_t plane = blockIdx.z;
    const float* xp = x + plane * (int64_t)H * W;
    float* yp = y + plane * (int64_t)H * W;
    const int w0 = blockIdx.x * 32, h0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int r = ty; r < 32; r += 8)
        if (h0 + r < H && w0 + tx < W) tile[r][tx] = xp[(int64_t)(h0 + r) * W + w0 + tx];
    __syncthreads();
    for (int r = ty; r < 32; r += 8)
        if (w0 + r < W && h0 + tx < H) yp[(int64_t)(w0 + r) * H + h0 + tx] = tile[tx][r];
}


// y[n][c][p] = a[n][c][p] op b[n % b_batch][c] (or b op a when b_first): a per-channel value of every image
// applied to a whole map (squeeze-and-excitation gates).  Indexing as channel_affine_kernel; padding channels are written 0.
template <typename T>
__global__ void __launch_bounds__(kThreads) binary_bcast_kernel(const T* a, const T* b, T* y, int64_t count, int C, int cs,
                                                                int64_t inner, int channel_last, int op, int b_batch,
                                                                int b_first) {
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    const int64_t per_image = channel_last ? inner * cs : inner * C;
    const int bcs = channel_last ? cs : C;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count; i += step) {
        const int c = channel_last ? (int)(i % cs) : (int)((i / inner) % C);
        const int64_t n = i / per_image;
        float v = 0.f;
        if (c < C) {
            const float av = ld1(a + i), bv = ld1(b + (n % b_batch) * bcs + c);
            v = b_first ? bin_apply(op, bv, av) : bin_apply(op, av, bv);
        }
        st1(y + i, v);
    }
}


// Softmax over the C values of every (image, position): y[n][c][p] = exp(x - max_c) / sum_c exp(x - max_c).
// One thread per (n, p); C is small (class scores).  x may have a padded image stride.
__global__ void __launch_bounds__(kThreads) softmax_channels_kernel(const float* __restrict__ x, float* __restrict__ y, int N,
                                                                    int C, int64_t inner, int64_t x_image_stride) {
    const int64_t total = (int64_t)N * inner;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += step) {
        const int64_t n = i / inner, p = i - n * inner;
        const float* xp = x + n * x_image_stride + p;
        float* yp = y + n * C * inner + p;
        float m = xp[0];
        for (int c = 1; c < C; ++c) m = fmaxf(m, xp[c * inner]);
        float sum = 0.f;
        for (int c = 0; c < C; ++c) {
            const float e = expf(xp[c * inner] - m);
            yp[c * inner] = e;
            sum += e;
        }
        for (int c = 0; c < C; ++c) yp[c * inner] = yp[c * inner] / sum;
    }
}


// Detection-head export: y[n][a][p][k] = x[n][p][a*K + k] (channel-last fp16 in, fp32 out) - what a Reshape of the
// (N, A*K, H, W) head to (N, A, K, H*W) followed by a Transpose of the last two axes computes on NCHW data.
// A warp per position: the lanes read the A*K channels of the pixel (one contiguous run) and write A runs of K
// floats; channel -> (a, k) with a float reciprocal, exact for the few hundred channels of a head.
__global__ void __launch_bounds__(kThreads) split_heads_kernel(const __half* __restrict__ x, float* __restrict__ y, int64_t rows,
                                                               int P, int cs, int A, int K) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    const float inv_k = 1.0f / (float)K;
    const int C = A * K;
    for (int64_t r = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < rows; r += warps) {
        const int64_t n = r / P;
        const int p = (int)(r - n * P);
        const __half* src = x + r * cs;
        float* dst = y + (n * A * P + p) * (int64_t)K;
        for (int c = lane; c < C; c += 32) {
            const int a = (int)(((float)c + 0.5f) * inv_k);
            const int k = c - a * K;
            dst[(int64_t)a * P * K + k] = __half2float(src[c]);
        }
    }
}


// Depth-to-space of a channel-last fp16 tensor straight into an fp32 NCHW tensor (a transposed convolution whose
// result leaves the network): y[n][c][h*rh + a][w*rw + b] = x[n][h][w][(a*rw + b)*C + c].  One thread per output
// value, the output column fastest: writes are contiguous, reads of neighbouring threads fall into the same pixel.
__global__ void __launch_bounds__(kThreads) depth_to_space_nchw_f32_kernel(const __half* __restrict__ x, float* __restrict__ y,
                                                                           int N, int H, int W, int rh, int rw, int C, int xs) {
    const int OH = H * rh, OW = W * rw;
    const int64_t work = (int64_t)N * C * OH * OW;
    const int64_t step = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < work; i += step) {
        const int ox = (int)(i % OW);
        int64_t p = i / OW;
        const int oy = (int)(p % OH);
        p /= OH;
        const int c = (int)(p % C);
        const int n = (int)(p / C);
        const int h = oy / rh, a = oy - h * rh, w = ox / rw, b = ox - w * rw;
        y[i] = __half2float(x[(((int64_t)n * H + h) * W + w) * xs + (a * rw + b) * C + c]);
    }
}

}  // namespace
}  // namespace exb

using namespace exb;

// Grid for the 8-channel vector kernels: the grid stride (grid * kThreads vectors) a multiple of the vectors per
// pixel whenever that costs at most a few CTAs, so that a thread keeps its channel slice.
static int slice_grid(const exb_ctx* ctx, int64_t nvec, int cs8) {
    int grid = stream_grid(ctx, nvec, kThreads);
    int a = cs8, b = kThreads;
    while (b) { const int t = a % b; a = b; b = t; }
    const int q = cs8 / a;                      // grid must be a multiple of q
    if (q > 1 && grid >= q) grid = grid / q * q;
    return grid;
}

extern "C" int exb_concat_fwd(exb_ctx* ctx, int n_in, const void* const* xs, const int64_t* widths,
                              const int64_t* x_strides, void* y, int64_t y_stride, int64_t rows, int dtype,
                              void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(n_in >= 1 && xs && widths && x_strides, "exb_concat_fwd: null argument or no inputs");
    if (n_in > kMaxConcatInputs)
        return fail(EXB_ERR_UNSUPPORTED, "concat supports at most %d inputs, got %d", kMaxConcatInputs, n_in);
    const int64_t es = (int64_t)dtype_size(dtype);
    if (es == 0) return fail(EXB_ERR_UNSUPPORTED, "exb_concat_fwd: dtype %d", dtype);
    EXB_REQUIRE(rows >= 0, "exb_concat_fwd: negative row count");
    ConcatArgs a;
    a.n_in = n_in;
    int64_t off = 0;
    bool vec = aligned16(y) && (y_stride * es) % 16 == 0;
    for (int i = 0; i < n_in; ++i) {
        EXB_REQUIRE(widths[i] >= 0 && x_strides[i] >= widths[i], "exb_concat_fwd: input %d has stride < width", i);
        EXB_REQUIRE(xs[i] != nullptr || widths[i] == 0 || rows == 0, "exb_concat_fwd: input %d is null", i);
        a.x[i] = xs[i];
        a.width[i] = widths[i];
        a.stride[i] = x_strides[i];
        a.offset[i] = off;
        vec = vec && aligned16(xs[i]) && (widths[i] * es) % 16 == 0 && (x_strides[i] * es) % 16 == 0 && (off * es) % 16 == 0;
        off += widths[i];
    }
    a.offset[n_in] = off;
    for (int i = n_in + 1; i <= kMaxConcatInputs; ++i) a.offset[i] = off;
    EXB_REQUIRE(y_stride >= off, "exb_concat_fwd: output stride %lld smaller than the summed width %lld",
                (long long)y_stride, (long long)off);
    if (rows == 0 || off == 0) return EXB_OK;
    EXB_REQUIRE(y != nullptr, "exb_concat_fwd: null output");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec) {
        const int64_t per = 16 / es;
        for (int i = 0; i < n_in; ++i) { a.width[i] /= per; a.stride[i] /= per; a.offset[i] /= per; }
        for (int i = n_in; i <= kMaxConcatInputs; ++i) a.offset[i] = off / per;
        int grid = stream_grid(ctx, rows * (off / per), kThreads);
        concat_rows_kernel<uint4><<<grid, kThreads, 0, st>>>(a, static_cast<uint4*>(y), y_stride / per, rows);
    } else {
        int grid = stream_grid(ctx, rows * off, kThreads);
        if (es == 1) concat_rows_kernel<uint8_t><<<grid, kThreads, 0, st>>>(a, static_cast<uint8_t*>(y), y_stride, rows);
        else if (es == 2) concat_rows_kernel<uint16_t><<<grid, kThreads, 0, st>>>(a, static_cast<uint16_t*>(y), y_stride, rows);
        else concat_rows_kernel<uint32_t><<<grid, kThreads, 0, st>>>(a, static_cast<uint32_t*>(y), y_stride, rows);
    }
    return after_launch("exb_concat_fwd");
}

extern "C" int exb_interp_nearest_fwd(exb_ctx* ctx, const void* x, void* y, int N, int H, int W, int C, int c_stride,
                                      int OH, int OW, int dtype, int channel_last, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && H > 0 && W > 0 && C > 0 && OH > 0 && OW > 0, "exb_interp_nearest_fwd: bad shape");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_interp_nearest_fwd: null buffer");
    // source coordinate = (int)(o * (in / (float)out)), clamped: src/Excalibur/operation_interp.cpp:247-262
    const float hs = H / (float)OH, ws = W / (float)OW;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!channel_last) {
        if (dtype != EXB_F32) return fail(EXB_ERR_UNSUPPORTED, "planar nearest resize is implemented for EXB_F32 only");
        const int64_t planes = (int64_t)N * C;
        EXB_REQUIRE(planes < (1ll << 31), "exb_interp_nearest_fwd: too many planes");
        int grid = stream_grid(ctx, planes * OH * OW, kThreads);
        interp_nearest_nchw_kernel<<<grid, kThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y),
                                                              (int)planes, H, W, OH, OW, hs, ws);
        return after_launch("exb_interp_nearest_fwd");
    }
    const int cs = c_stride ? c_stride : C;
    EXB_REQUIRE(cs >= C, "exb_interp_nearest_fwd: channel stride smaller than channel count");
    const int64_t es = (int64_t)dtype_size(dtype);
    if (es == 0 || dtype == EXB_I32) return fail(EXB_ERR_UNSUPPORTED, "exb_interp_nearest_fwd: dtype %d", dtype);
    if ((cs * es) % 16 == 0 && aligned16(x) && aligned16(y)) {
        const int v = (int)(cs * es / 16);
        int grid = stream_grid(ctx, (int64_t)N * OH * OW * v, kThreads);
        interp_nearest_nhwc_kernel<uint4><<<grid, kThreads, 0, st>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y),
                                                                     N, H, W, v, OH, OW, hs, ws);
    } else {
        int grid = stream_grid(ctx, (int64_t)N * OH * OW * cs, kThreads);
        if (es == 1)
            interp_nearest_nhwc_kernel<uint8_t><<<grid, kThreads, 0, st>>>(static_cast<const uint8_t*>(x),
                                                                           static_cast<uint8_t*>(y), N, H, W, cs, OH, OW, hs, ws);
        else if (es == 2)
            interp_nearest_nhwc_kernel<uint16_t><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(x),
                                                                            static_cast<uint16_t*>(y), N, H, W, cs, OH, OW, hs, ws);
        else
            interp_nearest_nhwc_kernel<uint32_t><<<grid, kThreads, 0, st>>>(static_cast<const uint32_t*>(x),
                                                                            static_cast<uint32_t*>(y), N, H, W, cs, OH, OW, hs, ws);
    }
    return after_launch("exb_interp_nearest_fwd");
}

extern "C" int exb_focus_fwd(exb_ctx* ctx, const void* x, void* y, int N, int C, int H, int W, int in_stride,
                             int out_stride, int dtype, int channel_last, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && C > 0 && H >= 2 && W >= 2, "exb_focus_fwd: bad shape");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_focus_fwd: null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (!channel_last && dtype != EXB_F32) return fail(EXB_ERR_UNSUPPORTED, "planar focus is implemented for EXB_F32 only");
    if (channel_last) {
        if (in_stride == 0) in_stride = C;
        if (out_stride == 0) out_stride = 4 * C;
        EXB_REQUIRE(in_stride >= C && out_stride >= 4 * C, "exb_focus_fwd: channel stride smaller than channel count");
    }
    const int64_t work = (int64_t)N * (H / 2) * (W / 2) * (channel_last ? out_stride : 4 * C);
    const int grid = stream_grid(ctx, work, kThreads);
    switch (dtype) {
    case EXB_F32:
        focus_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), N, C, H, W,
                                                       in_stride, out_stride, channel_last);
        break;
    case EXB_F16:
        focus_kernel<uint16_t><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(y), N, C, H,
                                                          W, in_stride, out_stride, channel_last);
        break;
    case EXB_I8:
        focus_kernel<uint8_t><<<grid, kThreads, 0, st>>>(static_cast<const uint8_t*>(x), static_cast<uint8_t*>(y), N, C, H, W,
                                                         in_stride, out_stride, channel_last);
        break;
    default: return fail(EXB_ERR_UNSUPPORTED, "exb_focus_fwd: dtype %d", dtype);
    }
    return after_launch("exb_focus_fwd");
}

static int channel_affine_impl(exb_ctx* ctx, const void* x, void* y, const float* mul, const float* add, const float* slope,
                               int n_slope, int64_t outer, int C, int c_stride, int64_t inner, int dtype, int channel_last,
                               int act, void* stream, const char* what) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(outer >= 0 && C > 0 && inner > 0, "%s: bad shape", what);
    if (dtype != EXB_F16 && dtype != EXB_F32)
        return fail(EXB_ERR_UNSUPPORTED, "%s supports EXB_F16 and EXB_F32, got dtype %d", what, dtype);
    if (!act_supported(act)) return fail(EXB_ERR_UNSUPPORTED, "activation type %d is not implemented", act);
    const int cs = channel_last ? (c_stride ? c_stride : C) : C;
    EXB_REQUIRE(cs >= C, "%s: channel stride smaller than channel count", what);
    // channel-last: outer = pixels, inner ignored; planar: outer = images, inner = H*W
    const int64_t count = channel_last ? outer * cs : outer * C * inner;
    if (count == 0) return EXB_OK;
    EXB_REQUIRE(x && y && mul && add, "%s: null buffer", what);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == EXB_F16 && channel_last && cs % 8 == 0 && aligned16(x) && aligned16(y)) {
        const int64_t nvec = count / 8;
        channel_affine_nhwc_f16x8_kernel<<<slice_grid(ctx, nvec, cs / 8), kThreads, 0, st>>>(
            static_cast<const uint4*>(x), static_cast<uint4*>(y), mul, add, slope, n_slope, act, nvec, C, cs / 8);
        return after_launch(what);
    }
    int grid = stream_grid(ctx, count, kThreads);
    if (dtype == EXB_F16)
        channel_affine_kernel<__half><<<grid, kThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), mul,
                                                                 add, count, C, cs, inner, channel_last, act, slope, n_slope);
    else
        channel_affine_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), mul,
                                                                add, count, C, cs, inner, channel_last, act, slope, n_slope);
    return after_launch(what);
}

extern "C" int exb_channel_affine_fwd(exb_ctx* ctx, const void* x, void* y, const float* mul, const float* add,
                                      int64_t outer, int C, int c_stride, int64_t inner, int dtype, int channel_last,
                                      int act, void* stream) {
    return channel_affine_impl(ctx, x, y, mul, add, nullptr, 0, outer, C, c_stride, inner, dtype, channel_last, act, stream,
                               "exb_channel_affine_fwd");
}

extern "C" int exb_channel_affine_prelu_fwd(exb_ctx* ctx, const void* x, void* y, const float* mul, const float* add,
                                            const float* slope, int n_slope, int64_t outer, int C, int c_stride,
                                            int64_t inner, int dtype, int channel_last, void* stream) {
    EXB_REQUIRE(slope != nullptr && (n_slope == 1 || n_slope == C), "exb_channel_affine_prelu_fwd: %d slopes for %d channels",
                n_slope, C);
    return channel_affine_impl(ctx, x, y, mul, add, slope, n_slope, outer, C, c_stride, inner, dtype, channel_last,
                               EXB_ACT_NONE, stream, "exb_channel_affine_prelu_fwd");
}

extern "C" int exb_prelu_fwd(exb_ctx* ctx, const void* x, void* y, const float* slope, int n_slope, int64_t outer, int C,
                             int c_stride, int64_t inner, int dtype, int channel_last, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(outer >= 0 && C > 0 && inner > 0, "exb_prelu_fwd: bad shape");
    EXB_REQUIRE(n_slope == 1 || n_slope == C, "exb_prelu_fwd: %d slopes for %d channels", n_slope, C);
    if (dtype != EXB_F16 && dtype != EXB_F32)
        return fail(EXB_ERR_UNSUPPORTED, "exb_prelu_fwd supports EXB_F16 and EXB_F32, got dtype %d", dtype);
    const int cs = channel_last ? (c_stride ? c_stride : C) : C;
    EXB_REQUIRE(cs >= C, "exb_prelu_fwd: channel stride smaller than channel count");
    const int64_t count = channel_last ? outer * cs : outer * C * inner;
    if (count == 0) return EXB_OK;
    EXB_REQUIRE(x && y && slope, "exb_prelu_fwd: null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == EXB_F16 && channel_last && cs % 8 == 0 && aligned16(x) && aligned16(y)) {
        const int64_t nvec = count / 8;
        channel_affine_nhwc_f16x8_kernel<<<slice_grid(ctx, nvec, cs / 8), kThreads, 0, st>>>(
            static_cast<const uint4*>(x), static_cast<uint4*>(y), nullptr, nullptr, slope, n_slope, EXB_ACT_NONE, nvec, C, cs / 8);
        return after_launch("exb_prelu_fwd");
    }
    int grid = stream_grid(ctx, count, kThreads);
    if (dtype == EXB_F16)
        prelu_kernel<__half><<<grid, kThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<__half*>(y), slope, n_slope,
                                                        count, C, cs, inner, channel_last);
    else
        prelu_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(x), static_cast<float*>(y), slope, n_slope,
                                                       count, C, cs, inner, channel_last);
    return after_launch("exb_prelu_fwd");
}

extern "C" int exb_depth_to_space_fwd(exb_ctx* ctx, const void* x, void* y, int N, int H, int W, int rh, int rw, int C,
                                      int x_stride, int y_stride, int dtype, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && H >= 0 && W >= 0 && rh > 0 && rw > 0 && C > 0, "exb_depth_to_space_fwd: bad shape");
    const int64_t es = (int64_t)dtype_size(dtype);
    if (es != 2 && es != 4) return fail(EXB_ERR_UNSUPPORTED, "exb_depth_to_space_fwd: dtype %d", dtype);
    const int xs = x_stride ? x_stride : rh * rw * C, ys = y_stride ? y_stride : C;
    EXB_REQUIRE(xs >= rh * rw * C && ys >= C, "exb_depth_to_space_fwd: stride smaller than channel count");
    const int64_t work = (int64_t)N * H * rh * W * rw * ys;
    if (work == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_depth_to_space_fwd: null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (es == 2 && ys % 8 == 0 && aligned16(y)) {
        const bool whole = C % 8 == 0 && xs % 8 == 0 && aligned16(x);
        const int g8 = stream_grid(ctx, work / 8, kThreads);
        if (whole)
            depth_to_space_f16x8_kernel<false><<<g8, kThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<uint4*>(y), N, H,
                                                                        W, rh, rw, C, xs, ys / 8);
        else
            depth_to_space_f16x8_kernel<true><<<g8, kThreads, 0, st>>>(static_cast<const __half*>(x), static_cast<uint4*>(y), N, H,
                                                                       W, rh, rw, C, xs, ys / 8);
        return after_launch("exb_depth_to_space_fwd");
    }
    int grid = stream_grid(ctx, work, kThreads);
    if (es == 2)
        depth_to_space_kernel<uint16_t><<<grid, kThreads, 0, st>>>(static_cast<const uint16_t*>(x), static_cast<uint16_t*>(y),
                                                                   N, H, W, rh, rw, C, xs, ys);
    else
        depth_to_space_kernel<uint32_t><<<grid, kThreads, 0, st>>>(static_cast<const uint32_t*>(x), static_cast<uint32_t*>(y),
                                                                   N, H, W, rh, rw, C, xs, ys);
    return after_launch("exb_depth_to_space_fwd");
}

extern "C" int exb_transpose_hw_f32(exb_ctx* ctx, const float* x, float* y, int64_t planes, int H, int W, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(planes >= 0 && H >= 0 && W >= 0, "exb_transpose_hw_f32: bad shape");
    if (planes == 0 || H == 0 || W == 0) return EXB_OK;
    EXB_REQUIRE(x && y && x != y, "exb_transpose_hw_f32: null or aliased buffer");
    EXB_REQUIRE((H + 31) / 32 <= 65535, "exb_transpose_hw_f32: height %d too large", H);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    for (int64_t p0 = 0; p0 < planes; p0 += 65535) {
        const int64_t np = planes - p0 < 65535 ? planes - p0 : 65535;
        dim3 grid((W + 31) / 32, (H + 31) / 32, (unsigned)np);
        transpose_planes_f32_kernel<<<grid, 256, 0, st>>>(x + p0 * (int64_t)H * W, y + p0 * (int64_t)H * W, H, W);
    }
    return after_launch("exb_transpose_hw_f32");
}

extern "C" int exb_binaryop_channel_bcast_fwd(exb_ctx* ctx, int op, const void* a, const void* b, int b_first, void* y, int N,
                                              int b_batch, int C, int c_stride, int64_t inner, int dtype, int channel_last,
                                              void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && C > 0 && inner > 0, "exb_binaryop_channel_bcast_fwd: bad shape");
    EXB_REQUIRE(b_batch == N || b_batch == 1, "exb_binaryop_channel_bcast_fwd: %d gate images for a batch of %d", b_batch, N);
    if (op < 0 || op > 3) return fail(EXB_ERR_UNSUPPORTED, "binary op type %d", op);
    if (dtype != EXB_F16 && dtype != EXB_F32)
        return fail(EXB_ERR_UNSUPPORTED, "exb_binaryop_channel_bcast_fwd supports EXB_F16 and EXB_F32, got dtype %d", dtype);
    const int cs = channel_last ? (c_stride ? c_stride : C) : C;
    EXB_REQUIRE(cs >= C, "exb_binaryop_channel_bcast_fwd: channel stride smaller than channel count");
    const int64_t count = (int64_t)N * inner * cs;
    if (count == 0) return EXB_OK;
    EXB_REQUIRE(a && b && y, "exb_binaryop_channel_bcast_fwd: null buffer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == EXB_F16 && channel_last && cs % 8 == 0 && aligned16(a) && aligned16(b) && aligned16(y)) {
        const int64_t nvec = count / 8;
        binary_bcast_nhwc_f16x8_kernel<<<stream_grid(ctx, nvec, kThreads), kThreads, 0, st>>>(
            static_cast<const uint4*>(a), static_cast<const uint4*>(b), static_cast<uint4*>(y), nvec, C, cs / 8, inner * (cs / 8), op,
            b_batch, b_first);
        return after_launch("exb_binaryop_channel_bcast_fwd");
    }
    const int grid = stream_grid(ctx, count, kThreads);
    if (dtype == EXB_F16)
        binary_bcast_kernel<__half><<<grid, kThreads, 0, st>>>(static_cast<const __half*>(a), static_cast<const __half*>(b),
                                                               static_cast<__half*>(y), count, C, cs, inner, channel_last, op, b_batch,
                                                               b_first);
    else
        binary_bcast_kernel<float><<<grid, kThreads, 0, st>>>(static_cast<const float*>(a), static_cast<const float*>(b),
                                                              static_cast<float*>(y), count, C, cs, inner, channel_last, op, b_batch,
                                                              b_first);
    return after_launch("exb_binaryop_channel_bcast_fwd");
}

extern "C" int exb_softmax_channels_f32(exb_ctx* ctx, const float* x, float* y, int N, int C, int64_t inner,
                                        int64_t x_image_stride, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && C > 0 && inner > 0, "exb_softmax_channels_f32: bad shape");
    if (x_image_stride == 0) x_image_stride = (int64_t)C * inner;
    EXB_REQUIRE(x_image_stride >= (int64_t)C * inner, "exb_softmax_channels_f32: image stride smaller than an image");
    if (N == 0) return EXB_OK;
    EXB_REQUIRE(x && y && x != y, "exb_softmax_channels_f32: null or aliased buffer");
    softmax_channels_kernel<<<stream_grid(ctx, (int64_t)N * inner, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        x, y, N, C, inner, x_image_stride);
    return after_launch("exb_softmax_channels_f32");
}

extern "C" int exb_nhwc_f16_split_heads_f32(exb_ctx* ctx, const void* x, float* y, int N, int P, int c_stride, int A, int K,
                                            void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && P > 0 && A > 0 && K > 0 && c_stride >= A * K, "exb_nhwc_f16_split_heads_f32: bad shape");
    const int64_t total = (int64_t)N * A * P * K;
    if (total == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_nhwc_f16_split_heads_f32: null buffer");
    EXB_REQUIRE(A * K <= 65536, "exb_nhwc_f16_split_heads_f32: %d channels", A * K);
    const int64_t rows = (int64_t)N * P;
    split_heads_kernel<<<stream_grid(ctx, rows * 32, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), y, rows, P, c_stride, A, K);
    return after_launch("exb_nhwc_f16_split_heads_f32");
}

extern "C" int exb_depth_to_space_nchw_f32(exb_ctx* ctx, const void* x, float* y, int N, int H, int W, int rh, int rw, int C,
                                           int x_stride, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "null context");
    EXB_REQUIRE(N >= 0 && H >= 0 && W >= 0 && rh > 0 && rw > 0 && C > 0, "exb_depth_to_space_nchw_f32: bad shape");
    const int xs = x_stride ? x_stride : rh * rw * C;
    EXB_REQUIRE(xs >= rh * rw * C, "exb_depth_to_space_nchw_f32: stride smaller than channel count");
    const int64_t work = (int64_t)N * C * H * rh * W * rw;
    if (work == 0) return EXB_OK;
    EXB_REQUIRE(x && y, "exb_depth_to_space_nchw_f32: null buffer");
    depth_to_space_nchw_f32_kernel<<<stream_grid(ctx, work, kThreads), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __half*>(x), y, N, H, W, rh, rw, C, xs);
    return after_launch("exb_depth_to_space_nchw_f32");
}
