/*
 * TEST INFRASTRUCTURE - NOT PRODUCT CODE.  See exb_oracle.h for what this file is, which
 * reference lines each function follows, and how it is pinned against the reference.
 * Scalar loops only: it is meant to be obviously right, not fast.
 */
#include "exb_oracle.h"

#include <float.h>
#include <math.h>
#include <stdlib.h>
#include <string.h>

int exbo_conv_out_dim(int in, int pad_a, int pad_b, int k, int stride) {
    return (in + pad_a + pad_b - k) / stride + 1;
}

int exbo_pool_out_dim(int in, int pad_a, int pad_b, int k, int stride, int pad_mode) {
    float q = (float)(in + pad_a + pad_b - k) / (float)stride;
    return (int)(pad_mode == 0 ? ceilf(q) : floorf(q)) + 1;
}

void exbo_activation_f32(float* y, int64_t n, int act) {
    int64_t i;
    switch (act) {
    case EXBO_ACT_NONE:
        return;
    case EXBO_ACT_RELU:
        for (i = 0; i < n; ++i) y[i] = y[i] >= 0.0f ? y[i] : 0.0f;
        return;
    case EXBO_ACT_RELU6_QUIRK:
        for (i = 0; i < n; ++i) y[i] = (y[i] >= 0.0f && y[i] <= 6.0f) ? y[i] : 0.0f;
        return;
    case EXBO_ACT_SIGMOID:
        for (i = 0; i < n; ++i) y[i] = (float)(1. / (1. + exp(-(double)y[i])));
        return;
    case EXBO_ACT_MISH:
        for (i = 0; i < n; ++i) y[i] = (float)((double)y[i] * tanh(log(1 + exp((double)y[i]))));
        return;
    case EXBO_ACT_RELU6:
        for (i = 0; i < n; ++i) y[i] = y[i] < 0.0f ? 0.0f : (y[i] > 6.0f ? 6.0f : y[i]);
        return;
    case EXBO_ACT_SILU:
        for (i = 0; i < n; ++i) y[i] = (float)((double)y[i] / (1. + exp(-(double)y[i])));
        return;
    default:
        abort();
    }
}

void exbo_conv2d_f32(const float* x, const float* w, const float* bias, float* y,
                     int N, int C, int H, int W, int Cout, int kh, int kw,
                     int sh, int sw, int pt, int pb, int pl, int pr, int group, int act) {
    const int OH = exbo_conv_out_dim(H, pt, pb, kh, sh);
    const int OW = exbo_conv_out_dim(W, pl, pr, kw, sw);
    const int cpg = C / group, opg = Cout / group;
    for (int n = 0; n < N; ++n)
        for (int o = 0; o < Cout; ++o) {
            const int g = o / opg;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    double acc = 0.0;
                    for (int ci = 0; ci < cpg; ++ci) {
                        const int c = g * cpg + ci;
                        for (int r = 0; r < kh; ++r) {
                            const int ih = oh * sh - pt + r;
                            if (ih < 0 || ih >= H) continue;
                            for (int s = 0; s < kw; ++s) {
                                const int iw = ow * sw - pl + s;
                                if (iw < 0 || iw >= W) continue;
                                acc += (double)x[(((int64_t)n * C + c) * H + ih) * W + iw] *
                                       (double)w[(((int64_t)o * cpg + ci) * kh + r) * kw + s];
                            }
                        }
                    }
                    if (bias) acc += (double)bias[o];
                    y[(((int64_t)n * Cout + o) * OH + oh) * OW + ow] = (float)acc;
                }
        }
    exbo_activation_f32(y, (int64_t)N * Cout * OH * OW, act);
}

int8_t exbo_float32_to_int8(float v) {
    float t = v >= 0.f ? v + 0.5f : v - 0.5f;
    if (t > 127) return 127;
    if (t < -128) return -128;
    return (int8_t)t; /* truncation toward zero */
}

void exbo_quantize_f32_i8(const float* x, int8_t* q, int N, int C, int HW,
                          const float* scales, int n_scales) {
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const float s = n_scales == 1 ? scales[0] : scales[c];
            const int64_t base = ((int64_t)n * C + c) * HW;
            for (int i = 0; i < HW; ++i) q[base + i] = exbo_float32_to_int8(x[base + i] * s);
        }
}

void exbo_requantize_rne_f32_i8(const float* v, int8_t* q, int64_t n, float scale) {
    for (int64_t i = 0; i < n; ++i) {
        float t = rintf(v[i] * scale); /* default rounding mode: half to even */
        if (t > 127.f) t = 127.f;
        if (t < -128.f) t = -128.f;
        q[i] = (int8_t)t;
    }
}

void exbo_conv2d_i8_acc(const int8_t* xq, const int8_t* wq, int32_t* acc,
                        int N, int C, int H, int W, int Cout, int kh, int kw,
                        int sh, int sw, int pt, int pb, int pl, int pr, int group) {
    const int OH = exbo_conv_out_dim(H, pt, pb, kh, sh);
    const int OW = exbo_conv_out_dim(W, pl, pr, kw, sw);
    const int cpg = C / group, opg = Cout / group;
    for (int n = 0; n < N; ++n)
        for (int o = 0; o < Cout; ++o) {
            const int g = o / opg;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    int32_t a = 0;
                    for (int ci = 0; ci < cpg; ++ci) {
                        const int c = g * cpg + ci;
                        for (int r = 0; r < kh; ++r) {
                            const int ih = oh * sh - pt + r;
                            if (ih < 0 || ih >= H) continue;
                            for (int s = 0; s < kw; ++s) {
                                const int iw = ow * sw - pl + s;
                                if (iw < 0 || iw >= W) continue;
                                a += (int32_t)xq[(((int64_t)n * C + c) * H + ih) * W + iw] *
                                     (int32_t)wq[(((int64_t)o * cpg + ci) * kh + r) * kw + s];
                            }
                        }
                    }
                    acc[(((int64_t)n * Cout + o) * OH + oh) * OW + ow] = a;
                }
        }
}

void exbo_dequant_scales(const float* ws, int n_ws, const float* fs, int n_fs,
                         float* out, int Cout) {
    for (int q = 0; q < Cout; ++q) {
        const float f = n_fs == 1 ? fs[0] : fs[q];
        const float wsc = n_ws == 1 ? ws[0] : ws[q];
        out[q] = (fabsf(wsc) <= 1e-6) ? 0.f : (1.0f / (wsc * f));
    }
}

void exbo_dequantize_i32_f32(const int32_t* acc, const float* scale, const float* bias,
                             float* y, int N, int C, int HW) {
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const int64_t base = ((int64_t)n * C + c) * HW;
            const float b = bias ? bias[c] : 0.0f;
            for (int i = 0; i < HW; ++i)
                y[base + i] = bias ? fmaf((float)acc[base + i], scale[c], b)
                                   : (float)acc[base + i] * scale[c];
        }
}

void exbo_conv2d_i8(const float* x, const int8_t* wq, const float* bias,
                    const float* ws, int n_ws, const float* fs, int n_fs, float* y,
                    int N, int C, int H, int W, int Cout, int kh, int kw,
                    int sh, int sw, int pt, int pb, int pl, int pr, int group, int act) {
    const int OH = exbo_conv_out_dim(H, pt, pb, kh, sh);
    const int OW = exbo_conv_out_dim(W, pl, pr, kw, sw);
    int8_t* xq = (int8_t*)malloc((size_t)N * C * H * W);
    int32_t* acc = (int32_t*)malloc(sizeof(int32_t) * (size_t)N * Cout * OH * OW);
    float* sc = (float*)malloc(sizeof(float) * (size_t)Cout);
    exbo_quantize_f32_i8(x, xq, N, C, H * W, fs, n_fs);
    exbo_conv2d_i8_acc(xq, wq, acc, N, C, H, W, Cout, kh, kw, sh, sw, pt, pb, pl, pr, group);
    exbo_dequant_scales(ws, n_ws, fs, n_fs, sc, Cout);
    exbo_dequantize_i32_f32(acc, sc, bias, y, N, Cout, OH * OW);
    exbo_activation_f32(y, (int64_t)N * Cout * OH * OW, act);
    free(xq);
    free(acc);
    free(sc);
}

void exbo_dwconv2d_f32(const float* x, const float* w, const float* bias, float* y,
                       int N, int C, int H, int W, int kh, int kw,
                       int sh, int sw, int pt, int pb, int pl, int pr, int act) {
    const int OH = exbo_conv_out_dim(H, pt, pb, kh, sh);
    const int OW = exbo_conv_out_dim(W, pl, pr, kw, sw);
    for (int n = 0; n < N; ++n)
        for (int c = 0; c < C; ++c) {
            const float* xp = x + ((int64_t)n * C + c) * H * W;
            const float* wp = w + (int64_t)c * kh * kw;
            float* yp = y + ((int64_t)n * C + c) * OH * OW;
            for (int oh = 0; oh < OH; ++oh)
                for (int ow = 0; ow < OW; ++ow) {
                    double acc = 0.0;
                    for (int r = 0; r < kh; ++r) {
                        const int ih = oh * sh - pt + r;
                        if (ih < 0 || ih >= H) continue;
                        for (int s = 0; s < kw; ++s) {
                            const int iw = ow * sw - pl + s;
                            if (iw < 0 || iw >= W) continue;
                            acc += (double)xp[ih * W + iw] * (double)wp[r * kw + s];
                        }
                    }
                    if (bias) acc += (double)bias[c];
                    yp[oh * OW + ow] = (float)acc;
                }
        }
    exbo_activation_f32(y, (int64_t)N * C * OH * OW, act);
}

void exbo_pool2d_f32(const float* x, float* y, int N, int C, int H, int W,
                     int type, int kh, int kw, int sh, int sw,
                     int pt, int pb, int pl, int pr, int global, int pad_mode,
                     int count_include_pad) {
    if (global) {
        kh = H; kw = W; pt = pb = pl = pr = 0; sh = sw = 1;
    }
    const int PH = exbo_pool_out_dim(H, pt, pb, kh, sh, pad_mode);
    const int PW = exbo_pool_out_dim(W, pl, pr, kw, sw, pad_mode);
    for (int64_t nc = 0; nc < (int64_t)N * C; ++nc) {
        const float* xp = x + nc * H * W;
        float* yp = y + nc * PH * PW;
        for (int ph = 0; ph < PH; ++ph)
            for (int pw = 0; pw < PW; ++pw) {
                int hs = ph * sh - pt, ws = pw * sw - pl;
                if (type == 0) {
                    int he = hs + kh < H ? hs + kh : H;
                    int we = ws + kw < W ? ws + kw : W;
                    if (hs < 0) hs = 0;
                    if (ws < 0) ws = 0;
                    float m = -FLT_MAX;
                    for (int h = hs; h < he; ++h)
                        for (int w2 = ws; w2 < we; ++w2)
                            if (xp[h * W + w2] > m) m = xp[h * W + w2];
                    yp[ph * PW + pw] = m;
                } else {
                    int he = hs + kh < H + pb ? hs + kh : H + pb;
                    int we = ws + kw < W + pr ? ws + kw : W + pr;
                    int pool_size = (he - hs) * (we - ws);
                    if (hs < 0) hs = 0;
                    if (ws < 0) ws = 0;
                    if (he > H) he = H;
                    if (we > W) we = W;
                    float s = 0.0f; /* fp32 running sum in window order, like the reference */
                    int area = 0;
                    for (int h = hs; h < he; ++h)
                        for (int w2 = ws; w2 < we; ++w2) {
                            s += xp[h * W + w2];
                            ++area;
                        }
                    if (count_include_pad == 0) pool_size = area;
                    yp[ph * PW + pw] = s / (float)pool_size;
                }
            }
    }
}

void exbo_eltwise_f32(const float* const* xs, int n_in, const float* coeffs, int type,
                      float* y, int64_t count) {
    for (int64_t i = 0; i < count; ++i) {
        float v;
        if (type == 1) {
            v = 0.0f;
            for (int k = 0; k < n_in; ++k) v = (coeffs ? coeffs[k] : 1.0f) * xs[k][i] + v;
        } else if (type == 2) {
            v = xs[0][i] > xs[1][i] ? xs[0][i] : xs[1][i];
            for (int k = 2; k < n_in; ++k) v = v > xs[k][i] ? v : xs[k][i];
        } else {
            v = xs[0][i] * xs[1][i];
            for (int k = 2; k < n_in; ++k) v = v * xs[k][i];
        }
        y[i] = v;
    }
}

void exbo_binaryop_f32(const float* a, const float* b, float* y, int64_t count, int op) {
    for (int64_t i = 0; i < count; ++i) {
        switch (op) {
        case 0: y[i] = a[i] + b[i]; break;
        case 1: y[i] = a[i] - b[i]; break;
        case 2: y[i] = a[i] * b[i]; break;
        case 3: y[i] = a[i] / b[i]; break;
        default: abort();
        }
    }
}

void exbo_relu_f32(const float* x, float* y, int64_t count) {
    for (int64_t i = 0; i < count; ++i) y[i] = x[i] >= 0.0f ? x[i] : 0.0f;
}
