/*
 * TEST INFRASTRUCTURE - NOT PRODUCT CODE.
 *
 * Plain-C restatement of the arithmetic of the reference CNN forward path (convolution,
 * depthwise convolution, pooling, eltwise / binary op, ReLU, int8 quantise / dequantise).
 * It exists only to check the CUDA kernels: tests, the smoke check and the CPU-baseline
 * leg of the benchmark may call it; no product code path does.
 *
 * Parity pin: the reference ships no tests and no golden vectors, so this restatement is
 * pinned against outputs of the reference library itself (oracle/_ref, built from the
 * reference sources by oracle/Makefile) through tests/golden/*.npz and, where the reference
 * tree is available, live in tests/test_oracle_vs_reference.py.
 *
 * All tensors are dense NCHW unless a function says otherwise, like the reference's
 * memory::tensor default (reference include/Primitives/tensor.hpp:15-173).
 */
#ifndef EXB_ORACLE_H_
#define EXB_ORACLE_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Activation codes: 0..5 are the reference's conv key 9 (operation_general_conv.cpp:127-272);
 * 100+ are activations our fused epilogues add. */
enum {
    EXBO_ACT_NONE = 0,
    EXBO_ACT_RELU = 1,
    EXBO_ACT_RELU6_QUIRK = 3,   /* reference "ReLU6": x>6 -> 0 (operation_general_conv.cpp:206-237) */
    EXBO_ACT_SIGMOID = 4,
    EXBO_ACT_MISH = 5,
    EXBO_ACT_RELU6 = 103,       /* true clip to [0,6] (operation_clip.cpp:33-57 with 0=0 1=6) */
    EXBO_ACT_SILU = 104         /* x*sigmoid(x) (Sigmoid + BinaryOp mul in reference graphs) */
};

/* (in + pad_a + pad_b - k) / stride + 1, integer division
 * (operation_convolution.cpp:270-273). */
int exbo_conv_out_dim(int in, int pad_a, int pad_b, int k, int stride);

/* Pooling output size, pad_mode 0 = ceil, 1 = floor (operation_pooling.cpp:101-120). */
int exbo_pool_out_dim(int in, int pad_a, int pad_b, int k, int stride, int pad_mode);

void exbo_activation_f32(float* y, int64_t n, int act);

/* Dense / grouped convolution, fp32, zero padding, dilation 1, double accumulation,
 * bias (may be NULL) then activation.  Semantics of operation_convolution::forward_cpu_f32
 * (operation_convolution.cpp:251-329); w is OIHW [Cout][Cin/group][kh][kw]. */
void exbo_conv2d_f32(const float* x, const float* w, const float* bias, float* y,
                     int N, int C, int H, int W, int Cout, int kh, int kw,
                     int sh, int sw, int pt, int pb, int pl, int pr, int group, int act);

/* float32_to_int8: round half away from zero, saturate to [-128,127]
 * (src/Primitives/simd_types.cpp:140-152). */
int8_t exbo_float32_to_int8(float v);

/* q = float32_to_int8(x * scale); n_scales == 1 -> per tensor, == C -> per input channel
 * (operation_general_conv.cpp:584-720). */
void exbo_quantize_f32_i8(const float* x, int8_t* q, int N, int C, int HW,
                          const float* scales, int n_scales);

/* Our producer-side requantisation: q = sat8(rintf(v * scale)), round half to even. */
void exbo_requantize_rne_f32_i8(const float* v, int8_t* q, int64_t n, float scale);

/* Exact int32 accumulators of an int8 convolution (what both reference int8 paths produce:
 * operation_convolution.cpp:1783-2161 and :2269-2978). */
void exbo_conv2d_i8_acc(const int8_t* xq, const int8_t* wq, int32_t* acc,
                        int N, int C, int H, int W, int Cout, int kh, int kw,
                        int sh, int sw, int pt, int pb, int pl, int pr, int group);

/* scale[c] = |ws| <= 1e-6 ? 0 : 1.0f / (ws * fs)  (operation_convolution.cpp:397-404). */
void exbo_dequant_scales(const float* ws, int n_ws, const float* fs, int n_fs,
                         float* out, int Cout);

/* y = fma(float(acc), scale[c], bias[c])  (operation_general_conv.cpp:724-941; the x86 build
 * contracts the multiply-add, and the im2col path uses _mm256_fmadd_ps). bias may be NULL. */
void exbo_dequantize_i32_f32(const int32_t* acc, const float* scale, const float* bias,
                             float* y, int N, int C, int HW);

/* The whole of operation_convolution::forward_cpu_i8 (operation_convolution.cpp:332-409):
 * quantise fp32 input with fs, int8 conv, dequantise with 1/(ws*fs), bias, activation. */
void exbo_conv2d_i8(const float* x, const int8_t* wq, const float* bias,
                    const float* ws, int n_ws, const float* fs, int n_fs, float* y,
                    int N, int C, int H, int W, int Cout, int kh, int kw,
                    int sh, int sw, int pt, int pb, int pl, int pr, int group, int act);

/* Depthwise k x k convolution (group == C == Cout), direct form
 * (cuda/operation_convolutiondepthwise.cu:21-52; CPU operation_convolutiondepthwise.cpp:18-181). */
void exbo_dwconv2d_f32(const float* x, const float* w, const float* bias, float* y,
                       int N, int C, int H, int W, int kh, int kw,
                       int sh, int sw, int pt, int pb, int pl, int pr, int act);

/* Max (type 0) / average (type 1) pooling (operation_pooling.cpp:80-309).  Max ignores the
 * padding; average divides by the window clipped to H+pad_bottom / W+pad_right, or by the
 * number of valid taps when count_include_pad == 0.  global != 0 pools the whole map. */
void exbo_pool2d_f32(const float* x, float* y, int N, int C, int H, int W,
                     int type, int kh, int kw, int sh, int sw,
                     int pt, int pb, int pl, int pr, int global, int pad_mode,
                     int count_include_pad);

/* N-ary eltwise (operation_eltwise.cpp:42-94): type 0 PROD, 1 SUM (with coeffs), 2 MAX. */
void exbo_eltwise_f32(const float* const* xs, int n_in, const float* coeffs, int type,
                      float* y, int64_t count);

/* Equal-shape binary op (operation_binaryop.cpp:74-84): 0 add, 1 sub, 2 mul, 3 div. */
void exbo_binaryop_f32(const float* a, const float* b, float* y, int64_t count, int op);

/* max(x, 0) (operation_relu.cpp:31-81). */
void exbo_relu_f32(const float* x, float* y, int64_t count);

#ifdef __cplusplus
}
#endif
#endif /* EXB_ORACLE_H_ */
