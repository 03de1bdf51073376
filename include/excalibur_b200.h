/*
 * excalibur_b200 - C ABI of the B200 (sm_100a) CNN forward hot path.
 *
 * One shared library (libexcalibur_b200.so), extern "C", plain pointers and sizes only.
 * Every entry point returns an int status (0 = ok, negative = error, see exb_status); none
 * aborts the process.  Device buffers are owned by the caller, activations are dense NHWC
 * (channels innermost) in fp16 or int8, `stream` is a cudaStream_t passed as void* (NULL =
 * the legacy default stream, which is what the reference uses everywhere).
 *
 * Each function names the reference interface it stands in for (paths are relative to the
 * reference project's root).  The C++ classes in excalibur_b200/csrc/host/ mirror
 * glasssix::excalibur::operation<Dtype> on top of this ABI.
 */
#ifndef EXCALIBUR_B200_H_
#define EXCALIBUR_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define EXB_API __attribute__((visibility("default")))
#else
#define EXB_API
#endif

typedef enum exb_status {
    EXB_OK = 0,
    EXB_ERR_BAD_ARG = -1,      /* null pointer, non-positive size, misaligned buffer ... */
    EXB_ERR_UNSUPPORTED = -2,  /* valid request this build has no kernel for */
    EXB_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed */
    EXB_ERR_TIMEOUT = -4,      /* a bounded device-side wait ran out (kernel error word set) */
    EXB_ERR_NOMEM = -5
} exb_status;

typedef enum exb_dtype {
    EXB_F16 = 0,  /* IEEE half, the reference's `unsigned short` tensors */
    EXB_I8 = 1,   /* signed char */
    EXB_F32 = 2,
    EXB_I32 = 3   /* raw int32 accumulators (parity / debugging output of the int8 conv) */
} exb_dtype;

/* 0..5: conv key 9 of the reference (src/Excalibur/operation_general_conv.cpp:127-272);
 * 103/104 are activations the reference expresses as separate ops (Clip 0..6; Sigmoid+Mul). */
typedef enum exb_act {
    EXB_ACT_NONE = 0,
    EXB_ACT_RELU = 1,
    EXB_ACT_RELU6_QUIRK = 3, /* reference behaviour: x > 6 -> 0 */
    EXB_ACT_SIGMOID = 4,
    EXB_ACT_MISH = 5,        /* x * tanh(ln(1 + e^x)) (operation_general_conv.cpp:255-266) */
    EXB_ACT_RELU6 = 103,
    EXB_ACT_SILU = 104,
    EXB_ACT_HARDSWISH = 105,  /* x * clamp(x/6 + 0.5, 0, 1): HardSwish with alpha = 1/6, beta = 0.5 */
    EXB_ACT_PRELU = 106       /* x >= 0 ? x : slope[c] * x (PReLU, LeakyRelu): convolutions only, slopes attached to
                                 the packed weights with exb_conv_weights_set_slopes / exb_dw_weights_set_slopes */
} exb_act;

typedef struct exb_ctx exb_ctx;                   /* per-device context */
typedef struct exb_conv_weights exb_conv_weights; /* packed, device-resident conv weights */
typedef struct exb_dw_weights exb_dw_weights;     /* packed depthwise weights */

/* ---------------------------------------------------------------------------------------
 * Context.  Stands in for the per-pipeline device selection + cublasCreate of the reference
 * (src/Excalibur/pipeline.cpp:37-48); binds AFTER selecting the device.
 * ------------------------------------------------------------------------------------- */
EXB_API int exb_ctx_create(int device, exb_ctx** out);
EXB_API int exb_ctx_destroy(exb_ctx* ctx);
/* Message of the last failing call on this thread (never NULL). */
EXB_API const char* exb_last_error_string(void);
/* Library version string, e.g. "0.1.0". (pipeline<Dtype>::version, include/Excalibur/pipeline.hpp:41) */
EXB_API const char* exb_version(void);
/* Number of SMs of the context's device (grid sizing of persistent kernels). */
EXB_API int exb_ctx_sm_count(const exb_ctx* ctx, int* out);
/* Wait for `stream` and report what the kernels launched on it left behind: EXB_OK,
 * EXB_ERR_CUDA (sticky CUDA error) or EXB_ERR_TIMEOUT when a kernel's bounded device-side wait
 * ran out (the error word is cleared by this call).  The reference has no counterpart: its
 * kernels run on the legacy stream and errors surface as CHECK failures that terminate the
 * process (include/Primitives/logger.hpp:101-118). */
EXB_API int exb_ctx_sync_check(exb_ctx* ctx, void* stream);
/* Failure-path self-test without a fault: launches a one-warp kernel whose bounded mbarrier wait
 * (the same wait the convolution kernel uses, at most max_polls <= 4096 tries of about a microsecond)
 * can never be satisfied.  The kernel gives up, records role code 9 and returns; the following
 * exb_ctx_sync_check reports EXB_ERR_TIMEOUT and the context stays usable.  No reference counterpart. */
EXB_API int exb_selftest_bounded_wait(exb_ctx* ctx, int max_polls, void* stream);
/* Best-case tensor-core rate of this GPU (the denominator of the convolution kernel's tensor roofline):
 * sm_count * ctas_per_sm CTAs each issue iters * kblk * 4 tcgen05.mma instructions (M = 128, N = n, K = 32
 * bytes; EXB_I8: s8 x s8 -> s32, EXB_F16: fp16 x fp16 -> fp32) on seeded operands that stay in shared
 * memory - no TMA, no epilogue, no global traffic.  *ops_per_launch receives 2 * MACs of the launch;
 * d_cycles (device pointer or NULL) receives CTA 0's SM cycles.  Time the launch with events on `stream`.
 * n: multiple of 16 up to 256; ctas_per_sm 1 or 2; kblk 1..8 K blocks of 128 bytes per operand row.
 * No reference counterpart (the reference quotes no tensor rate). */
EXB_API int exb_tensor_peak_probe(exb_ctx* ctx, int dtype, int n, int ctas_per_sm, int kblk, int iters,
                                  double* ops_per_launch, unsigned long long* d_cycles, void* stream);
/* The same probe with the A operand laid out as the convolution kernel's variants lay it out: K blocks of kb_bytes
 * (32 / 64 / 128, swizzle of the same width), m = 64 or 128 accumulator rows (64: what a GEMM with the output
 * channels of a narrow layer on M would issue), a_sbo bytes between consecutive 8-row groups (8 * kb_bytes = dense
 * rows; more = rows of a box wider than the tile) and a descriptor that starts a_shift bytes into its region (a
 * shifted window of a wider box).  Shows what an operand layout costs the tensor pipe before a kernel is built
 * around it.  No reference counterpart. */
EXB_API int exb_tensor_peak_probe_layout(exb_ctx* ctx, int dtype, int m, int n, int ctas_per_sm, int kblk, int iters,
                                         int kb_bytes, int a_sbo, int a_shift, double* ops_per_launch,
                                         unsigned long long* d_cycles, void* stream);

/* ---------------------------------------------------------------------------------------
 * Layout / precision converts at the API edge.  The reference keeps NCHW fp32 tensors
 * between ops (include/Primitives/tensor.hpp:15-173) and converts NHWC->NCHW on the CPU
 * (src/Primitives/tensor.cpp:334-377); these kernels move between that edge format and the
 * NHWC fp16 / int8 layout the kernels use.  c_stride >= C is the physical channel count of
 * the NHWC buffer (padding channels are written as zero / ignored on read).
 * For EXB_I8, q = sat8(round(x * scale)) with rounding 0 = half away from zero (reference
 * float32_to_int8, src/Primitives/simd_types.cpp:140-152) or 1 = half to even.
 * ------------------------------------------------------------------------------------- */
EXB_API int exb_nchw_f32_to_nhwc(exb_ctx* ctx, const float* x_nchw, void* y_nhwc, int dtype,
                                 int N, int C, int H, int W, int c_stride, float scale,
                                 int rounding, void* stream);
/* Same conversion into rows that are physically zero-padded along W: y is
 * [N][H][w_pitch][c_stride], pixel 0 of each row at index w_pad; padding pixels and channels are
 * written as zero.  For images with up to 8 channels (the network input). */
EXB_API int exb_nchw_f32_to_nhwc_padded(exb_ctx* ctx, const float* x_nchw, void* y_nhwc, int dtype,
                                        int N, int C, int H, int W, int c_stride, int w_pad,
                                        int w_pitch, float scale, int rounding, void* stream);
/* The two conversions above with the input normalisation of operation_input fused in
 * (src/Excalibur/operation_input.cpp:92-96): y = convert(x * mul[c] + add[c]), device arrays of C entries, the
 * same fma as exb_channel_affine_fwd followed by the same conversion, so the results equal the two-pass form.
 * exb_image_f32_to_nhwc_norm: images of up to 4 channels into a dense channel-last tensor (EXB_F16 with
 * c_stride 8 or 16, EXB_I8 with c_stride 16 or 32; mul == add == NULL skips the normalisation).
 * exb_nchw_f32_to_nhwc4_padded_norm: the padded-row fp16 NHWC4 form (C <= 3; W, w_pad, w_pitch multiples of 4). */
EXB_API int exb_image_f32_to_nhwc_norm(exb_ctx* ctx, const float* x_nchw, void* y_nhwc, int dtype, int N, int C,
                                       int H, int W, int c_stride, const float* mul, const float* add,
                                       float scale, int rounding, void* stream);
EXB_API int exb_nchw_f32_to_nhwc4_padded_norm(exb_ctx* ctx, const float* x_nchw, void* y_nhwc, int N, int C, int H,
                                              int W, int w_pad, int w_pitch, const float* mul, const float* add,
                                              void* stream);
/* The same for an image that is already fp16 NCHW (converted on the host so that half the bytes cross
 * PCIe; same round-to-nearest-even as the fp32 entry, so the results are identical): c_stride 4, fp16
 * output, C <= 3, W / w_pad / w_pitch multiples of 4. */
EXB_API int exb_nchw_f16_to_nhwc4_padded(exb_ctx* ctx, const void* x_nchw_f16, void* y_nhwc, int N, int C, int H,
                                         int W, int w_pad, int w_pitch, void* stream);
EXB_API int exb_nhwc_to_nchw_f32(exb_ctx* ctx, const void* x_nhwc, int dtype, float* y_nchw,
                                 int N, int C, int H, int W, int c_stride, float scale,
                                 void* stream);

/* ---------------------------------------------------------------------------------------
 * Dense convolution forward.  Stands in for operation_convolution::forward_{cpu,gpu}_{f32,
 * f16,i8} (src/Excalibur/operation_convolution.cpp:251-409, src/Excalibur/cuda/
 * operation_convolution.cu:118-262,338-394,484-549): implicit GEMM on the tensor cores, with
 * what the reference runs as separate passes fused into the epilogue:
 *   v  = acc * scale[c] + bias[c]      (int8: scale[c] = 1/(wscale[c]*act_scale), exactly the
 *                                       reference's dequantize scale; fp16: scale = 1)
 *   v += residual                      (the Eltwise/BinaryOp add that follows in ResNet graphs)
 *   v  = act(v)                        (conv key 9, or the ReLU op that follows)
 *   y  = convert(v)                    (fp16 / fp32, or int8 q = sat8(rne(v*out_scale)), i.e.
 *                                       the NEXT int8 conv's input quantisation)
 *   y2 = optional second copy in another dtype (e.g. fp16 skip + int8 for the next conv)
 * ------------------------------------------------------------------------------------- */
typedef struct exb_conv_desc {
    int32_t N, H, W;        /* input batch / height / width */
    int32_t Cin, Cout;      /* logical channels */
    int32_t cin_stride;     /* physical channels of x (NHWC), 0 => Cin; >= Cin */
    int32_t cout_stride;    /* physical channels of y / y2 / residual, 0 => Cout */
    int32_t kh, kw;
    int32_t stride_h, stride_w;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t dilation;       /* only 1 is supported (the reference's forward ignores it too) */
    int32_t group;          /* 1 for the tensor-core path; other values use the direct kernel */
    int32_t in_dtype;       /* EXB_F16 or EXB_I8 */
    int32_t out_dtype;      /* EXB_F16, EXB_I8, EXB_F32 or (int8 input only) EXB_I32 */
    int32_t out2_dtype;     /* -1 = no second output, else EXB_F16 or EXB_I8 */
    int32_t res_dtype;      /* -1 = no residual, else EXB_F16 */
    int32_t act;            /* exb_act */
    float out_scale;        /* multiplier used when out_dtype == EXB_I8 */
    float out2_scale;       /* multiplier used when out2_dtype == EXB_I8 */
    int32_t impl;           /* 0 = auto (tensor cores when eligible), 1 = force direct kernel */
    /* Optional physically padded input rows: x is [N][H][x_w_pitch][cin_stride] and pixel 0 of a
     * row sits x_w_pad pixels in; the padding pixels hold zeros (exb_nchw_f32_to_nhwc_padded
     * writes this layout).  0 / 0 = dense rows.  With few input channels (a stem conv) this lets
     * the tensor-core kernel take kw taps x cin channels as ONE contiguous K row per output pixel. */
    int32_t x_w_pitch;
    int32_t x_w_pad;
    /* 1: a 3x3 stride-2 pad-1 max pooling (floor output size, padding ignored: the reference's
     * Pooling with keys 0=0 1=3 2=2 3=1) is applied to the activated convolution output inside the
     * convolution's epilogue; y / y2 then hold the POOLED map [N][PH][PW][cout_stride] and the
     * convolution output itself is never written.  Only for descriptors for which
     * exb_conv2d_pool_fusable() returns 1; 0 = plain convolution. */
    int32_t fuse_pool;
    /* Elements between consecutive output pixels of y, 0 = cout_stride.  A larger value lets the convolution
     * write its cout_stride channels into a slice of a wider channel-last tensor (the caller passes y already
     * offset to the slice's first channel): a Concat becomes the producers' epilogue stores
     * (operation_concat, src/Excalibur/operation_concat.cpp:30-80).  Needs the tensor-core kernel, one fp16
     * output, no residual, cout_stride % 16 == 0 and y_pitch % 16 == 0. */
    int32_t y_pitch;
} exb_conv_desc;

/* Output spatial size: (in + pad_a + pad_b - k) / stride + 1
 * (src/Excalibur/operation_convolution.cpp:270-273). */
/* With fuse_pool = 1 these are the dimensions of the pooled map. */
EXB_API int exb_conv_out_dims(const exb_conv_desc* d, int* OH, int* OW);

/* Weight pre-transform, the analogue of the reference's *_tr_kernel repacks done once in
 * init_weights (src/Excalibur/operation_convolution.cpp:88-98,412-467,873-971).  Inputs are
 * HOST pointers in the reference's on-disk layout: OIHW weights [Cout][Cin/group][kh][kw],
 * bias[Cout] or NULL.  fp16 variant converts fp32 -> fp16 (round to nearest even).
 * int8 variant also takes the per-output-channel weight scale table (n_wscale == Cout or 1)
 * and the activation scale of this conv's input, and forms the dequantise multiplier
 * 1.0f / (wscale * act_scale) (0 when |wscale| <= 1e-6) in fp32 on the host exactly as
 * src/Excalibur/operation_convolution.cpp:397-404 does. */
EXB_API int exb_conv_weights_pack_f16(exb_ctx* ctx, const exb_conv_desc* d, const float* w_oihw,
                                      const float* bias, exb_conv_weights** out);
EXB_API int exb_conv_weights_pack_i8(exb_ctx* ctx, const exb_conv_desc* d, const int8_t* w_oihw,
                                     const float* bias, const float* wscale, int n_wscale,
                                     float act_scale, exb_conv_weights** out);
/* Per-output-channel slopes for EXB_ACT_PRELU (operation_prelu / operation_leakyrelu behind a convolution,
 * src/Excalibur/operation_prelu.cpp:58-147): HOST array of n == Cout values, or n == 1 for one shared slope.
 * May be called again to replace them; a forward with act == EXB_ACT_PRELU fails if none were set. */
EXB_API int exb_conv_weights_set_slopes(exb_ctx* ctx, exb_conv_weights* w, const float* slopes, int n);
EXB_API int exb_conv_weights_destroy(exb_conv_weights* w);

/* x: NHWC in_dtype [N][H][W][cin_stride]; y (and y2, residual): NHWC [N][OH][OW][cout_stride].
 * residual / y2 may be NULL when the descriptor says so.  All device pointers, 16-byte aligned. */
EXB_API int exb_conv2d_fwd(exb_ctx* ctx, const exb_conv_desc* d, const void* x,
                           const exb_conv_weights* w, const void* residual, void* y, void* y2,
                           void* stream);
/* Which kernel exb_conv2d_fwd would run for this descriptor: 1 = tcgen05 implicit GEMM,
 * 0 = direct kernel; negative = error. */
EXB_API int exb_conv2d_uses_tensor_cores(const exb_conv_desc* d);
/* 1 when exb_conv2d_fwd can run this descriptor with fuse_pool = 1 (a few-channel stride-2 fp16
 * stem on padded NHWC4 rows with 64 output channels, ReLU or ReLU6, fp16 output and an optional
 * int8 copy, no residual), else 0; negative = error.  The descriptor's own fuse_pool is ignored. */
EXB_API int exb_conv2d_pool_fusable(const exb_conv_desc* d);

/* ---------------------------------------------------------------------------------------
 * Depthwise convolution forward.  Stands in for operation_convolutiondepthwise::forward_*
 * (src/Excalibur/operation_convolutiondepthwise.cpp:18-222, src/Excalibur/cuda/
 * operation_convolutiondepthwise.cu:12-93,146-229).  fp32 math on fp16 or int8 activations;
 * the reference's int8 variant likewise dequantises the WEIGHTS once and computes in fp32
 * (operation_convolutiondepthwise.cpp:184-222).  in_scale multiplies int8 inputs back to real
 * values (1/act_scale); out_scale is the consumer's quantisation multiplier.
 * ------------------------------------------------------------------------------------- */
typedef struct exb_dwconv_desc {
    int32_t N, H, W, C;
    int32_t c_stride;       /* physical channels of x and y, 0 => C */
    int32_t kh, kw, stride_h, stride_w;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t in_dtype;       /* EXB_F16 or EXB_I8 */
    int32_t out_dtype;      /* EXB_F16 or EXB_I8 */
    int32_t act;
    float in_scale;         /* int8 input: real = q * in_scale */
    float out_scale;        /* int8 output: q = sat8(rne(v * out_scale)) */
} exb_dwconv_desc;

/* w: HOST fp32 [C][kh][kw] (the reference's OIHW with Cin/group == 1), bias[C] or NULL. */
EXB_API int exb_dw_weights_pack(exb_ctx* ctx, const exb_dwconv_desc* d, const float* w,
                                const float* bias, exb_dw_weights** out);
/* As exb_conv_weights_set_slopes, n == C or 1. */
EXB_API int exb_dw_weights_set_slopes(exb_ctx* ctx, exb_dw_weights* w, const float* slopes, int n);
EXB_API int exb_dw_weights_destroy(exb_dw_weights* w);
EXB_API int exb_dwconv2d_fwd(exb_ctx* ctx, const exb_dwconv_desc* d, const void* x,
                             const exb_dw_weights* w, void* y, void* stream);

/* ---------------------------------------------------------------------------------------
 * Pooling forward.  Stands in for operation_pooling::forward_* (src/Excalibur/
 * operation_pooling.cpp:80-309, src/Excalibur/cuda/operation_pooling.cu:15-171,276-434) with
 * the CPU path's rules: max ignores padding; average divides by the window clipped to
 * H+pad_bottom / W+pad_right, or by the valid tap count when count_include_pad == 0;
 * pad_mode 0 = ceil, 1 = floor output size; global_pool pools the whole map.
 * A second, int8 copy of the result (q = sat8(rne(v*out2_scale))) can be written at once.
 * ------------------------------------------------------------------------------------- */
typedef struct exb_pool_desc {
    int32_t N, H, W, C;
    int32_t c_stride;       /* physical channels, 0 => C */
    int32_t type;           /* 0 max, 1 average */
    int32_t kh, kw, stride_h, stride_w;
    int32_t pad_t, pad_b, pad_l, pad_r;
    int32_t global_pool;
    int32_t pad_mode;
    int32_t count_include_pad;
    int32_t dtype;          /* EXB_F16, EXB_I8 (max only) or EXB_F32: x and y */
    int32_t out2_dtype;     /* -1 or EXB_I8 */
    float out2_scale;
} exb_pool_desc;

EXB_API int exb_pool_out_dims(const exb_pool_desc* d, int* PH, int* PW);
EXB_API int exb_pool2d_fwd(exb_ctx* ctx, const exb_pool_desc* d, const void* x, void* y,
                           void* y2, void* stream);

/* Pooling of an fp32 NCHW tensor (the reference's own tensor layout) WITHOUT ANY ALLOCATION.
 * This entry point has no counterpart in the reference.  It is meant for callers that must not
 * allocate at the point where they run inference: hosts that hand out all device memory at
 * start-up and forbid cudaMalloc afterwards (hard real-time or safety-reviewed loops), and
 * plug-ins living inside an application whose allocator may not be entered from the inference
 * thread.  It needs no exb_ctx.
 *
 * d->dtype must be EXB_F32 and d->out2_dtype -1; d->c_stride is ignored.  x_nchw is
 * [N][C][H][W], y_nchw [N][C][PH][PW] (exb_pool_out_dims), both device pointers owned by the
 * caller.  The two NHWC intermediates the kernels need are kept in a 16 MiB buffer that is part
 * of the library image on every GPU that loads it (it stays resident until the process exits):
 *   (N*H*W + N*PH*PW) * round_up(C,4) * 4 bytes, each part rounded up to 256, must fit in
 *   16 MiB; larger tensors are refused with EXB_ERR_NOMEM and a message, nothing is launched.
 * The first call on a device looks up the buffer's device address (a query, not an allocation);
 * make that first call before starting a stream capture.  All calls on a device share the
 * buffer: calls whose kernels may overlap on the GPU (different streams, or different threads)
 * race with each other - serialise them.  The buffer keeps the previous call's data; the entry
 * point overwrites every byte it later reads, so no clearing is needed between calls. */
EXB_API int exb_pool2d_nchw_f32_static(int device, const exb_pool_desc* d, const float* x_nchw,
                                       float* y_nchw, void* stream);

/* ---------------------------------------------------------------------------------------
 * Element-wise ops on `count` contiguous elements of dtype EXB_F16 or EXB_F32.
 * exb_eltwise_fwd   - operation_eltwise (src/Excalibur/operation_eltwise.cpp:42-94,
 *                     cuda/operation_eltwise.cu:29-163): type 0 PROD, 1 SUM with coeffs
 *                     (NULL => all 1), 2 MAX over n_in >= 2 inputs, ONE pass.
 * exb_binaryop_fwd  - operation_binaryop equal-shape path (src/Excalibur/
 *                     operation_binaryop.cpp:74-84, cuda/operation_binaryop.cu:94-102):
 *                     op 0 add, 1 sub, 2 mul, 3 div.
 * exb_binaryop_scalar_fwd - its with_scalar mode (operation_binaryop.cpp:389-409).
 * exb_relu_fwd      - operation_relu (src/Excalibur/operation_relu.cpp:31-81,
 *                     cuda/operation_relu.cu:13-73).
 * exb_activation_fwd - the conv suffix activation as a standalone pass
 *                     (operation_general_conv.cpp:127-272).
 * ------------------------------------------------------------------------------------- */
EXB_API int exb_eltwise_fwd(exb_ctx* ctx, int type, int n_in, const void* const* xs,
                            const float* coeffs, void* y, int64_t count, int dtype,
                            void* stream);
EXB_API int exb_binaryop_fwd(exb_ctx* ctx, int op, const void* a, const void* b, void* y,
                             int64_t count, int dtype, void* stream);
EXB_API int exb_binaryop_scalar_fwd(exb_ctx* ctx, int op, const void* a, float scalar, void* y,
                                    int64_t count, int dtype, void* stream);
EXB_API int exb_relu_fwd(exb_ctx* ctx, const void* x, void* y, int64_t count, int dtype,
                         void* stream);
EXB_API int exb_activation_fwd(exb_ctx* ctx, int act, const void* x, void* y, int64_t count,
                               int dtype, void* stream);

/* ---------------------------------------------------------------------------------------
 * Quantise / dequantise passes.  Stand in for quantize_float32_to_int8 /
 * dequantize_int32_to_float32 (src/Excalibur/operation_general_conv.cpp:584-941) and the
 * GPU quant kernels (src/Excalibur/cuda/operation_convolution.cu:449-481).  Per-tensor scale.
 * rounding 0 = half away from zero (reference), 1 = half to even.
 * ------------------------------------------------------------------------------------- */
EXB_API int exb_quantize_fwd(exb_ctx* ctx, const void* x, int in_dtype, int8_t* q,
                             int64_t count, float scale, int rounding, void* stream);
EXB_API int exb_dequantize_fwd(exb_ctx* ctx, const int8_t* q, void* y, int out_dtype,
                               int64_t count, float scale, void* stream);

/* ---------------------------------------------------------------------------------------
 * Graph glue around the convolution trunk.
 *
 * exb_concat_fwd stands in for operation_concat::forward_* (src/Excalibur/
 * operation_concat.cpp:30-150, src/Excalibur/cuda/operation_concat.cu) for a concatenation along
 * one axis, written as a row-wise concatenation: y[r][off_i + k] = x_i[r][k] for k < widths[i],
 * off_i = widths[0] + ... + widths[i-1].  Channel concat of NHWC tensors: rows = N*H*W,
 * widths = channel counts, strides = physical channels.  Channel concat of NCHW tensors:
 * rows = N, widths = strides = C_i*H*W.  Up to 8 inputs; dtype gives the element size only.
 *
 * exb_interp_nearest_fwd stands in for operation_interp's nearest mode (resize_type 1,
 * align_corner 0: src/Excalibur/operation_interp.cpp:247-268, src/Excalibur/cuda/
 * operation_interp.cu:9-66): source index = min((int)(o * (in / (float)out)), in - 1) per axis.
 * channel_last 1: NHWC with c_stride physical channels (EXB_F16, EXB_I8, EXB_F32);
 * channel_last 0: NCHW EXB_F32.
 *
 * exb_channel_affine_fwd computes y = act(x * mul[c] + add[c]); it stands in for
 * operation_batchnorm::forward_* (src/Excalibur/operation_batchnorm.cpp:33-69,123-160: b = slope /
 * sqrt(var + eps), a = bias - slope * mean / sqrt(var + eps)) and for the per-channel
 * normalisation of operation_input (src/Excalibur/operation_input.cpp:61-151).  mul / add are
 * DEVICE fp32 arrays of C entries.  channel_last 1: x is [outer][c_stride] (outer = N*H*W;
 * padding channels are written as 0); channel_last 0: x is [outer][C][inner] (outer = N,
 * inner = H*W).  EXB_F16 or EXB_F32; y may alias x.
 * ------------------------------------------------------------------------------------- */
/* y = x * clamp(alpha*x + beta, 0, 1): operation_hardswish (src/Excalibur/operation_hardswish.cpp:34-71,
 * src/Excalibur/cuda/operation_hardswish.cu:10-36).  EXB_F16 or EXB_F32. */
EXB_API int exb_hardswish_fwd(exb_ctx* ctx, const void* x, void* y, int64_t count, int dtype, float alpha,
                              float beta, void* stream);
/* Network input straight to the Focus layer's output: fp32 NCHW image -> optional y = x * mul[c] + add[c]
 * (operation_input, src/Excalibur/operation_input.cpp:92-96; device arrays of C entries, both or neither)
 * -> space-to-depth as exb_focus_fwd -> channel-last fp16 [N][H/2][W/2][c_stride], c_stride 16 or 32 and
 * >= 4*C, padding channels 0.  Replaces three passes over the image (normalise, ingest, focus). */
EXB_API int exb_nchw_f32_focus_to_nhwc_f16(exb_ctx* ctx, const float* x, void* y, int N, int C, int H, int W,
                                           int c_stride, const float* mul, const float* add, void* stream);
/* y = max(0, min(1, alpha*x + beta)): operation_hardsigmoid (src/Excalibur/operation_hardsigmoid.cpp:34-46).
 * EXB_F16 or EXB_F32. */
EXB_API int exb_hardsigmoid_fwd(exb_ctx* ctx, const void* x, void* y, int64_t count, int dtype, float alpha,
                                float beta, void* stream);
/* Softmax over the channels of every position of an fp32 NCHW tensor, inner = H*W: operation_softmax
 * (src/Excalibur/operation_softmax.cpp:34-96).  x_image_stride: floats between images of x (0 = C*inner;
 * larger for the padded rows an InnerProduct writes); y is dense.  x and y must differ. */
EXB_API int exb_softmax_channels_f32(exb_ctx* ctx, const float* x, float* y, int N, int C, int64_t inner,
                                     int64_t x_image_stride, void* stream);
/* Space-to-depth of operation_yolov5focus (src/Excalibur/operation_yolov5focus.cpp:16-47):
 * out[n][g*C + c][i][j] = in[n][c][2i + g%2][2j + g/2], g = 0..3, output H/2 x W/2 with 4*C channels.
 * Every image of the batch is converted (the reference only converts image 0).
 * channel_last 0: fp32 NCHW; channel_last 1: NHWC with in_stride / out_stride physical channels
 * (EXB_F16, EXB_I8 or EXB_F32; padding channels of the output are written as 0). */
EXB_API int exb_focus_fwd(exb_ctx* ctx, const void* x, void* y, int N, int C, int H, int W, int in_stride,
                          int out_stride, int dtype, int channel_last, void* stream);
/* y[n][c][p] = a[n][c][p] op b[n % b_batch][c], or b op a when b_first != 0 (op as exb_binaryop_fwd):
 * operation_binaryop with a (N,C,H,W) and a (N,C,1,1) operand in either order
 * (src/Excalibur/operation_binaryop.cpp:12-44,168-190).  a and y: [N][inner][c_stride] channel-last or
 * [N][C][inner] planar; b: [b_batch][c_stride] or [b_batch][C]; b_batch is N or 1.  EXB_F16 or EXB_F32;
 * y may alias a. */
EXB_API int exb_binaryop_channel_bcast_fwd(exb_ctx* ctx, int op, const void* a, const void* b, int b_first,
                                           void* y, int N, int b_batch, int C, int c_stride, int64_t inner,
                                           int dtype, int channel_last, void* stream);
/* y = prelu(x * mul[c] + add[c], slope): a BatchNorm followed by a PReLU / LeakyRelu in one pass (the
 * BottleneckCSP tail of the shipped YOLOv5s description).  Arguments as exb_channel_affine_fwd and exb_prelu_fwd. */
EXB_API int exb_channel_affine_prelu_fwd(exb_ctx* ctx, const void* x, void* y, const float* mul, const float* add,
                                         const float* slope, int n_slope, int64_t outer, int C, int c_stride,
                                         int64_t inner, int dtype, int channel_last, void* stream);
/* y = x >= 0 ? x : x * slope[c]: operation_prelu (src/Excalibur/operation_prelu.cpp:58-147; n_slope == C, or 1 for
 * a slope shared by every channel) and operation_leakyrelu (src/Excalibur/operation_leakyrelu.cpp:31-58; n_slope
 * == 1).  slope is a device array.  Tensor indexing as exb_channel_affine_fwd.  EXB_F16 or EXB_F32; y may alias x. */
EXB_API int exb_prelu_fwd(exb_ctx* ctx, const void* x, void* y, const float* slope, int n_slope, int64_t outer,
                          int C, int c_stride, int64_t inner, int dtype, int channel_last, void* stream);
/* Channel-last depth-to-space, the scatter half of a transposed convolution whose kernel equals its stride
 * (operation_deconvolution, src/Excalibur/operation_deconvolution.cpp:83-150: GEMM to a column buffer, then
 * col2im): y[n][h*rh + a][w*rw + b][c] = x[n][h][w][(a*rw + b)*C + c].  x has x_stride physical channels
 * (0 = rh*rw*C), y has y_stride (0 = C; channels c >= C are written as 0).  EXB_F16 or EXB_F32. */
EXB_API int exb_depth_to_space_fwd(exb_ctx* ctx, const void* x, void* y, int N, int H, int W, int rh, int rw,
                                   int C, int x_stride, int y_stride, int dtype, void* stream);
/* Detection-head export in one pass: y[n][a][p][k] = x[n][p][a*K + k], channel-last fp16 x with c_stride >= A*K
 * physical channels and P = H*W positions, fp32 y.  Equals operation_reshape of the (N, A*K, H, W) head to
 * (N, A, K, H*W) followed by operation_transpose 1,0,2 (the tail of the shipped yolov5s_simp description). */
EXB_API int exb_nhwc_f16_split_heads_f32(exb_ctx* ctx, const void* x, float* y, int N, int P, int c_stride, int A,
                                         int K, void* stream);
/* The same scatter from a channel-last fp16 x straight into an fp32 NCHW y (a transposed convolution whose result
 * is a network output): y[n][c][h*rh + a][w*rw + b] = x[n][h][w][(a*rw + b)*C + c]. */
EXB_API int exb_depth_to_space_nchw_f32(exb_ctx* ctx, const void* x, float* y, int N, int H, int W, int rh, int rw,
                                        int C, int x_stride, void* stream);
/* y[p][w][h] = x[p][h][w] for `planes` fp32 planes: operation_transpose with permutation 1,0,2
 * (src/Excalibur/operation_transpose.cpp:47-66). */
EXB_API int exb_transpose_hw_f32(exb_ctx* ctx, const float* x, float* y, int64_t planes, int H, int W,
                                 void* stream);
EXB_API int exb_concat_fwd(exb_ctx* ctx, int n_in, const void* const* xs, const int64_t* widths,
                           const int64_t* x_strides, void* y, int64_t y_stride, int64_t rows,
                           int dtype, void* stream);
EXB_API int exb_interp_nearest_fwd(exb_ctx* ctx, const void* x, void* y, int N, int H, int W, int C,
                                   int c_stride, int OH, int OW, int dtype, int channel_last,
                                   void* stream);
EXB_API int exb_channel_affine_fwd(exb_ctx* ctx, const void* x, void* y, const float* mul,
                                   const float* add, int64_t outer, int C, int c_stride,
                                   int64_t inner, int dtype, int channel_last, int act,
                                   void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EXCALIBUR_B200_H_ */
