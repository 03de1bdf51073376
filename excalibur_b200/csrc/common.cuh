// Shared declarations of the C-ABI implementation: context, error reporting, launch helpers
// and the scalar conversion rules every kernel uses.
#pragma once
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdarg.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/excalibur_b200.h"

struct exb_ctx {
    int device;
    int sm_count;
    int smem_optin;          // max dynamic shared memory per block (opt-in)
    int* d_error;            // device error word written by kernels whose bounded waits ran out
    int* h_error;            // pinned host mirror
    int pdl;                 // launch the conv kernel with programmatic stream serialization (default 1; EXB_PDL=0 turns it off)
};

namespace exb {

// Record a message for exb_last_error_string() and return `code`.
int fail(int code, const char* fmt, ...);

// A failing runtime call is reported once and cleared (cudaGetLastError), so that it cannot be blamed on the next
// launch's check.
#define EXB_CUDA_TRY(expr)                                                                  \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess) {                                                           \
            (void)cudaGetLastError();                                                       \
            return ::exb::fail(EXB_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,                \
                               cudaGetErrorString(e__), __FILE__, __LINE__);                \
        }                                                                                   \
    } while (0)

#define EXB_REQUIRE(cond, ...)                                                              \
    do {                                                                                    \
        if (!(cond)) return ::exb::fail(EXB_ERR_BAD_ARG, __VA_ARGS__);                      \
    } while (0)

// Launch check.  cudaGetLastError returns AND clears the calling thread's error: a launch that was refused (or an
// error some other code of the process left behind) is reported by this call only and does not make every later
// launch of the library fail.  Sticky errors (a faulted context) keep coming back from the runtime by themselves.
inline int after_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess)
        return fail(EXB_ERR_CUDA, "launch of %s failed: %s", what, cudaGetErrorString(e));
    return EXB_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

inline size_t dtype_size(int dt) {
    switch (dt) {
    case EXB_F16: return 2;
    case EXB_I8: return 1;
    case EXB_F32: return 4;
    case EXB_I32: return 4;
    default: return 0;
    }
}

// ---- device-side scalar rules -------------------------------------------------------------
// Quantise, half away from zero then truncate and saturate: the reference's float32_to_int8.
__device__ __forceinline__ int quant_half_away(float v) {
    float t = v >= 0.f ? v + 0.5f : v - 0.5f;
    t = fminf(fmaxf(t, -128.f), 127.f);
    return (int)t;  // truncation toward zero
}
// Quantise, round half to even, saturate.
__device__ __forceinline__ int quant_rne(float v) {
    float t = rintf(v);
    t = fminf(fmaxf(t, -128.f), 127.f);
    return (int)t;
}

// Four floats -> four int8 (round half to even, saturate), packed little-endian in 32 bits.
__device__ __forceinline__ uint32_t quant_pack4(float a, float b, float c, float d, float qscale) {
    const int q0 = __float2int_rn(a * qscale), q1 = __float2int_rn(b * qscale);
    const int q2 = __float2int_rn(c * qscale), q3 = __float2int_rn(d * qscale);
    uint32_t r;
    // cvt.pack.sat.s8.s32.b32 d, a, b, c:  d = (c << 16) | (sat8(a) << 8) | sat8(b)
    asm("{\n\t.reg .b32 t;\n\t"
        "cvt.pack.sat.s8.s32.b32 t, %4, %3, 0;\n\t"
        "cvt.pack.sat.s8.s32.b32 %0, %2, %1, t;\n\t}"
        : "=r"(r)
        : "r"(q0), "r"(q1), "r"(q2), "r"(q3));
    return r;
}

// 1 / (1 + e^-v) for the sigmoid-type activations: hardware reciprocal plus one Newton step (within 1 ulp of the
// IEEE division at a third of its instructions).  The exponent is clamped so that the denominator stays finite
// (the Newton step of an infinite one would be NaN); e^80 already gives a sigmoid of 2e-35.
__device__ __forceinline__ float sigmoid_fast(float v) {
    const float d = 1.f + __expf(fminf(-v, 80.f));
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(d));
    return fmaf(r, fmaf(-d, r, 1.f), r);
}

__device__ __forceinline__ float apply_act(float v, int act) {
    switch (act) {
    case EXB_ACT_NONE: return v;
    case EXB_ACT_RELU: return v >= 0.f ? v : 0.f;
    case EXB_ACT_RELU6_QUIRK: return (v >= 0.f && v <= 6.f) ? v : 0.f;
    case EXB_ACT_SIGMOID: return sigmoid_fast(v);
    case EXB_ACT_MISH: return v * tanhf(v > 20.f ? v : log1pf(expf(v)));   // ln(1 + e^v) = v to fp32 accuracy above 20
    case EXB_ACT_RELU6: return fminf(fmaxf(v, 0.f), 6.f);
    case EXB_ACT_SILU: return v * sigmoid_fast(v);
    case EXB_ACT_HARDSWISH: return v * fminf(fmaxf(fmaf(v, 1.f / 6.f, 0.5f), 0.f), 1.f);
    default: return v;
    }
}

// The same over a small register vector, with the selector outside the element loop: one uniform
// branch per vector instead of a switch per element.
template <int N>
__device__ __forceinline__ void apply_act_vec(float (&v)[N], int act) {
    if (act == EXB_ACT_NONE) return;
    if (act == EXB_ACT_RELU) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = fmaxf(v[i], 0.f);
    } else if (act == EXB_ACT_RELU6) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = fminf(fmaxf(v[i], 0.f), 6.f);
    } else if (act == EXB_ACT_SILU) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = v[i] * sigmoid_fast(v[i]);
    } else if (act == EXB_ACT_HARDSWISH) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = v[i] * fminf(fmaxf(fmaf(v[i], 1.f / 6.f, 0.5f), 0.f), 1.f);
    } else if (act == EXB_ACT_SIGMOID) {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = sigmoid_fast(v[i]);
    } else {
#pragma unroll
        for (int i = 0; i < N; ++i) v[i] = apply_act(v[i], act);
    }
}

inline bool act_supported(int act) {
    return act == EXB_ACT_NONE || act == EXB_ACT_RELU || act == EXB_ACT_RELU6_QUIRK ||
           act == EXB_ACT_SIGMOID || act == EXB_ACT_MISH || act == EXB_ACT_RELU6 || act == EXB_ACT_SILU || act == EXB_ACT_HARDSWISH;
}

// Grid for a bandwidth-bound grid-stride kernel: enough CTAs to fill every SM a few times
// over, a multiple of the SM count, never more than the work needs.
inline int stream_grid(const exb_ctx* ctx, int64_t work_items, int threads, int ctas_per_sm = 8) {
    int64_t need = (work_items + threads - 1) / threads;
    int64_t cap = (int64_t)ctx->sm_count * ctas_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

}  // namespace exb
