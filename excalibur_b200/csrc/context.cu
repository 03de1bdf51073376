// Context, error reporting and version of the C ABI.
#include <stdlib.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

#include <string.h>

namespace exb {

static thread_local char g_last_error[512] = "no error";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_last_error, sizeof(g_last_error), fmt, ap);
    va_end(ap);
    return code;
}

}  // namespace exb

using namespace exb;

extern "C" const char* exb_last_error_string(void) { return g_last_error; }

extern "C" const char* exb_version(void) { return "0.1.0"; }

extern "C" int exb_ctx_create(int device, exb_ctx** out) {
    EXB_REQUIRE(out != nullptr, "exb_ctx_create: null output pointer");
    *out = nullptr;
    int n = 0;
    EXB_CUDA_TRY(cudaGetDeviceCount(&n));
    EXB_REQUIRE(device >= 0 && device < n, "exb_ctx_create: device %d out of range (%d devices)", device, n);
    EXB_CUDA_TRY(cudaSetDevice(device));
    cudaDeviceProp prop;
    EXB_CUDA_TRY(cudaGetDeviceProperties(&prop, device));
    if (prop.major != 10)
        return fail(EXB_ERR_UNSUPPORTED,
                    "device %d is sm_%d%d; this library only contains sm_100a code", device,
                    prop.major, prop.minor);
    exb_ctx* c = new exb_ctx();
    c->device = device;
    c->sm_count = prop.multiProcessorCount;
    c->smem_optin = (int)prop.sharedMemPerBlockOptin;
    c->d_error = nullptr;
    c->h_error = nullptr;
    {
        const char* e = getenv("EXB_PDL");   // EXB_PDL=0: plain stream-ordered launches of the conv kernel
        c->pdl = (e && e[0] == '0') ? 0 : 1;
    }
    cudaError_t e = cudaMalloc(&c->d_error, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(c->d_error, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMallocHost(&c->h_error, sizeof(int));
    if (e != cudaSuccess) {
        if (c->d_error) cudaFree(c->d_error);
        delete c;
        return fail(EXB_ERR_CUDA, "exb_ctx_create: %s", cudaGetErrorString(e));
    }
    *c->h_error = 0;
    *out = c;
    return EXB_OK;
}

extern "C" int exb_ctx_destroy(exb_ctx* ctx) {
    if (!ctx) return EXB_OK;
    cudaSetDevice(ctx->device);
    if (ctx->d_error) cudaFree(ctx->d_error);
    if (ctx->h_error) cudaFreeHost(ctx->h_error);
    delete ctx;
    return EXB_OK;
}

extern "C" int exb_ctx_sm_count(const exb_ctx* ctx, int* out) {
    EXB_REQUIRE(ctx && out, "exb_ctx_sm_count: null argument");
    *out = ctx->sm_count;
    return EXB_OK;
}

namespace exb {
namespace {
// One thread waits, with the kernels' own bounded wait, on an mbarrier nobody ever arrives at; when the
// limit runs out it records role code 9 in the context's error word and the kernel returns normally.
__global__ void bounded_wait_selftest_kernel(int* error, uint32_t max_polls) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(&bar, 1);
        ptx::fence_mbar_init();
        if (!ptx::mbar_wait_bounded(&bar, 0, &abort_flag, max_polls)) atomicExch(error, 9);
    }
}
}  // namespace
}  // namespace exb

extern "C" int exb_selftest_bounded_wait(exb_ctx* ctx, int max_polls, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "exb_selftest_bounded_wait: null context");
    EXB_REQUIRE(max_polls >= 1 && max_polls <= 4096, "exb_selftest_bounded_wait: max_polls must be 1..4096");
    exb::bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctx->d_error, (uint32_t)max_polls);
    return after_launch("bounded_wait_selftest_kernel");
}

extern "C" int exb_ctx_sync_check(exb_ctx* ctx, void* stream) {
    EXB_REQUIRE(ctx != nullptr, "exb_ctx_sync_check: null context");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    EXB_CUDA_TRY(cudaMemcpyAsync(ctx->h_error, ctx->d_error, sizeof(int), cudaMemcpyDeviceToHost, st));
    EXB_CUDA_TRY(cudaStreamSynchronize(st));
    const int word = *ctx->h_error;
    if (word != 0) {
        EXB_CUDA_TRY(cudaMemsetAsync(ctx->d_error, 0, sizeof(int), st));
        EXB_CUDA_TRY(cudaStreamSynchronize(st));
        return fail(EXB_ERR_TIMEOUT, "a kernel gave up a bounded wait (role code %d)", word);
    }
    return EXB_OK;
}
