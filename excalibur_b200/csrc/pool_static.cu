// Pooling on the reference's fp32 NCHW tensors for callers that are not allowed to allocate.
//
// The library's kernels work on NHWC data, so pooling an NCHW tensor needs two intermediate
// buffers (the NHWC copy of the input and the NHWC result).  The regular path expects the caller
// to provide them; here they live in a fixed array that is part of the library image instead, so
// the entry point below performs no allocation of any kind.
#include "common.cuh"

#include <mutex>

namespace {

constexpr size_t kStaticScratchBytes = size_t(16) << 20;   // 16 MiB, resident on every GPU that loads the library

// Device-side storage.  In host code this name is only a handle for cudaGetSymbolAddress; the
// kernels get the device address obtained from it.
static __device__ __align__(256) unsigned char g_pool_scratch[kStaticScratchBytes];

struct device_setup {
    bool ready = false;
    void* scratch = nullptr;
    int sm_count = 0;
};
constexpr int kMaxDevices = 64;
device_setup g_setup[kMaxDevices];
std::mutex g_setup_mutex;

size_t round256(size_t v) { return (v + 255) & ~size_t(255); }

// Puts the caller's current device back on every way out of the entry point.
struct device_restore {
    int saved = -1;
    ~device_restore() {
        if (saved >= 0) cudaSetDevice(saved);
    }
};

}  // namespace

extern "C" int exb_pool2d_nchw_f32_static(int device, const exb_pool_desc* d, const float* x_nchw, float* y_nchw,
                                          void* stream) {
    using namespace exb;
    EXB_REQUIRE(d != nullptr, "exb_pool2d_nchw_f32_static: null descriptor");
    EXB_REQUIRE(device >= 0 && device < kMaxDevices, "exb_pool2d_nchw_f32_static: device %d out of range", device);
    if (d->dtype != EXB_F32 || d->out2_dtype != -1)
        return fail(EXB_ERR_UNSUPPORTED, "exb_pool2d_nchw_f32_static handles fp32 tensors without a second output");
    EXB_REQUIRE(d->N >= 0 && d->C > 0 && d->H > 0 && d->W > 0, "exb_pool2d_nchw_f32_static: bad tensor shape");

    exb_pool_desc nd = *d;
    nd.c_stride = (d->C + 3) / 4 * 4;   // the fp32 pooling kernel moves 4 channels per thread
    int PH = 0, PW = 0;
    if (int rc = exb_pool_out_dims(&nd, &PH, &PW)) return rc;
    const size_t in_bytes = round256((size_t)d->N * d->H * d->W * nd.c_stride * sizeof(float));
    const size_t out_bytes = round256((size_t)d->N * PH * PW * nd.c_stride * sizeof(float));
    if (in_bytes + out_bytes > kStaticScratchBytes)
        return fail(EXB_ERR_NOMEM,
                    "exb_pool2d_nchw_f32_static: this tensor needs %zu bytes of intermediate storage, the built-in "
                    "buffer holds %zu; use exb_pool2d_fwd with caller-provided buffers",
                    in_bytes + out_bytes, kStaticScratchBytes);
    if (d->N == 0) return EXB_OK;
    EXB_REQUIRE(x_nchw && y_nchw, "exb_pool2d_nchw_f32_static: null tensor");

    device_restore restore;
    EXB_CUDA_TRY(cudaGetDevice(&restore.saved));
    EXB_CUDA_TRY(cudaSetDevice(device));
    device_setup st;
    {
        // First call on this device: resolve the device address of the built-in buffer.  It is a
        // query, not an allocation, and it is done with the device current.
        std::lock_guard<std::mutex> lock(g_setup_mutex);
        device_setup& s = g_setup[device];
        if (!s.ready) {
            void* p = nullptr;
            cudaError_t e = cudaGetSymbolAddress(&p, g_pool_scratch);
            if (e != cudaSuccess || p == nullptr) (void)cudaGetLastError();
            if (e != cudaSuccess || p == nullptr)
                return fail(EXB_ERR_CUDA, "exb_pool2d_nchw_f32_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            int sms = 0;
            e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device);
            if (e != cudaSuccess) return fail(EXB_ERR_CUDA, "exb_pool2d_nchw_f32_static: %s", cudaGetErrorString(e));
            s.scratch = p;
            s.sm_count = sms;
            s.ready = true;
        }
        st = s;
    }

    // A context value that only carries what the three kernels' launch helpers read.
    exb_ctx local{};          // every field zero: no error word, no programmatic dependent launch
    local.device = device;
    local.sm_count = st.sm_count;

    unsigned char* in_nhwc = static_cast<unsigned char*>(st.scratch);
    unsigned char* out_nhwc = in_nhwc + in_bytes;
    // Every byte of both regions that is read later is written first (the layout kernel also
    // writes the padding channels), so nothing depends on what an earlier call left behind.
    if (int rc = exb_nchw_f32_to_nhwc(&local, x_nchw, in_nhwc, EXB_F32, d->N, d->C, d->H, d->W, nd.c_stride, 1.f, 0, stream))
        return rc;
    if (int rc = exb_pool2d_fwd(&local, &nd, in_nhwc, out_nhwc, nullptr, stream)) return rc;
    return exb_nhwc_to_nchw_f32(&local, out_nhwc, EXB_F32, y_nchw, d->N, d->C, PH, PW, nd.c_stride, 1.f, stream);
}
