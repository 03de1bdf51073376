// Best-case tensor-core rate of this GPU, measured with the library's own MMA instruction stream.
//
// Every CTA fills a few K blocks of A (128 rows) and B (n rows) in shared memory with seeded values
// in the 128-byte-swizzled K-major layout the convolution kernel uses, allocates n TMEM columns and lets
// one thread issue tcgen05.mma (kind::i8 or kind::f16, M = 128, N = n, K = 32 bytes) back to back:
// no TMA, no epilogue, no global memory traffic.  What comes out is the denominator of the
// convolution kernel's tensor roofline: the rate the tensor pipe sustains when nothing else is in
// its way (for one and for two CTAs per SM, and per N - narrow N tiles run below the peak because
// the A operand is re-read from shared memory for only N MACs per byte).
//
// The single wait at the end is bounded like every other wait in the library.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace exb {
namespace {

constexpr uint32_t kProbeMaxSpins = 1u << 22;

template <bool kInt8>
__global__ void __launch_bounds__(128, 1) tensor_peak_kernel(int m, int n, int kblk, int iters, uint32_t idesc, int tmem_cols,
                                                             int* error, unsigned long long* cycles, int kb_bytes, int a_sbo,
                                                             int a_shift) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ __align__(8) uint64_t done_bar;
    __shared__ uint32_t tmem_base_smem;
    __shared__ int abort_flag;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    // a_sbo: bytes between consecutive 8-row groups of A (8 * kb_bytes = dense rows; larger = rows of a wider box),
    // a_shift: byte offset of the first row inside its region (a descriptor that starts part-way into a swizzle atom)
    const int a_bytes = (m / 8) * a_sbo + 1024, b_bytes = n * kb_bytes;
    uint8_t* smem_a = smem;
    uint8_t* smem_b = smem + (size_t)kblk * a_bytes;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        abort_flag = 0;
        ptx::mbar_init(&done_bar, 1);
        ptx::fence_mbar_init();
    }
    if (warp == 0) {
        ptx::tmem_alloc(&tmem_base_smem, (uint32_t)tmem_cols);
        ptx::tmem_relinquish();
    }
    // Seeded operand values (power drawn by the tensor pipe depends on the data: zeros would flatter
    // the sustained figure).  int8: any byte; fp16: values in [-1, 1).
    const int total = kblk * (a_bytes + b_bytes);
    uint32_t s = 0x9e3779b9u * (blockIdx.x + 1) + threadIdx.x;
    for (int i = threadIdx.x * 4; i < total; i += blockDim.x * 4) {
        s = s * 1664525u + 1013904223u;
        uint32_t v = s;
        if (!kInt8) {
            const __half2 h = __floats2half2_rn((float)(int)(s >> 16 & 0xffff) * (1.f / 32768.f) - 1.f,
                                                (float)(int)(s & 0xffff) * (1.f / 32768.f) - 1.f);
            v = *reinterpret_cast<const uint32_t*>(&h);
        }
        *reinterpret_cast<uint32_t*>(smem + i) = v;
    }
    ptx::fence_proxy_async();
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_smem;
    if (threadIdx.x == 0) {
        const uint64_t d0 = ptx::make_smem_desc(ptx::smem_u32(smem_a) + (uint32_t)a_shift, (uint32_t)kb_bytes);
        const uint32_t desc_hi = (uint32_t)(d0 >> 32);
        const uint32_t a_hi = (desc_hi & ~0x3FFFu) | (((uint32_t)a_sbo >> 4) & 0x3FFFu);
        const uint32_t a_lo0 = (uint32_t)d0;
        const uint32_t b_lo0 = (uint32_t)ptx::make_smem_desc(ptx::smem_u32(smem_b), (uint32_t)kb_bytes);
        const int ksteps = kb_bytes / 32;
        const uint32_t a_blk = (uint32_t)a_bytes >> 4, b_blk = (uint32_t)b_bytes >> 4;
        const unsigned long long t0 = clock64();
        uint32_t accumulate = 0;
        for (int it = 0; it < iters; ++it) {
            uint32_t a_lo = a_lo0, b_lo = b_lo0;
            for (int kb = 0; kb < kblk; ++kb) {
                if (ksteps == 4) {      // unrolled: the issuing thread's own loop overhead must not be what is measured
                    ptx::tc_mma_ab<kInt8>(tmem_base, a_lo, a_hi, b_lo, desc_hi, idesc, accumulate);
                    ptx::tc_mma_ab<kInt8>(tmem_base, a_lo + 2, a_hi, b_lo + 2, desc_hi, idesc, 1);
                    ptx::tc_mma_ab<kInt8>(tmem_base, a_lo + 4, a_hi, b_lo + 4, desc_hi, idesc, 1);
                    ptx::tc_mma_ab<kInt8>(tmem_base, a_lo + 6, a_hi, b_lo + 6, desc_hi, idesc, 1);
                } else {
                    for (int ks = 0; ks < ksteps; ++ks)
                        ptx::tc_mma_ab<kInt8>(tmem_base, a_lo + 2 * ks, a_hi, b_lo + 2 * ks, desc_hi, idesc, ks ? 1u : accumulate);
                }
                accumulate = 1;
                a_lo += a_blk;
                b_lo += b_blk;
            }
        }
        ptx::tc_commit(&done_bar);
        if (!ptx::mbar_wait_bounded(&done_bar, 0, &abort_flag, kProbeMaxSpins)) atomicExch(error, 8);
        if (cycles && blockIdx.x == 0) *cycles = clock64() - t0;
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (warp == 0) {
        ptx::tc_fence_after_sync();
        ptx::tmem_dealloc(tmem_base, (uint32_t)tmem_cols);
    }
}

}  // namespace
}  // namespace exb

using namespace exb;

extern "C" int exb_tensor_peak_probe_layout(exb_ctx* ctx, int dtype, int m, int n, int ctas_per_sm, int kblk, int iters, int kb_bytes,
                                            int a_sbo, int a_shift, double* ops_per_launch, unsigned long long* d_cycles,
                                            void* stream);
extern "C" int exb_tensor_peak_probe(exb_ctx* ctx, int dtype, int n, int ctas_per_sm, int kblk, int iters,
                                     double* ops_per_launch, unsigned long long* d_cycles, void* stream) {
    return exb_tensor_peak_probe_layout(ctx, dtype, 128, n, ctas_per_sm, kblk, iters, 128, 1024, 0, ops_per_launch, d_cycles, stream);
}

extern "C" int exb_tensor_peak_probe_layout(exb_ctx* ctx, int dtype, int m, int n, int ctas_per_sm, int kblk, int iters, int kb_bytes,
                                            int a_sbo, int a_shift, double* ops_per_launch, unsigned long long* d_cycles,
                                            void* stream) {
    EXB_REQUIRE(ctx != nullptr, "exb_tensor_peak_probe: null context");
    EXB_REQUIRE(dtype == EXB_I8 || dtype == EXB_F16, "exb_tensor_peak_probe: dtype must be EXB_I8 or EXB_F16");
    EXB_REQUIRE(m == 64 || m == 128, "exb_tensor_peak_probe: m must be 64 or 128");
    EXB_REQUIRE(n >= 16 && n <= 256 && n % 16 == 0, "exb_tensor_peak_probe: n must be a multiple of 16 in 16..256");
    EXB_REQUIRE(ctas_per_sm == 1 || ctas_per_sm == 2, "exb_tensor_peak_probe: ctas_per_sm must be 1 or 2");
    EXB_REQUIRE(kblk >= 1 && kblk <= 8 && iters >= 1 && iters <= (1 << 20), "exb_tensor_peak_probe: kblk 1..8, iters 1..2^20");
    EXB_REQUIRE(kb_bytes == 32 || kb_bytes == 64 || kb_bytes == 128, "exb_tensor_peak_probe: kb_bytes must be 32, 64 or 128");
    EXB_REQUIRE(a_sbo >= 8 * kb_bytes && a_sbo % 16 == 0 && a_sbo <= 4096 && a_shift >= 0 && a_shift % 16 == 0 && a_shift < 1024,
                "exb_tensor_peak_probe: a_sbo must be a multiple of 16 in [8 * kb_bytes, 4096], a_shift a multiple of 16 below 1024");
    const size_t smem = (size_t)kblk * ((size_t)(m / 8) * a_sbo + 1024 + (size_t)n * kb_bytes) + 1024;
    const size_t limit = ctas_per_sm == 2 ? (size_t)(228 * 1024 / 2 - 2048) : (size_t)ctx->smem_optin - 1024;
    EXB_REQUIRE(smem <= limit, "exb_tensor_peak_probe: %d K blocks of (%d + %d) rows do not fit shared memory", kblk, m, n);
    int cols = 32;
    while (cols < n) cols *= 2;
    const bool int8 = dtype == EXB_I8;
    const uint32_t idesc = ptx::make_idesc(int8, (uint32_t)m, (uint32_t)n);
    const int grid = ctx->sm_count * ctas_per_sm;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    auto kern = int8 ? tensor_peak_kernel<true> : tensor_peak_kernel<false>;
    EXB_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kern<<<grid, 128, smem, st>>>(m, n, kblk, iters, idesc, cols, ctx->d_error, d_cycles, kb_bytes, a_sbo, a_shift);
    if (ops_per_launch) {
        const double k_per_mma = int8 ? 32.0 : 16.0;
        *ops_per_launch = 2.0 * m * n * k_per_mma * (kb_bytes / 32) * kblk * (double)iters * grid;
    }
    return after_launch("tensor_peak_kernel");
}
