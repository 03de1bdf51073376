#include "host_convert.hpp"

#include <cstring>

#if defined(__x86_64__) || defined(__i386__)
#include <immintrin.h>
#define EXB_X86 1
#endif

namespace glasssix {
namespace excalibur {

uint16_t f32_to_f16_rne(float v) {
    uint32_t x;
    std::memcpy(&x, &v, 4);
    const uint32_t sign = (x >> 16) & 0x8000u;
    x &= 0x7fffffffu;
    if (x >= 0x7f800000u) return (uint16_t)(sign | (x > 0x7f800000u ? 0x7e00u : 0x7c00u));   // NaN, infinity
    if (x >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);                                   // >= 65536
    if (x < 0x38800000u) {
        // below the smallest normal half (2^-14): adding 0.5f aligns the value's bits with the half's
        // subnormal mantissa in the low bits of the sum, and the float addition rounds to nearest even
        float f;
        std::memcpy(&f, &x, 4);
        f += 0.5f;
        uint32_t y;
        std::memcpy(&y, &f, 4);
        return (uint16_t)(sign | (y - 0x3f000000u));
    }
    // normal: re-bias the exponent (127 -> 15) and round the 13 dropped mantissa bits to nearest even;
    // a carry out of the mantissa moves into the exponent, up to infinity for values >= 65520
    const uint32_t odd = (x >> 13) & 1u;
    x += ((uint32_t)(15 - 127) << 23) + 0xfffu + odd;
    return (uint16_t)(sign | (x >> 13));
}

#ifdef EXB_X86
__attribute__((target("avx,f16c"))) static void convert_f16c(const float* src, uint16_t* dst, size_t n) {
    size_t i = 0;
    for (; i + 16 <= n; i += 16) {
        const __m256 a = _mm256_loadu_ps(src + i), b = _mm256_loadu_ps(src + i + 8);
        _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i), _mm256_cvtps_ph(a, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
        _mm_storeu_si128(reinterpret_cast<__m128i*>(dst + i + 8),
                         _mm256_cvtps_ph(b, _MM_FROUND_TO_NEAREST_INT | _MM_FROUND_NO_EXC));
    }
    for (; i < n; ++i) dst[i] = f32_to_f16_rne(src[i]);
}
bool host_has_f16c() {
    static const bool has = __builtin_cpu_supports("f16c") && __builtin_cpu_supports("avx");
    return has;
}
#else
bool host_has_f16c() { return false; }
#endif

void convert_f32_to_f16(const float* src, uint16_t* dst, size_t n, bool force_scalar) {
#ifdef EXB_X86
    if (!force_scalar && host_has_f16c()) {
        convert_f16c(src, dst, n);
        return;
    }
#endif
    (void)force_scalar;
    for (size_t i = 0; i < n; ++i) dst[i] = f32_to_f16_rne(src[i]);
}

convert_pool::convert_pool(int threads) {
    if (threads < 1) threads = 1;
    for (int t = 1; t < threads; ++t) workers_.emplace_back([this, t] { worker(t); });
}

convert_pool::~convert_pool() {
    {
        std::lock_guard<std::mutex> lk(mu_);
        stop_ = true;
    }
    start_cv_.notify_all();
    for (auto& w : workers_) w.join();
}

void convert_pool::slice(int index, int parts) {
    // ranges start on multiples of 16 values so every thread but the last runs whole vectors
    const size_t per = (n_ / parts) & ~(size_t)15;
    const size_t a = per * index, b = index == parts - 1 ? n_ : per * (index + 1);
    if (b > a) convert_f32_to_f16(src_ + a, dst_ + a, b - a);
}

void convert_pool::worker(int index) {
    uint64_t seen = 0;
    for (;;) {
        {
            std::unique_lock<std::mutex> lk(mu_);
            start_cv_.wait(lk, [&] { return stop_ || generation_ != seen; });
            if (stop_) return;
            seen = generation_;
        }
        slice(index, threads());
        {
            std::lock_guard<std::mutex> lk(mu_);
            if (--pending_ == 0) done_cv_.notify_one();
        }
    }
}

void convert_pool::run(const float* src, uint16_t* dst, size_t n) {
    const int parts = threads();
    {
        std::lock_guard<std::mutex> lk(mu_);
        src_ = src;
        dst_ = dst;
        n_ = n;
        pending_ = parts - 1;
        ++generation_;
    }
    start_cv_.notify_all();
    slice(0, parts);
    std::unique_lock<std::mutex> lk(mu_);
    done_cv_.wait(lk, [&] { return pending_ == 0; });
}

}  // namespace excalibur
}  // namespace glasssix
