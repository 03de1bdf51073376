// fp32 -> fp16 conversion of the network input on the host, so that half as many bytes cross PCIe.
// Round to nearest even, the rounding the device ingest kernels use (__float2half_rn): a forward that
// converts on the host gives bit-identical results to one that converts on the device.
//
// F16C (vcvtps2ph) where the CPU has it, a bit-level conversion otherwise; a persistent pool of worker
// threads splits one buffer into 16-element-aligned ranges.
#pragma once
#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <mutex>
#include <thread>
#include <vector>

namespace glasssix {
namespace excalibur {

// One value, bit level (round to nearest even, overflow to infinity, NaN kept quiet).
uint16_t f32_to_f16_rne(float v);
// n values; force_scalar skips the F16C path (tests).
void convert_f32_to_f16(const float* src, uint16_t* dst, size_t n, bool force_scalar = false);
bool host_has_f16c();

class convert_pool {
public:
    explicit convert_pool(int threads);
    ~convert_pool();
    int threads() const { return (int)workers_.size() + 1; }
    // Converts n values with every thread of the pool (the caller's included); returns when all are done.
    void run(const float* src, uint16_t* dst, size_t n);

private:
    void worker(int index);
    void slice(int index, int parts);
    std::vector<std::thread> workers_;
    std::mutex mu_;
    std::condition_variable start_cv_, done_cv_;
    uint64_t generation_ = 0;
    int pending_ = 0;
    bool stop_ = false;
    const float* src_ = nullptr;
    uint16_t* dst_ = nullptr;
    size_t n_ = 0;
};

}  // namespace excalibur
}  // namespace glasssix
