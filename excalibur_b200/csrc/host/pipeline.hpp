// Graph executor with the reference's public interface (include/Excalibur/pipeline.hpp:18-45):
// parse a .phai description, create operations through the reflector, load .racy weights in
// file order, run forward.  pipeline<float> on a GPU device additionally builds a FUSED plan
// (Conv + ReLU, Conv + residual add + ReLU, requantisation to the next int8 conv's scale, NHWC
// fp16/int8 tensors between kernels, CUDA-graph replay); set_fusion(false) runs op by op with
// the reference's tensor semantics instead.
#pragma once
#include <string>
#include <string_view>
#include <unordered_map>
#include <vector>

#include "operation.hpp"

namespace glasssix {
namespace excalibur {

// What dump_profile writes: a chrome://tracing file with one "B" / "E" event pair per (name, begin, end) entry.
EXB_HOST_API bool write_chrome_trace(std::string_view path, const std::vector<std::string>& names,
                                     const std::vector<double>& begin_ms, const std::vector<double>& end_ms);

template <typename Dtype>
class EXB_HOST_API pipeline {
public:
    class impl;
    typedef std::unordered_map<std::string, std::shared_ptr<memory::tensor<Dtype>>> result_map;

    explicit pipeline();
    explicit pipeline(std::string_view param_file, std::string_view model_file, int device = -1);
    explicit pipeline(std::string_view param_file, int device = -1);
    explicit pipeline(const std::vector<std::string>& hardcode_params, std::string_view model_file, int device = -1);
    ~pipeline();

    result_map forward(const std::shared_ptr<memory::tensor<Dtype>>& input_tensor);
    result_map forward_cpu(const std::shared_ptr<memory::tensor<Dtype>>& input_tensor);
    result_map forward_gpu(const std::shared_ptr<memory::tensor<Dtype>>& input_tensor);
    std::shared_ptr<memory::tensor<Dtype>> get_featmap(std::string_view featmap_name);
    // With the fused plan, "<name>:int8" returns the quantised form of a feature map that int8 convolutions read
    // (raw integers -128..127 as Dtype, not dequantised), or nullptr when the plan keeps no such form.

    void enable_profiler();
    void disable_profiler();
    // chrome://tracing JSON of the last profiled forward ("B"/"E" events per op, device time).
    bool dump_profile(std::string_view path);

    // Extras of this implementation.
    int device() const;                  // the device id given at construction (-1 = none)
    void set_fusion(bool on);            // default on for pipeline<float> on a GPU
    void set_cuda_graph(bool on);        // replay the fused plan as a CUDA graph (default on)
    // forward() of a batch divisible by k runs as k sub-batches: sub-batch c+1 is copied to the device
    // while sub-batch c is computed (default 1 = whole batch at once).  Only the pipeline outputs
    // cover the whole batch afterwards; get_featmap() of an inner map sees the last sub-batch.
    void set_h2d_chunks(int k);
    // t > 0: the forward converts the input to fp16 on the host with t threads before it is copied (half the
    // PCIe bytes, the same round-to-nearest-even as the device ingest kernel, so identical results); used
    // where the plan's ingest step can read fp16 planes (a 3-channel image feeding an fp16 stem conv, no
    // Input normalisation), ignored elsewhere.  Default 0 = the fp32 input is copied as it is.
    void set_host_f16_threads(int t);
    // Re-run the fused plan `iters` times on the input already resident on the device (the last
    // forward's), no host<->device copies; returns the device time in ms between CUDA events on the
    // plan's stream, or a negative value when there is no fused plan yet.
    double run_resident(int iters);
    // Per-kernel device times of the last profiled forward.
    int trace_size() const;
    bool trace_entry(int i, std::string& name, double& begin_ms, double& end_ms) const;
    int launches_last_forward() const;   // kernels launched by the last forward
    double device_ms_last_forward() const;   // device time of the last forward's kernels (events)
    std::vector<std::string> input_names() const;
    std::vector<std::string> output_names() const;

    static std::string version();

private:
    impl* impl_;
    DISABLE_COPY_AND_ASSIGN(pipeline);
};

}  // namespace excalibur
}  // namespace glasssix
