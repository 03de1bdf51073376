// One batch, several GPUs, one result: batch sharding as a product call.
//
// Inference images are independent, so a batch is cut into contiguous slices, one per replica; every replica
// is a pipeline<float> on its own device (the reference's pipeline takes a device id per instance,
// include/Excalibur/pipeline.hpp:24-26) driven by its own host thread and stream, with the weights replicated.
// The host scatters input slices by pointer offset (no staging copy: each replica uploads its slice from the
// caller's buffer) and gathers every output by row offset into one tensor.  There is no collective and no peer
// access on the data path.
#pragma once
#include <string>
#include <string_view>
#include <thread>
#include <vector>

#include "pipeline.hpp"

namespace glasssix {
namespace excalibur {

// Contiguous slice [lo, hi) of `total` items for shard `rank` of `world`: the first total % world shards get one
// item more.  (excalibur_b200/sharding.py::shard_bounds is the same rule for the one-process-per-GPU launcher.)
EXB_HOST_API void shard_bounds(int total, int world, int rank, int* lo, int* hi);

// Rows of `parts` (part i holds part_rows[i] rows of row_elems floats) written one after the other into `out`.
EXB_HOST_API void gather_rows(const float* const* parts, const int* part_rows, int n_parts, int64_t row_elems, float* out);

class EXB_HOST_API sharded_pipeline {
public:
    typedef pipeline<float>::result_map result_map;
    // One replica per entry of `devices` (a device may appear more than once: replicas then share that GPU).
    sharded_pipeline(const std::vector<std::string>& lines, std::string_view model_file, const std::vector<int>& devices);
    ~sharded_pipeline();

    // forward of N images in host memory (fp32 NCHW, page-locked for asynchronous uploads): slice r goes to replica
    // r; replicas whose slice is empty (N < replicas) do not run.  Returns every output for all N images.
    result_map forward(const float* input, int N, int C, int H, int W);
    result_map forward(const std::shared_ptr<memory::tensor<float>>& input);

    int replicas() const { return (int)nets_.size(); }
    pipeline<float>& replica(int r) { return *nets_[r]; }
    std::vector<std::string> output_names() const;
    // slowest replica's device time of the last forward, ms
    double device_ms_last_forward() const { return device_ms_; }

private:
    std::vector<std::unique_ptr<pipeline<float>>> nets_;
    std::vector<int> devices_;
    double device_ms_ = 0.0;
    DISABLE_COPY_AND_ASSIGN(sharded_pipeline);
};

}  // namespace excalibur
}  // namespace glasssix
