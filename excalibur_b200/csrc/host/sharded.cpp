// sharded_pipeline: see sharded.hpp.
#include "sharded.hpp"

#include <cstring>
#include <exception>

namespace glasssix {
namespace excalibur {

void shard_bounds(int total, int world, int rank, int* lo, int* hi) {
    CHECK(world > 0 && rank >= 0 && rank < world && total >= 0) << "bad shard request total=" << total << " world=" << world
                                                                  << " rank=" << rank;
    const int base = total / world, extra = total % world;
    *lo = rank * base + (rank < extra ? rank : extra);
    *hi = *lo + base + (rank < extra ? 1 : 0);
}

void gather_rows(const float* const* parts, const int* part_rows, int n_parts, int64_t row_elems, float* out) {
    int64_t at = 0;
    for (int i = 0; i < n_parts; ++i) {
        if (part_rows[i] <= 0) continue;
        std::memcpy(out + at, parts[i], sizeof(float) * (size_t)(part_rows[i] * row_elems));
        at += part_rows[i] * row_elems;
    }
}

sharded_pipeline::sharded_pipeline(const std::vector<std::string>& lines, std::string_view model_file,
                                   const std::vector<int>& devices)
    : devices_(devices) {
    CHECK(!devices.empty()) << "sharded_pipeline needs at least one device";
    for (int d : devices) {
        CHECK_GE(d, 0) << "sharded_pipeline runs on GPUs only";
        nets_.emplace_back(new pipeline<float>(lines, model_file, d));
    }
}

sharded_pipeline::~sharded_pipeline() {}

std::vector<std::string> sharded_pipeline::output_names() const { return nets_[0]->output_names(); }

sharded_pipeline::result_map sharded_pipeline::forward(const std::shared_ptr<memory::tensor<float>>& input) {
    CHECK(input != nullptr && !input->empty()) << "empty input tensor";
    if (input->order() == memory::NHWC) input->convert_order();
    return forward(input->cpu_data(), input->num(), input->channels(), input->height(), input->width());
}

sharded_pipeline::result_map sharded_pipeline::forward(const float* input, int N, int C, int H, int W) {
    CHECK(input != nullptr && N > 0 && C > 0 && H > 0 && W > 0) << "bad input";
    const int G = (int)nets_.size();
    const int64_t image = (int64_t)C * H * W;
    std::vector<result_map> part(G);
    std::vector<int> rows(G, 0);
    std::vector<std::string> failure(G);
    std::vector<std::thread> workers;
    auto run = [&](int r) {
        int lo = 0, hi = 0;
        shard_bounds(N, G, r, &lo, &hi);
        rows[r] = hi - lo;
        if (hi == lo) return;
        try {
            CUDA_CHECK(cudaSetDevice(devices_[r]));
            // a tensor that borrows this replica's slice of the caller's buffer
            auto t = std::shared_ptr<memory::tensor<float>>(
                new memory::tensor<float>(std::vector<int>{hi - lo, C, H, W}, devices_[r], memory::NCHW, nullptr));
            t->data()->set_external_cpu_data(const_cast<float*>(input + lo * image));
            part[r] = nets_[r]->forward(t);
        } catch (const std::exception& e) {
            failure[r] = e.what();
        }
    };
    // LOG(FATAL) terminates unless a handler that throws is installed (the C entry points install one); the
    // handler is a process-wide setting, so worker threads see the caller's and their failures are re-raised here.
    for (int r = 1; r < G; ++r) workers.emplace_back(run, r);
    run(0);
    for (auto& w : workers) w.join();
    for (int r = 0; r < G; ++r)
        if (!failure[r].empty()) LOG(FATAL) << "replica " << r << " (device " << devices_[r] << "): " << failure[r];
    device_ms_ = 0.0;
    for (int r = 0; r < G; ++r)
        if (rows[r] > 0 && nets_[r]->device_ms_last_forward() > device_ms_) device_ms_ = nets_[r]->device_ms_last_forward();
    // gather by row offset
    result_map out;
    int first = 0;
    while (first < G && rows[first] == 0) ++first;
    CHECK_LT(first, G);
    for (const auto& kv : part[first]) {
        const std::vector<int> shp = kv.second->data_shape();
        const int64_t row_elems = (int64_t)shp[1] * shp[2] * shp[3];
        auto full = std::shared_ptr<memory::tensor<float>>(
            new memory::tensor<float>(std::vector<int>{N, shp[1], shp[2], shp[3]}, -1, memory::NCHW, nullptr));
        std::vector<const float*> ptrs(G, nullptr);
        for (int r = 0; r < G; ++r) {
            if (rows[r] == 0) continue;
            auto it = part[r].find(kv.first);
            CHECK(it != part[r].end() && it->second && it->second->num() == rows[r]) << "replica " << r << " returned no " << kv.first;
            ptrs[r] = it->second->cpu_data();
        }
        gather_rows(ptrs.data(), rows.data(), G, row_elems, full->mutable_cpu_data());
        out[kv.first] = full;
    }
    return out;
}

}  // namespace excalibur
}  // namespace glasssix
