// Test infrastructure, not product code.
//
// extern "C" shim around the UNMODIFIED reference library (glasssix::excalibur::pipeline<float>,
// reference include/Excalibur/pipeline.hpp:18-45) so that Python tests and the CPU-baseline leg
// of the benchmark can drive it through ctypes.  It is compiled together with the reference's
// own sources by oracle/Makefile (target `ref`) into oracle/_ref/libexcalibur_ref.so.
//
// Graphs are given as the text of a .phai file (one op per line, pipeline.cpp:54-116) and the
// path of a .racy weight file (operation_convolution.cpp:71-152); everything runs on the CPU
// (device -1).
#include "Excalibur/pipeline.hpp"

#include <cstring>
#include <memory>
#include <sstream>
#include <string>
#include <unordered_map>
#include <vector>

using glasssix::excalibur::pipeline;
using glasssix::memory::tensor;

namespace {
struct ref_handle {
    std::unique_ptr<pipeline<float>> net;
    std::unordered_map<std::string, std::shared_ptr<tensor<float>>> outputs;
};

int copy_out(const std::shared_ptr<tensor<float>>& t, float* out, long long cap, int* shape4) {
    if (!t || t->empty()) return -1;
    auto shp = t->data_shape();
    for (int i = 0; i < 4; ++i) shape4[i] = i < (int)shp.size() ? shp[i] : 1;
    long long n = t->count();
    if (out == nullptr) return 0;       // shape query only
    if (n > cap) return -2;
    std::memcpy(out, t->cpu_data(), sizeof(float) * n);
    return 0;
}
}  // namespace

extern "C" {

void* ref_pipeline_create(const char* phai_text, const char* racy_path) {
    std::vector<std::string> lines;
    std::istringstream ss(phai_text);
    std::string line;
    while (std::getline(ss, line)) {
        while (!line.empty() && (line.back() == '\r' || line.back() == ' ')) line.pop_back();
        if (!line.empty()) lines.push_back(line);
    }
    auto* h = new ref_handle;
    h->net.reset(new pipeline<float>(lines, std::string_view(racy_path ? racy_path : ""), -1));
    return h;
}

void ref_pipeline_destroy(void* p) { delete static_cast<ref_handle*>(p); }

// input is NCHW fp32 (order 0) or NHWC fp32 (order 1), copied into a reference tensor.
int ref_pipeline_forward(void* p, const float* input, int n, int c, int h, int w, int order) {
    auto* hd = static_cast<ref_handle*>(p);
    std::vector<int> shape = order == 0 ? std::vector<int>{n, c, h, w} : std::vector<int>{n, h, w, c};
    auto in = std::make_shared<tensor<float>>(shape, -1,
        order == 0 ? glasssix::memory::NCHW : glasssix::memory::NHWC, nullptr);
    std::memcpy(in->mutable_cpu_data(), input, sizeof(float) * (size_t)n * c * h * w);
    hd->outputs = hd->net->forward(in);
    return (int)hd->outputs.size();
}

// Name of the i-th pipeline output of the last forward (iteration order of the result map).
int ref_pipeline_output_name(void* p, int i, char* buf, int cap) {
    auto* hd = static_cast<ref_handle*>(p);
    int k = 0;
    for (auto& kv : hd->outputs) {
        if (k++ == i) {
            std::strncpy(buf, kv.first.c_str(), cap - 1);
            buf[cap - 1] = 0;
            return 0;
        }
    }
    return -1;
}

// Any feature map by name (pipeline::get_featmap, pipeline.hpp:32). out == NULL => shape only.
int ref_pipeline_get_featmap(void* p, const char* name, float* out, long long cap, int* shape4) {
    auto* hd = static_cast<ref_handle*>(p);
    auto it = hd->outputs.find(name);
    if (it != hd->outputs.end()) return copy_out(it->second, out, cap, shape4);
    return copy_out(hd->net->get_featmap(name), out, cap, shape4);
}

}  // extern "C"
