// C entry points of the host layer (include/excalibur_b200_host.h).
#include "../../../include/excalibur_b200_host.h"

#include <cstring>
#include <sstream>

#include "ops.hpp"
#include "host_convert.hpp"
#include "pipeline.hpp"
#include "sharded.hpp"

using namespace glasssix;
using namespace glasssix::excalibur;

namespace {
thread_local std::string g_err = "no error";

void throwing_handler(const std::string& msg) { throw fatal_error(msg); }

struct fatal_guard {
    fatal_handler_t prev;
    fatal_guard() : prev(get_fatal_handler()) { set_fatal_handler(throwing_handler); }
    ~fatal_guard() { set_fatal_handler(prev); }
};

template <typename F>
int guarded(F f) {
    fatal_guard g;
    try {
        return f();
    } catch (const fatal_error& e) {
        g_err = e.what();
        return EXB_HOST_FATAL;
    } catch (const std::exception& e) {
        g_err = e.what();
        return EXB_HOST_FATAL;
    }
}

struct host_pipeline {
    std::unique_ptr<pipeline<float>> net;
    pipeline<float>::result_map outputs;
    std::vector<std::string> names;
};

int copy_out(const std::shared_ptr<memory::tensor<float>>& t, float* out, int64_t cap, int* shape4) {
    if (!t) {
        g_err = "no such feature map (or it was fused away)";
        return EXB_ERR_BAD_ARG;
    }
    auto shp = t->data_shape();
    for (int i = 0; i < 4; ++i) shape4[i] = shp[i];
    if (!out) return EXB_OK;
    if ((int64_t)t->count() > cap) {
        g_err = "output buffer too small";
        return EXB_ERR_BAD_ARG;
    }
    std::memcpy(out, t->cpu_data(), sizeof(float) * (size_t)t->count());
    return EXB_OK;
}

struct host_pipeline_f16 {
    std::unique_ptr<pipeline<unsigned short>> net;
    pipeline<unsigned short>::result_map outputs;
};

struct host_sharded {
    std::unique_ptr<sharded_pipeline> net;
    sharded_pipeline::result_map outputs;
    std::vector<std::string> names;
};

std::vector<std::string> split_lines(const char* text) {
    std::vector<std::string> lines;
    std::istringstream in(text ? text : "");
    std::string l;
    while (std::getline(in, l)) {
        while (!l.empty() && (l.back() == '\r' || l.back() == '\n')) l.pop_back();
        lines.push_back(l);
    }
    return lines;
}
}  // namespace

extern "C" const char* exb_host_last_error(void) { return g_err.c_str(); }

extern "C" int exb_host_registered(const char* class_name) {
    return operation_reflector<float>::instance().has(class_name) ? 1 : 0;
}

extern "C" int exb_host_pipeline_create(const char* phai_text, const char* racy_path, int device, void** out) {
    return guarded([&]() {
        set_log_quiet(true);
        std::vector<std::string> lines;
        std::istringstream ss(phai_text);
        std::string l;
        while (std::getline(ss, l)) {
            while (!l.empty() && (l.back() == '\r' || l.back() == ' ')) l.pop_back();
            lines.push_back(l);
        }
        auto* h = new host_pipeline;
        h->net.reset(new pipeline<float>(lines, racy_path ? racy_path : "", device));
        *out = h;
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_destroy(void* p) {
    return guarded([&]() {
        delete static_cast<host_pipeline*>(p);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_set_option(void* p, const char* key, int value) {
    auto* h = static_cast<host_pipeline*>(p);
    const std::string k = key;
    if (k == "fusion") h->net->set_fusion(value != 0);
    else if (k == "cuda_graph") h->net->set_cuda_graph(value != 0);
    else if (k == "profile") value ? h->net->enable_profiler() : h->net->disable_profiler();
    else if (k == "h2d_chunks") h->net->set_h2d_chunks(value);
    else if (k == "host_f16_threads") h->net->set_host_f16_threads(value);
    else {
        g_err = "unknown option " + k;
        return EXB_ERR_BAD_ARG;
    }
    return EXB_OK;
}

extern "C" int exb_host_pipeline_forward(void* p, const float* input, int N, int C, int H, int W) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline*>(p);
        // a tensor that borrows the caller's host memory
        auto t = std::shared_ptr<memory::tensor<float>>(
            new memory::tensor<float>(std::vector<int>{N, C, H, W}, h->net->device(), memory::NCHW, nullptr));
        t->data()->set_external_cpu_data(const_cast<float*>(input));
        h->outputs = h->net->forward(t);
        h->names.clear();
        for (auto& n : h->net->output_names()) h->names.push_back(n);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_num_outputs(void* p) { return (int)static_cast<host_pipeline*>(p)->names.size(); }

extern "C" int exb_host_pipeline_output_name(void* p, int i, char* buf, int cap) {
    auto* h = static_cast<host_pipeline*>(p);
    if (i < 0 || i >= (int)h->names.size() || cap <= 0) return EXB_ERR_BAD_ARG;
    std::strncpy(buf, h->names[i].c_str(), cap - 1);
    buf[cap - 1] = 0;
    return EXB_OK;
}

extern "C" int exb_host_pipeline_get(void* p, const char* name, float* out, int64_t cap, int* shape4) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline*>(p);
        auto it = h->outputs.find(name);
        if (it != h->outputs.end()) return copy_out(it->second, out, cap, shape4);
        return copy_out(h->net->get_featmap(name), out, cap, shape4);
    });
}

extern "C" int exb_host_pipeline_output_ptr(void* p, const char* name, const float** data, int* shape4) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline*>(p);
        auto it = h->outputs.find(name);
        if (it == h->outputs.end() || !it->second) {
            g_err = std::string("not an output of the last forward: ") + name;
            return (int)EXB_ERR_BAD_ARG;
        }
        auto shp = it->second->data_shape();
        for (int i = 0; i < 4; ++i) shape4[i] = shp[i];
        *data = it->second->cpu_data();
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_stats(void* p, int* launches, double* device_ms) {
    auto* h = static_cast<host_pipeline*>(p);
    if (launches) *launches = h->net->launches_last_forward();
    if (device_ms) *device_ms = h->net->device_ms_last_forward();
    return EXB_OK;
}

extern "C" int exb_host_pipeline_dump_profile(void* p, const char* path) {
    return static_cast<host_pipeline*>(p)->net->dump_profile(path) ? EXB_OK : EXB_ERR_BAD_ARG;
}

extern "C" int exb_host_pipeline_run_resident(void* p, int iters, double* ms) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline*>(p);
        const double t = h->net->run_resident(iters);
        if (t < 0) {
            g_err = "run_resident needs a previous fused forward";
            return (int)EXB_ERR_BAD_ARG;
        }
        if (ms) *ms = t;
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_trace_size(void* p) { return static_cast<host_pipeline*>(p)->net->trace_size(); }

extern "C" int exb_host_pipeline_trace_entry(void* p, int i, char* name, int cap, double* begin_ms, double* end_ms) {
    std::string n;
    double b = 0, e = 0;
    if (!static_cast<host_pipeline*>(p)->net->trace_entry(i, n, b, e) || cap <= 0) return EXB_ERR_BAD_ARG;
    std::strncpy(name, n.c_str(), cap - 1);
    name[cap - 1] = 0;
    if (begin_ms) *begin_ms = b;
    if (end_ms) *end_ms = e;
    return EXB_OK;
}

extern "C" int exb_host_op_run(const char* type, const char* params, const char* racy_path, int device, int n_in,
                               const float* const* inputs, const int* shapes, float* out, int64_t cap,
                               int* out_shape4) {
    return guarded([&]() {
        set_log_quiet(true);
        CUDA_CHECK(cudaSetDevice(device));
        std::vector<std::string> ins, outs{"out"};
        for (int i = 0; i < n_in; ++i) ins.push_back("in" + std::to_string(i));
        operation_param prm(type, std::string(type) + "_0", n_in, 1, ins, outs, false, false, false, false, device,
                            params ? params : "");
        auto op = operation_reflector<float>::instance().create_object(prm);
        if (racy_path && racy_path[0]) {
            FILE* fp = fopen(racy_path, "rb");
            if (!fp) LOG(FATAL) << "Cannot open " << racy_path;
            op->init_weights(fp);
            fclose(fp);
        } else {
            op->init_weights();
        }
        exb_ctx* ctx = nullptr;
        exb_check(exb_ctx_create(device, &ctx), "exb_ctx_create");
        std::vector<std::shared_ptr<memory::tensor<float>>> bottoms, tops(1);
        for (int i = 0; i < n_in; ++i) {
            std::vector<int> shp(shapes + 4 * i, shapes + 4 * i + 4);
            auto t = std::shared_ptr<memory::tensor<float>>(new memory::tensor<float>(shp, device, memory::NCHW, nullptr));
            t->copy_from(inputs[i], sizeof(float) * (size_t)t->count());
            bottoms.push_back(t);
        }
        op->forward_gpu(ctx, bottoms, tops);
        int rc = exb_ctx_sync_check(ctx, nullptr);
        if (rc == EXB_OK) rc = copy_out(tops[0], out, cap, out_shape4);
        else g_err = exb_last_error_string();
        tops.clear();
        bottoms.clear();
        op.reset();
        exb_ctx_destroy(ctx);
        return rc;
    });
}

// fp32 -> fp16 on the host, round to nearest even (what "host_f16_threads" runs before the copy); needs no GPU.
extern "C" int exb_host_convert_f32_to_f16(const float* src, uint16_t* dst, int64_t n, int threads, int force_scalar) {
    return guarded([&]() {
        if (n < 0 || (n > 0 && (!src || !dst))) {
            g_err = "exb_host_convert_f32_to_f16: bad argument";
            return (int)EXB_ERR_BAD_ARG;
        }
        if (threads > 1 && !force_scalar) {
            glasssix::excalibur::convert_pool pool(threads);
            pool.run(src, dst, (size_t)n);
        } else {
            glasssix::excalibur::convert_f32_to_f16(src, dst, (size_t)n, force_scalar != 0);
        }
        return (int)EXB_OK;
    });
}

// ---- one batch over several GPUs ------------------------------------------------------------------
extern "C" int exb_host_shard_bounds(int total, int world, int rank, int* lo, int* hi) {
    return guarded([&]() {
        if (!lo || !hi) {
            g_err = "exb_host_shard_bounds: null output";
            return (int)EXB_ERR_BAD_ARG;
        }
        shard_bounds(total, world, rank, lo, hi);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_gather_rows(const float* const* parts, const int* part_rows, int n_parts, int64_t row_elems, float* out) {
    if (!parts || !part_rows || !out || n_parts < 0 || row_elems < 0) {
        g_err = "exb_host_gather_rows: bad argument";
        return EXB_ERR_BAD_ARG;
    }
    gather_rows(parts, part_rows, n_parts, row_elems, out);
    return EXB_OK;
}

extern "C" int exb_host_sharded_create(const char* phai_text, const char* racy_path, const int* devices, int n_devices, void** out) {
    return guarded([&]() {
        if (!out || !devices || n_devices < 1) {
            g_err = "exb_host_sharded_create: bad argument";
            return (int)EXB_ERR_BAD_ARG;
        }
        *out = nullptr;
        std::unique_ptr<host_sharded> h(new host_sharded());
        h->net.reset(new sharded_pipeline(split_lines(phai_text), racy_path ? racy_path : "",
                                          std::vector<int>(devices, devices + n_devices)));
        *out = h.release();
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_sharded_destroy(void* p) {
    return guarded([&]() {
        delete static_cast<host_sharded*>(p);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_sharded_set_option(void* p, const char* key, int value) {
    return guarded([&]() {
        auto* h = static_cast<host_sharded*>(p);
        const std::string k = key ? key : "";
        for (int r = 0; r < h->net->replicas(); ++r) {
            pipeline<float>& n = h->net->replica(r);
            if (k == "fusion") n.set_fusion(value != 0);
            else if (k == "cuda_graph") n.set_cuda_graph(value != 0);
            else if (k == "h2d_chunks") n.set_h2d_chunks(value);
            else {
                g_err = "unknown option " + k;
                return (int)EXB_ERR_BAD_ARG;
            }
        }
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_sharded_forward(void* p, const float* input, int N, int C, int H, int W) {
    return guarded([&]() {
        auto* h = static_cast<host_sharded*>(p);
        h->outputs = h->net->forward(input, N, C, H, W);
        h->names = h->net->output_names();
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_sharded_num_outputs(void* p) { return (int)static_cast<host_sharded*>(p)->names.size(); }

extern "C" int exb_host_sharded_output_name(void* p, int i, char* buf, int cap) {
    auto* h = static_cast<host_sharded*>(p);
    if (i < 0 || i >= (int)h->names.size() || cap <= 0) return EXB_ERR_BAD_ARG;
    std::strncpy(buf, h->names[i].c_str(), cap - 1);
    buf[cap - 1] = 0;
    return EXB_OK;
}

extern "C" int exb_host_sharded_get(void* p, const char* name, float* out, int64_t cap, int* shape4) {
    return guarded([&]() {
        auto* h = static_cast<host_sharded*>(p);
        auto it = h->outputs.find(name ? name : "");
        if (it == h->outputs.end()) {
            g_err = std::string("not an output of the last forward: ") + (name ? name : "");
            return (int)EXB_ERR_BAD_ARG;
        }
        return copy_out(it->second, out, cap, shape4);
    });
}

extern "C" int exb_host_sharded_device_ms(void* p, double* ms) {
    if (!p || !ms) return EXB_ERR_BAD_ARG;
    *ms = static_cast<host_sharded*>(p)->net->device_ms_last_forward();
    return EXB_OK;
}

// ---- pipeline<unsigned short>: fp16 tensors at the API edge ----------------------------------------
extern "C" int exb_host_pipeline_f16_create(const char* phai_text, const char* racy_path, int device, void** out) {
    return guarded([&]() {
        if (!out) {
            g_err = "exb_host_pipeline_f16_create: null output";
            return (int)EXB_ERR_BAD_ARG;
        }
        *out = nullptr;
        std::unique_ptr<host_pipeline_f16> h(new host_pipeline_f16());
        h->net.reset(new pipeline<unsigned short>(split_lines(phai_text), racy_path ? racy_path : "", device));
        *out = h.release();
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_f16_destroy(void* p) {
    return guarded([&]() {
        delete static_cast<host_pipeline_f16*>(p);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_f16_set_option(void* p, const char* key, int value) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline_f16*>(p);
        const std::string k = key ? key : "";
        if (k == "fusion") h->net->set_fusion(value != 0);
        else if (k == "cuda_graph") h->net->set_cuda_graph(value != 0);
        else if (k == "h2d_chunks") h->net->set_h2d_chunks(value);
        else {
            g_err = "unknown option " + k;
            return (int)EXB_ERR_BAD_ARG;
        }
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_f16_forward(void* p, const uint16_t* input, int N, int C, int H, int W) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline_f16*>(p);
        auto t = std::shared_ptr<memory::tensor<unsigned short>>(
            new memory::tensor<unsigned short>(std::vector<int>{N, C, H, W}, h->net->device(), memory::NCHW, nullptr));
        t->data()->set_external_cpu_data(const_cast<uint16_t*>(input));
        h->outputs = h->net->forward(t);
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_f16_get(void* p, const char* name, uint16_t* out, int64_t cap, int* shape4) {
    return guarded([&]() {
        auto* h = static_cast<host_pipeline_f16*>(p);
        std::shared_ptr<memory::tensor<unsigned short>> t;
        auto it = h->outputs.find(name ? name : "");
        t = it != h->outputs.end() ? it->second : h->net->get_featmap(name ? name : "");
        if (!t) {
            g_err = "no such feature map (or it was fused away)";
            return (int)EXB_ERR_BAD_ARG;
        }
        if (t->order() == memory::NHWC) {      // op-by-op fp16 tensors are channel-last: hand out NCHW like everything else
            auto c = std::shared_ptr<memory::tensor<unsigned short>>(new memory::tensor<unsigned short>(t->clone()));
            c->convert_order();
            t = c;
        }
        auto shp = t->data_shape();
        for (int i = 0; i < 4; ++i) shape4[i] = shp[i];
        if (!out) return (int)EXB_OK;
        if ((int64_t)t->count() > cap) {
            g_err = "output buffer too small";
            return (int)EXB_ERR_BAD_ARG;
        }
        std::memcpy(out, t->cpu_data(), sizeof(uint16_t) * (size_t)t->count());
        return (int)EXB_OK;
    });
}

extern "C" int exb_host_pipeline_f16_stats(void* p, int* launches, double* device_ms) {
    auto* h = static_cast<host_pipeline_f16*>(p);
    if (launches) *launches = h->net->launches_last_forward();
    if (device_ms) *device_ms = h->net->device_ms_last_forward();
    return EXB_OK;
}

extern "C" int exb_host_write_chrome_trace(const char* path, int n, const char* const* names, const double* begin_ms,
                                           const double* end_ms) {
    return guarded([&]() {
        if (!path || n < 0 || (n > 0 && (!names || !begin_ms || !end_ms))) {
            g_err = "exb_host_write_chrome_trace: bad argument";
            return (int)EXB_ERR_BAD_ARG;
        }
        std::vector<std::string> nm;
        for (int i = 0; i < n; ++i) nm.push_back(names[i] ? names[i] : "");
        if (!write_chrome_trace(path, nm, std::vector<double>(begin_ms, begin_ms + n), std::vector<double>(end_ms, end_ms + n))) {
            g_err = std::string("cannot write ") + path;
            return (int)EXB_ERR_BAD_ARG;
        }
        return (int)EXB_OK;
    });
}
