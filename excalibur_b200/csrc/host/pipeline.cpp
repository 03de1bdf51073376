// pipeline<Dtype>: .phai parser, .racy loader, sequential executor (reference
// src/Excalibur/pipeline.cpp:35-194,234-404,422-451) and, for pipeline<float> on a GPU, the fused
// NHWC plan that is the fast path of this library.
#include "pipeline.hpp"

#include <cuda_fp16.h>

#include <fstream>
#include <functional>
#include <set>

#include "host_convert.hpp"
#include "ops.hpp"

namespace glasssix {
namespace excalibur {

namespace {

int round_up(int a, int b) { return (a + b - 1) / b * b; }

std::vector<std::string> read_lines(std::string_view path) {
    std::ifstream in{std::string(path)};
    if (!in) LOG(FATAL) << "Cannot open " << path;
    std::vector<std::string> lines;
    std::string l;
    while (std::getline(in, l)) {
        while (!l.empty() && (l.back() == '\r' || l.back() == '\n')) l.pop_back();
        lines.push_back(l);
    }
    return lines;
}

struct trace_event {
    std::string name;
    float begin_ms, end_ms;
};

// What the fused plan throws while it is built when the graph needs something only the op-by-op executor
// can do (or nothing can): forward() then runs op by op, where an unimplemented case fails with its own message.
struct plan_refusal : std::runtime_error {
    using std::runtime_error::runtime_error;
};
class refuse_line {
public:
    ~refuse_line() noexcept(false) { throw plan_refusal(os_.str()); }
    std::ostringstream& stream() { return os_; }

private:
    std::ostringstream os_;
};
#define PLAN_REFUSE refuse_line().stream()

// ------------------------------------------------------------------------------------------
// Fused plan (float pipelines on a GPU)
// ------------------------------------------------------------------------------------------
struct dev_buf {
    void* p = nullptr;
    size_t bytes = 0;
    ~dev_buf() { if (p) cudaFree(p); }
    void* ensure(size_t n, int device) {
        if (n > bytes) {
            if (p) cudaFree(p);
            p = nullptr;
            CUDA_CHECK(cudaSetDevice(device));
            CUDA_CHECK(cudaMalloc(&p, n ? n : 16));
            bytes = n;
        }
        return p;
    }
};

struct fmap_info {
    std::string name;
    int root = -1;                 // featmap this one aliases (Split), or itself
    int N = 0, C = 0, H = 0, W = 0;
    int cs = 0;                    // physical channels of the NHWC device forms
    int w_pitch = 0, w_pad = 0;    // physically zero-padded rows (network input feeding a stem conv); 0 = dense
    int f32_pitch = 0;             // floats per image of the fp32 form when it is a padded [N][pitch] matrix; 0 = dense
    bool need_f16 = false, need_i8 = false, need_f32 = false;
    float i8_scale = 0.f;          // multiplier of the int8 form
    std::vector<float> extra_i8_scales;   // further int8 consumers with other scales
    std::shared_ptr<dev_buf> f16, i8, f32;
    std::vector<std::shared_ptr<dev_buf>> extra_i8;
    bool produced = false;
    bool f32_only = false;         // result of a Reshape / Transpose at the tail of the graph: fp32 NCHW only
};

struct plan_step {
    std::string name;
    std::function<void(cudaStream_t)> run;
    int launches = 1;
};

class fused_plan {
public:
    typedef operation<float> op_t;
    fused_plan(const std::vector<operation_param>& params, const std::vector<std::shared_ptr<op_t>>& ops,
               const std::vector<std::string>& inputs, const std::vector<std::string>& outputs, int device)
        : params_(params), ops_(ops), inputs_(inputs), outputs_(outputs), device_(device) {}
    ~fused_plan() {
        if (host_f16_) cudaFreeHost(host_f16_);
        if (graph_exec_) cudaGraphExecDestroy(graph_exec_);
        for (auto e : copied_) cudaEventDestroy(e);
        if (copy_stream_) cudaStreamDestroy(copy_stream_);
        if (stream_) cudaStreamDestroy(stream_);
        if (ev0_) cudaEventDestroy(ev0_);
        if (ev1_) cudaEventDestroy(ev1_);
        if (ctx_) exb_ctx_destroy(ctx_);
    }

    // Why the graph cannot be fused, or "" when it can.
    std::string unsupported_reason() const {
        static const std::set<std::string> ok = {"convolution", "convolutiondepthwise", "pooling", "eltwise", "binaryop",
                                                  "relu", "relu6", "split", "innerproduct", "clip", "sigmoid", "concat", "interp",
                                                 "batchnorm", "hardswish", "input", "yolov5focus", "prelu", "leakyrelu",
                                                 "deconvolution", "reshape", "transpose", "hardsigmoid", "softmax", "flatten"};
        for (const auto& p : params_) {
            std::string t = p.type_;
            std::transform(t.begin(), t.end(), t.begin(), ::tolower);
            if (!ok.count(t)) return "operation type " + p.type_ + " has no fused implementation";
        }
        if (inputs_.size() != 1) return "fused plan needs exactly one input feature map";
        return "";
    }

    void build(int N, int C, int H, int W);
    bool built() const { return built_; }
    bool built_for(int N, int C, int H, int W) const { return built_ && N == N_ && C == C_ && H == H_ && W == W_; }
    void run(const float* host_input, bool use_graph, bool profile, std::vector<trace_event>* trace);
    std::shared_ptr<memory::tensor<float>> fetch(const std::string& name);
    double run_resident(int iters, bool use_graph);
    // forward of k * N_ images: chunk c+1 is copied to the device while chunk c is computed.  host_threads > 0:
    // each chunk is first converted to fp16 on the host by that many threads (half the PCIe bytes), when the
    // plan's ingest step can read fp16 planes; otherwise the fp32 input is copied as it is.
    // host_f16 != nullptr: the caller's input is already fp16 NCHW (pipeline<unsigned short>); it is copied as it is.
    void run_chunked(const float* host_input, int k, bool use_graph, int host_threads = 0, const uint16_t* host_f16 = nullptr);
    bool host_f16_capable() const { return ingest_f16_capable_; }
    int launches() const { return launches_; }
    double device_ms() const { return device_ms_; }
    exb_ctx* ctx() { return ctx_; }

private:
    int fid(const std::string& n) {
        auto it = index_.find(n);
        if (it != index_.end()) return it->second;
        fmap_info f;
        f.name = n;
        f.root = (int)fmaps_.size();
        index_[n] = f.root;
        fmaps_.push_back(f);
        return f.root;
    }
    int root(int f) const {
        while (fmaps_[f].root != f) f = fmaps_[f].root;
        return f;
    }
    static std::string lower_type(const operation_param& p) {
        std::string t = p.type_;
        std::transform(t.begin(), t.end(), t.begin(), ::tolower);
        return t;
    }
    void add_step(const std::string& name, std::function<void(cudaStream_t)> fn, int launches = 1) {
        steps_.push_back({name, fn, launches});
    }
    void* form_f16(fmap_info& f) {
        if (!f.f16) f.f16 = std::make_shared<dev_buf>();
        return f.f16->ensure((size_t)f.N * f.H * (f.w_pitch ? f.w_pitch : f.W) * f.cs * 2, device_);
    }
    void* form_i8(fmap_info& f) {
        if (!f.i8) f.i8 = std::make_shared<dev_buf>();
        return f.i8->ensure((size_t)f.N * f.H * f.W * f.cs, device_);
    }
    void* form_f32(fmap_info& f) {
        if (!f.f32) f.f32 = std::make_shared<dev_buf>();
        return f.f32->ensure((size_t)f.N * (f.f32_pitch ? f.f32_pitch : f.H * f.W * f.C) * 4, device_);
    }
    void set_shape(fmap_info& f, int N, int C, int H, int W) {
        f.N = N; f.C = C; f.H = H; f.W = W;
        f.cs = round_up(C, (f.need_i8 || C > 16) ? 32 : 16);
    }
    // After a producer wrote f's primary forms: emit quantise passes for what it could not fuse.
    void finish_forms(fmap_info& f, bool wrote_i8);
    const void* int8_form_for(fmap_info& f, float scale);

    const std::vector<operation_param>& params_;
    const std::vector<std::shared_ptr<op_t>>& ops_;
    std::vector<std::string> inputs_, outputs_;
    int device_;
    exb_ctx* ctx_ = nullptr;
    cudaStream_t stream_ = nullptr;
    cudaEvent_t ev0_ = nullptr, ev1_ = nullptr;
    cudaGraphExec_t graph_exec_ = nullptr;
    bool built_ = false;
    int N_ = 0, C_ = 0, H_ = 0, W_ = 0;
    std::vector<fmap_info> fmaps_;
    std::unordered_map<std::string, int> index_;
    std::vector<plan_step> steps_;
    dev_buf staging_in_;
    dev_buf norm_in_;                      // normalised fp32 input when the graph starts with an Input op
    dev_buf chunk_stage_;                  // k chunks of fp32 input for run_chunked
    const void* ingest_src_ = nullptr;     // what the ingest step (steps_[0]) reads; never part of the graph
    bool ingest_src_f16_ = false;          // ingest_src_ holds fp16 planes (converted on the host)
    bool ingest_f16_capable_ = false;      // the ingest step has an fp16-source variant
    void* host_f16_ = nullptr;             // pinned staging for the host-converted input
    size_t host_f16_bytes_ = 0;
    std::unique_ptr<convert_pool> pool_;
    cudaStream_t copy_stream_ = nullptr;
    std::vector<cudaEvent_t> copied_;
    void launch_body(bool use_graph);
    int launches_ = 0;
    double device_ms_ = 0.0;
    bool warmed_ = false;

public:
    // results of the last run, by output feature map name
    std::unordered_map<std::string, std::shared_ptr<memory::tensor<float>>> host_out_;
    // results of the last run_chunked (all k * N_ images)
    std::unordered_map<std::string, std::shared_ptr<memory::tensor<float>>> chunk_out_;
};

void fused_plan::finish_forms(fmap_info& f, bool wrote_i8) {
    f.produced = true;
    exb_ctx* ctx = ctx_;
    if (f.need_i8 && !wrote_i8) {
        CHECK(f.need_f16) << "internal: int8 form requested without a source";
        void* src = form_f16(f);
        void* dst = form_i8(f);
        const int64_t count = (int64_t)f.N * f.H * f.W * f.cs;
        const float s = f.i8_scale;
        add_step("quantize " + f.name, [=](cudaStream_t st) {
            exb_check(exb_quantize_fwd(ctx, src, EXB_F16, static_cast<int8_t*>(dst), count, s, 1, st), "exb_quantize_fwd");
        });
    }
    f.extra_i8.clear();
    for (float s : f.extra_i8_scales) {
        auto b = std::make_shared<dev_buf>();
        void* dst = b->ensure((size_t)f.N * f.H * f.W * f.cs, device_);
        f.extra_i8.push_back(b);
        void* src = form_f16(f);
        const int64_t count = (int64_t)f.N * f.H * f.W * f.cs;
        add_step("quantize " + f.name, [=](cudaStream_t st) {
            exb_check(exb_quantize_fwd(ctx, src, EXB_F16, static_cast<int8_t*>(dst), count, s, 1, st), "exb_quantize_fwd");
        });
    }
}

const void* fused_plan::int8_form_for(fmap_info& f, float scale) {
    if (f.i8 && f.i8_scale == scale) return f.i8->p;
    for (size_t i = 0; i < f.extra_i8_scales.size(); ++i)
        if (f.extra_i8_scales[i] == scale) return f.extra_i8[i]->p;
    LOG(FATAL) << "internal: no int8 form of " << f.name << " with scale " << scale;
    return nullptr;
}

void fused_plan::build(int N, int C, int H, int W) {
    CUDA_CHECK(cudaSetDevice(device_));
    if (!ctx_) exb_check(exb_ctx_create(device_, &ctx_), "exb_ctx_create");
    if (!stream_) CUDA_CHECK(cudaStreamCreateWithFlags(&stream_, cudaStreamNonBlocking));
    if (!ev0_) {
        CUDA_CHECK(cudaEventCreate(&ev0_));
        CUDA_CHECK(cudaEventCreate(&ev1_));
    }
    if (graph_exec_) {
        cudaGraphExecDestroy(graph_exec_);
        graph_exec_ = nullptr;
    }
    steps_.clear();
    fmaps_.clear();
    index_.clear();
    warmed_ = false;
    ingest_f16_capable_ = false;
    const size_t n_ops = ops_.size();

    // ---- 1. feature maps, Split aliases, consumers ------------------------------------------
    std::vector<std::vector<int>> in_ids(n_ops), out_ids(n_ops);
    for (size_t i = 0; i < n_ops; ++i) {
        for (const auto& n : params_[i].input_featmaps_) in_ids[i].push_back(fid(n));
        for (const auto& n : params_[i].output_featmaps_) out_ids[i].push_back(fid(n));
    }
    // Split outputs alias their input.  So does an Input (normalisation) op that reads the network
    // input: its arithmetic runs on the fp32 staging buffer in front of the ingest kernel.
    std::vector<char> alias_op(n_ops, 0);
    int input_norm_op = -1;
    for (size_t i = 0; i < n_ops; ++i) {
        const std::string t = lower_type(params_[i]);
        if (t == "split") {
            alias_op[i] = 1;
            for (int o : out_ids[i]) fmaps_[o].root = root(in_ids[i][0]);
        } else if (t == "input" && input_norm_op < 0 && in_ids[i].size() == 1 && out_ids[i].size() == 1 &&
                   root(in_ids[i][0]) == root(fid(inputs_[0]))) {
            alias_op[i] = 1;
            input_norm_op = (int)i;
            fmaps_[out_ids[i][0]].root = root(in_ids[i][0]);
        }
    }
    std::vector<std::vector<int>> consumers(fmaps_.size());   // by root id -> op indices
    for (size_t i = 0; i < n_ops; ++i) {
        if (alias_op[i]) continue;
        for (int f : in_ids[i]) consumers[root(f)].push_back((int)i);
    }
    std::set<int> output_roots;
    for (const auto& n : outputs_) output_roots.insert(root(fid(n)));

    // ---- 2. fusion groups -------------------------------------------------------------------
    struct group {
        int conv = -1;          // leading op
        int residual = -1;      // root featmap added in the epilogue
        int act = EXB_ACT_NONE;
        int pool = -1;          // 3x3/2 max pooling op applied in the conv epilogue
        int bn = -1;            // BatchNorm op folded into the conv's weights and bias
        int slope_op = -1;      // PReLU / LeakyRelu op applied in the epilogue (act == EXB_ACT_PRELU)
        int cat = -1;           // Concat op whose output this group writes its channels into (epilogue stores at a
        int cat_off = 0;        // channel offset instead of a copy kernel); cat_total = channels of that output
        int cat_total = 0;
        int cat_bn = -1;        // BatchNorm behind that Concat, folded slice-wise into the producers
        int out = -1;           // root featmap the group finally produces
        int exec_at = -1;       // index of the last absorbed op
    };
    std::vector<int> absorbed(n_ops, 0);
    std::vector<group> groups(n_ops);
    auto sole_consumer = [&](int f) -> int {
        if (output_roots.count(f)) return -1;
        return consumers[f].size() == 1 ? consumers[f][0] : -1;
    };
    auto act_of_op = [&](int j) -> int {
        const std::string t = lower_type(params_[j]);
        if (t == "relu") return EXB_ACT_RELU;
        if (t == "relu6") return EXB_ACT_RELU6_QUIRK;   // the reference's ReLU6 operation writes 0 above 6
        if (t == "sigmoid") return EXB_ACT_SIGMOID;
        if (t == "clip") {
            auto* c = dynamic_cast<operation_clip<float>*>(ops_[j].get());
            if (c && c->is_relu6()) return EXB_ACT_RELU6;
        }
        if (t == "hardswish") {
            auto* hs = dynamic_cast<operation_hardswish<float>*>(ops_[j].get());
            if (hs && hs->is_standard()) return EXB_ACT_HARDSWISH;
        }
        if (t == "prelu" || t == "leakyrelu") return EXB_ACT_PRELU;     // slopes: slopes_of_op(j, channels)
        return -1;
    };
    // host slopes of a PReLU / LeakyRelu op, one per channel
    auto slopes_of_op = [&](int j, int channels, int first = 0) -> std::vector<float> {
        std::vector<float> sl((size_t)channels);
        if (lower_type(params_[j]) == "leakyrelu") {
            const float a = dynamic_cast<operation_leakyrelu<float>*>(ops_[j].get())->alpha_;
            for (auto& v : sl) v = a;
        } else {
            auto* pr = dynamic_cast<operation_prelu<float>*>(ops_[j].get());
            if (pr->num_slope_ != 1) CHECK_GE(pr->num_slope_, first + channels) << params_[j].name_ << ": slopes do not match the channels";
            for (int c = 0; c < channels; ++c) sl[c] = pr->slopes_cpu()[pr->num_slope_ == 1 ? 0 : first + c];
        }
        return sl;
    };
    auto is_plain_add = [&](int j) -> bool {
        const std::string t = lower_type(params_[j]);
        if (in_ids[j].size() != 2) return false;
        if (t == "binaryop") {
            auto* b = dynamic_cast<operation_binaryop<float>*>(ops_[j].get());
            return b && b->op_type_ == 0 && !b->with_scalar_;
        }
        if (t == "eltwise") {
            auto* e = dynamic_cast<operation_eltwise<float>*>(ops_[j].get());
            return e && e->type_ == 1 && e->coeffs_.size() >= 2 && e->coeffs_[0] == 1.f && e->coeffs_[1] == 1.f;
        }
        return false;
    };
    // x * sigmoid(x) spelled as Sigmoid + BinaryOp(mul) on the two aliases of one feature map
    auto silu_pattern = [&](int f, int* sig, int* mul) -> bool {
        if (output_roots.count(f) || consumers[f].size() != 2) return false;
        for (int a = 0; a < 2; ++a) {
            const int j = consumers[f][a], k = consumers[f][1 - a];
            if (absorbed[j] || absorbed[k] || j == k) continue;
            if (lower_type(params_[j]) != "sigmoid" || lower_type(params_[k]) != "binaryop") continue;
            auto* b = dynamic_cast<operation_binaryop<float>*>(ops_[k].get());
            if (!b || b->op_type_ != 2 || b->with_scalar_ || in_ids[k].size() != 2) continue;
            const int so = root(out_ids[j][0]);
            if (output_roots.count(so) || consumers[so].size() != 1 || consumers[so][0] != k) continue;
            const int a0 = root(in_ids[k][0]), a1 = root(in_ids[k][1]);
            if (!((a0 == so && a1 == f) || (a0 == f && a1 == so))) continue;
            *sig = j;
            *mul = k;
            return true;
        }
        return false;
    };
    for (size_t i = 0; i < n_ops; ++i) {
        const std::string t = lower_type(params_[i]);
        if (absorbed[i] || (t != "convolution" && t != "convolutiondepthwise" && t != "deconvolution")) continue;
        // null for a Deconvolution, which has no built-in activation and takes part in the BatchNorm and
        // activation patterns only
        auto* conv = dynamic_cast<operation_convolution<float>*>(ops_[i].get());
        auto* gconv = dynamic_cast<operation_general_conv<float>*>(ops_[i].get());
        group g;
        g.conv = (int)i;
        g.act = conv ? conv->exb_activation() : EXB_ACT_NONE;
        g.out = root(out_ids[i][0]);
        g.exec_at = (int)i;
        int j, sj = -1, mk = -1;
        // Conv -> BatchNorm: (conv + bias) * b + a is folded into the packed weights; what follows the
        // BatchNorm (activation, residual add) can then be fused as if it followed the conv.
        if (g.act == EXB_ACT_NONE && (j = sole_consumer(g.out)) >= 0 && !absorbed[j] &&
            lower_type(params_[j]) == "batchnorm") {
            auto* bn = dynamic_cast<operation_batchnorm<float>*>(ops_[j].get());
            if (bn && bn->channels_ == gconv->output_channel_) {
                g.bn = j;
                absorbed[j] = 1;
                g.out = root(out_ids[j][0]);
                g.exec_at = j;
            }
        }
        if (g.act == EXB_ACT_NONE && silu_pattern(g.out, &sj, &mk)) {
            g.act = EXB_ACT_SILU;
            absorbed[sj] = absorbed[mk] = 1;
            g.out = root(out_ids[mk][0]);
            g.exec_at = std::max(sj, mk);
        } else if (g.act == EXB_ACT_NONE && (j = sole_consumer(g.out)) >= 0 && !absorbed[j] && act_of_op(j) > 0) {
            g.act = act_of_op(j);
            if (g.act == EXB_ACT_PRELU) g.slope_op = j;
            absorbed[j] = 1;
            g.out = root(out_ids[j][0]);
            g.exec_at = j;
        } else if (t == "convolution" && g.act == EXB_ACT_NONE && (j = sole_consumer(g.out)) >= 0 && !absorbed[j] &&
                   is_plain_add(j)) {
            const int a = root(in_ids[j][0]), b = root(in_ids[j][1]);
            g.residual = a == g.out ? b : a;
            absorbed[j] = 1;
            g.out = root(out_ids[j][0]);
            g.exec_at = j;
            int k;
            if ((k = sole_consumer(g.out)) >= 0 && !absorbed[k] && act_of_op(k) > 0) {
                g.act = act_of_op(k);
                if (g.act == EXB_ACT_PRELU) g.slope_op = k;
                absorbed[k] = 1;
                g.out = root(out_ids[k][0]);
                g.exec_at = k;
            }
        }
        // Stem conv + ReLU followed by the classic 3x3/2 pad-1 max pooling: pooled in the epilogue.
        if (t == "convolution" && g.residual < 0 && (g.act == EXB_ACT_RELU || g.act == EXB_ACT_RELU6) &&
            root(in_ids[i][0]) == root(fid(inputs_[0])) && C <= 4 && !conv->is_int8() && conv->group_ == 1 &&
            conv->in_channels() == C && (j = sole_consumer(g.out)) >= 0 && !absorbed[j] &&
            lower_type(params_[j]) == "pooling" && consumers[root(in_ids[i][0])].size() == 1) {
            auto* pl = dynamic_cast<operation_pooling<float>*>(ops_[j].get());
            const bool classic = pl && pl->type_ == 0 && !pl->global_pooling_ && pl->kernel_size_w_ == 3 &&
                                 pl->kernel_size_h_ == 3 && pl->stride_w_ == 2 && pl->stride_h_ == 2 && pl->pad_left_ == 1 &&
                                 pl->pad_right_ == 1 && pl->pad_top_ == 1 && pl->pad_bottom_ == 1 && pl->pad_mode_ == 1;
            if (classic) {
                exb_conv_desc d = conv->base_desc(N, H, W);
                d.in_dtype = EXB_F16;
                d.out_dtype = EXB_F16;
                d.cin_stride = 4;
                d.x_w_pad = 4;
                d.x_w_pitch = round_up(W + 4 + 8, 8);
                d.act = g.act;
                d.cout_stride = round_up(conv->output_channel_, conv->output_channel_ > 16 ? 32 : 16);
                if (exb_conv2d_pool_fusable(&d) == 1) {
                    g.pool = j;
                    absorbed[j] = 1;
                    g.out = root(out_ids[j][0]);
                    g.exec_at = j;
                }
            }
        }
        groups[i] = g;
    }
    // Concat as the producers' epilogue stores: every input comes from a dense convolution group (no residual,
    // no fused pooling) that nothing else reads and whose channel count is a multiple of 16.  A BatchNorm (+
    // activation) behind such a Concat of activation-free convolutions is folded slice by slice into them
    // (the BottleneckCSP tail: conv, conv -> Concat -> BatchNorm -> LeakyRelu).
    std::vector<int> cat_left(n_ops, 0);      // producers of a direct Concat still to be emitted
    for (size_t k = 0; k < n_ops; ++k) {
        if (absorbed[k] || lower_type(params_[k]) != "concat") continue;
        auto* cc = dynamic_cast<operation_concat<float>*>(ops_[k].get());
        if (!cc || !cc->is_channel_concat() || in_ids[k].size() < 2) continue;
        std::vector<int> prod;
        bool ok = true, plain = true;
        int total = 0;
        for (int f : in_ids[k]) {
            const int rf = root(f);
            int gi = -1;
            for (size_t i = 0; i < k; ++i)
                if (groups[i].conv >= 0 && groups[i].out == rf) gi = (int)i;
            if (gi < 0 || sole_consumer(rf) != (int)k || std::find(prod.begin(), prod.end(), gi) != prod.end()) { ok = false; break; }
            const group& g = groups[gi];
            auto* conv = dynamic_cast<operation_convolution<float>*>(ops_[g.conv].get());
            if (lower_type(params_[g.conv]) != "convolution" || !conv || conv->group_ != 1 || g.residual >= 0 || g.pool >= 0 ||
                g.cat >= 0 || conv->output_channel_ % 16 != 0 || conv->stride_h_ != conv->stride_w_ ||
                (conv->stride_h_ != 1 && conv->stride_h_ != 2)) { ok = false; break; }
            plain = plain && g.act == EXB_ACT_NONE && g.bn < 0;
            prod.push_back(gi);
            total += conv->output_channel_;
        }
        if (!ok) continue;
        int out = root(out_ids[k][0]), bn_op = -1, act = EXB_ACT_NONE, slope_op = -1;
        if (plain) {
            const int j = sole_consumer(out);
            if (j > (int)k && !absorbed[j] && lower_type(params_[j]) == "batchnorm" &&
                dynamic_cast<operation_batchnorm<float>*>(ops_[j].get())->channels_ == total) {
                bn_op = j;
                absorbed[j] = 1;
                out = root(out_ids[j][0]);
                const int a = sole_consumer(out);
                if (a > j && !absorbed[a] && in_ids[a].size() == 1 && act_of_op(a) > 0) {
                    act = act_of_op(a);
                    if (act == EXB_ACT_PRELU) slope_op = a;
                    absorbed[a] = 1;
                    out = root(out_ids[a][0]);
                }
            }
        }
        absorbed[k] = 1;
        int off = 0;
        for (int gi : prod) {
            group& g = groups[gi];
            g.cat = (int)k;
            g.cat_off = off;
            g.cat_total = total;
            g.cat_bn = bn_op;
            if (bn_op >= 0) { g.act = act; g.slope_op = slope_op; }
            g.out = out;
            off += dynamic_cast<operation_convolution<float>*>(ops_[g.conv].get())->output_channel_;
        }
        cat_left[k] = (int)prod.size();
    }
    // Which op index triggers which group (a group runs where its last op stood).
    std::vector<int> run_group_at(n_ops, -1);
    for (size_t i = 0; i < n_ops; ++i)
        if (groups[i].conv >= 0) run_group_at[groups[i].exec_at] = (int)i;

    // ---- 3. forms every feature map must exist in -------------------------------------------
    auto want_i8 = [&](int f, float scale) {
        fmap_info& m = fmaps_[f];
        if (!m.need_i8) {
            m.need_i8 = true;
            m.i8_scale = scale;
        } else if (m.i8_scale != scale &&
                   std::find(m.extra_i8_scales.begin(), m.extra_i8_scales.end(), scale) == m.extra_i8_scales.end()) {
            m.extra_i8_scales.push_back(scale);
            m.need_f16 = true;
        }
    };
    for (size_t i = 0; i < n_ops; ++i) {
        const std::string t = lower_type(params_[i]);
        if (alias_op[i]) continue;
        if (absorbed[i]) {
            // an absorbed add reads its residual operand as fp16
            continue;
        }
        if (t == "convolution") {
            auto* conv = dynamic_cast<operation_convolution<float>*>(ops_[i].get());
            const int f = root(in_ids[i][0]);
            if (conv->is_int8() && conv->group_ == 1) want_i8(f, conv->act_scale());
            else fmaps_[f].need_f16 = true;
            if (groups[i].residual >= 0) fmaps_[groups[i].residual].need_f16 = true;
        } else {
            for (int f : in_ids[i]) fmaps_[root(f)].need_f16 = true;
        }
    }
    for (int f : output_roots) {
        // InnerProduct writes fp32 directly; everything else is converted from fp16.
        fmaps_[f].need_f16 = true;
    }
    for (auto& m : fmaps_)
        if (m.need_i8 && m.extra_i8_scales.size()) m.need_f16 = true;

    // ---- 4. steps in execution order ---------------------------------------------------------
    exb_ctx* ctx = ctx_;
    {
        const int in_id = root(fid(inputs_[0]));
        fmap_info& in = fmaps_[in_id];
        set_shape(in, N, C, H, W);
        ingest_src_ = static_cast<float*>(staging_in_.ensure((size_t)N * C * H * W * 4, device_));
        // A few-channel image that feeds one fp16 convolution is stored as NHWC4 rows with zero
        // padding along W when that lets the tensor-core kernel fold the kw taps into K.
        bool padded = false;
        if (C <= 4 && in.need_f16 && !in.need_i8 && consumers[in_id].size() == 1 &&
            lower_type(params_[consumers[in_id][0]]) == "convolution") {
            auto* conv = dynamic_cast<operation_convolution<float>*>(ops_[consumers[in_id][0]].get());
            if (conv && !conv->is_int8() && conv->group_ == 1 && conv->in_channels() == C) {
                exb_conv_desc d = conv->base_desc(N, H, W);
                d.in_dtype = EXB_F16;
                d.cin_stride = 4;
                d.x_w_pad = 4;
                d.x_w_pitch = round_up(W + 4 + 8, 8);
                if (exb_conv2d_uses_tensor_cores(&d) == 1) {
                    padded = true;
                    in.cs = 4;
                    in.w_pad = d.x_w_pad;
                    in.w_pitch = d.x_w_pitch;
                }
            }
        }
        // Network input -> (Input normalisation ->) YoloV5Focus: one kernel from the fp32 staging buffer to the
        // Focus layer's channel-last fp16 output.
        int focus_op = -1;
        if (C <= 4 && H % 2 == 0 && W % 2 == 0 && !in.need_i8 && consumers[in_id].size() == 1 && !output_roots.count(in_id) &&
            lower_type(params_[consumers[in_id][0]]) == "yolov5focus" && !absorbed[consumers[in_id][0]])
            focus_op = consumers[in_id][0];
        if (focus_op >= 0) {
            const float* mul = nullptr;
            const float* add = nullptr;
            if (input_norm_op >= 0)
                dynamic_cast<operation_input<float>*>(ops_[input_norm_op].get())->coefficients(C, &mul, &add);
            fmap_info& fy = fmaps_[root(out_ids[focus_op][0])];
            fy.need_f16 = true;
            set_shape(fy, N, 4 * C, H / 2, W / 2);
            void* yo = form_f16(fy);
            const int ocs = fy.cs;
            add_step("ingest+focus " + in.name, [=](cudaStream_t st) {
                exb_check(exb_nchw_f32_focus_to_nhwc_f16(ctx, static_cast<const float*>(this->ingest_src_), yo, N, C, H, W, ocs, mul, add, st),
                          "exb_nchw_f32_focus_to_nhwc_f16");
            });
            absorbed[focus_op] = 1;
            in.produced = true;      // consumed inside the fused kernel; it has no device form of its own
            finish_forms(fy, false);
        }
        // Input normalisation: inside the ingest kernel where that kernel has a fused form (few-channel images),
        // else a pass of its own from the fp32 staging buffer to a normalised copy.
        const bool direct_i8 = in.need_i8 && !in.need_f16;
        bool wrote_i8_from_f32 = false;
        void* dst = focus_op >= 0 ? nullptr : (direct_i8 ? form_i8(in) : form_f16(in));
        const int cs = in.cs, w_pad = in.w_pad, w_pitch = in.w_pitch;
        const float s = in.i8_scale;
        const float* nmul = nullptr;
        const float* nadd = nullptr;
        if (focus_op < 0 && input_norm_op >= 0)
            dynamic_cast<operation_input<float>*>(ops_[input_norm_op].get())->coefficients(C, &nmul, &nadd);
        const bool quad = padded && cs == 4 && C <= 3 && W % 4 == 0 && w_pad % 4 == 0 && w_pitch % 4 == 0;
        const bool image = !padded && C <= 4 && (direct_i8 ? (cs == 16 || cs == 32) : (cs == 8 || cs == 16));
        const float* ingest_fixed = nullptr;
        if (nmul && !quad && !image) {
            float* norm = static_cast<float*>(norm_in_.ensure((size_t)N * C * H * W * 4, device_));
            ingest_fixed = norm;
            add_step(params_[input_norm_op].name_, [=](cudaStream_t st) {
                exb_check(exb_channel_affine_fwd(ctx, static_cast<const float*>(this->ingest_src_), norm, nmul, nadd, N, C, 0,
                                                 (int64_t)H * W, EXB_F32, 0, EXB_ACT_NONE, st), "exb_channel_affine_fwd");
            });
        }
        if (focus_op >= 0) {
            // nothing else to ingest
        } else if (padded) {
            ingest_f16_capable_ = quad && !nmul;
            add_step("ingest " + in.name, [=](cudaStream_t st) {
                if (this->ingest_src_f16_)
                    exb_check(exb_nchw_f16_to_nhwc4_padded(ctx, this->ingest_src_, dst, N, C, H, W, w_pad, w_pitch, st),
                              "exb_nchw_f16_to_nhwc4_padded");
                else if (quad && nmul)
                    exb_check(exb_nchw_f32_to_nhwc4_padded_norm(ctx, static_cast<const float*>(this->ingest_src_), dst, N, C, H, W,
                                                                w_pad, w_pitch, nmul, nadd, st),
                              "exb_nchw_f32_to_nhwc4_padded_norm");
                else
                    exb_check(exb_nchw_f32_to_nhwc_padded(ctx, ingest_fixed ? ingest_fixed : static_cast<const float*>(this->ingest_src_),
                                                          dst, EXB_F16, N, C, H, W, cs, w_pad, w_pitch, 1.f, 1, st),
                              "exb_nchw_f32_to_nhwc_padded");
            });
        } else if (image) {
            add_step("ingest " + in.name, [=](cudaStream_t st) {
                exb_check(exb_image_f32_to_nhwc_norm(ctx, static_cast<const float*>(this->ingest_src_), dst, direct_i8 ? EXB_I8 : EXB_F16,
                                                     N, C, H, W, cs, nmul, nadd, direct_i8 ? s : 1.f, 1, st),
                          "exb_image_f32_to_nhwc_norm");
            });
        } else {
            // Both forms of a wide network input: the int8 form is quantised from the fp32 values themselves (as the
            // reference's first int8 convolution does), not from their fp16 rounding.  One step, two launches: the
            // ingest step is the only one that may read `ingest_src_`.
            void* dst8 = (in.need_i8 && in.need_f16) ? form_i8(in) : nullptr;
            wrote_i8_from_f32 = dst8 != nullptr;
            add_step("ingest " + in.name, [=](cudaStream_t st) {
                const float* src = ingest_fixed ? ingest_fixed : static_cast<const float*>(this->ingest_src_);
                exb_check(exb_nchw_f32_to_nhwc(ctx, src, dst, direct_i8 ? EXB_I8 : EXB_F16, N, C, H, W, cs, direct_i8 ? s : 1.f, 1, st),
                          "exb_nchw_f32_to_nhwc");
                if (dst8) exb_check(exb_nchw_f32_to_nhwc(ctx, src, dst8, EXB_I8, N, C, H, W, cs, s, 1, st), "exb_nchw_f32_to_nhwc");
            }, dst8 ? 2 : 1);
        }
        if (focus_op < 0) finish_forms(in, direct_i8 || wrote_i8_from_f32);
    }

    auto run_conv_group = [&](const group& g) {
        const int i = g.conv;
        const std::string t = lower_type(params_[i]);
        fmap_info& x = fmaps_[root(in_ids[i][0])];
        fmap_info& y = fmaps_[g.out];
        CHECK(x.produced) << "feature map " << x.name << " is consumed before it is produced";
        if (x.f32_only)
            PLAN_REFUSE << "(fused plan: " << params_[i].name_ << " reads the result of a Reshape / Transpose; call set_fusion(false))";
        if (t == "convolutiondepthwise") {
            auto* dw = dynamic_cast<operation_convolutiondepthwise<float>*>(ops_[i].get());
            CHECK_EQ(dw->output_channel_, dw->group_);
            CHECK_EQ(x.C, dw->output_channel_);
            exb_dwconv_desc d = dw->dw_desc(x.N, x.H, x.W, x.cs);
            d.act = g.act;
            const int OH = (x.H + d.pad_t + d.pad_b - d.kh) / d.stride_h + 1;
            const int OW = (x.W + d.pad_l + d.pad_r - d.kw) / d.stride_w + 1;
            // A depthwise layer whose result is read only by int8 convolutions at one scale (the projection of an
            // inverted-residual block) quantises in its own store: no fp16 copy of the map, no quantise pass.
            const bool i8_only = y.need_i8 && !y.need_f16 && y.extra_i8_scales.empty();
            if (!i8_only) y.need_f16 = true;
            set_shape(y, x.N, x.C, OH, OW);
            y.cs = x.cs;
            const void* xin = form_f16(x);
            void* yo = i8_only ? form_i8(y) : form_f16(y);
            if (i8_only) {
                d.out_dtype = EXB_I8;
                d.out_scale = y.i8_scale;
            }
            const operation_batchnorm<float>* bn =
                g.bn >= 0 ? dynamic_cast<operation_batchnorm<float>*>(ops_[g.bn].get()) : nullptr;
            exb_dw_weights* w = bn ? dw->dw_packed(ctx, d, bn->mul()->cpu_data(), bn->add()->cpu_data(), bn)
                                   : dw->dw_packed(ctx, d);
            if (g.act == EXB_ACT_PRELU) {
                const std::vector<float> sl = slopes_of_op(g.slope_op, x.C);
                exb_check(exb_dw_weights_set_slopes(ctx, w, sl.data(), (int)sl.size()), "exb_dw_weights_set_slopes");
            }
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_dwconv2d_fwd(ctx, &d, xin, w, yo, st), "exb_dwconv2d_fwd");
            });
            finish_forms(y, i8_only);
            return;
        }
        if (t == "deconvolution") {
            auto* dc = dynamic_cast<operation_deconvolution<float>*>(ops_[i].get());
            if (!dc->supported())
                PLAN_REFUSE << "(Deconvolution " << params_[i].name_
                                << ": implemented for kernel == stride, no padding, no dilation, one group)";
            CHECK_EQ(x.C, dc->in_channels()) << params_[i].name_ << ": input channels do not match the weights";
            const int rh = dc->kernel_size_h_, rw = dc->kernel_size_w_, Cout = dc->output_channel_;
            exb_conv_desc d = dc->inner_desc(x.N, x.H, x.W, x.cs);
            d.act = g.act;       // element-wise, so it commutes with the depth-to-space copy
            d.cout_stride = round_up(d.Cout, d.Cout > 16 ? 32 : 16);
            const void* xin = form_f16(x);
            auto mid = std::make_shared<dev_buf>();
            void* tmp = mid->ensure((size_t)x.N * x.H * x.W * d.cout_stride * 2, device_);
            // a few-channel result that only leaves the network: scattered straight into the fp32 NCHW output
            // instead of a 16-channel-padded fp16 map that an export kernel would read back
            const bool to_output = Cout <= 8 && output_roots.count(g.out) && consumers[g.out].empty() && !y.need_i8;
            if (to_output) {
                const operation_batchnorm<float>* obn =
                    g.bn >= 0 ? dynamic_cast<operation_batchnorm<float>*>(ops_[g.bn].get()) : nullptr;
                exb_conv_weights* ow = obn ? dc->packed(ctx, d, obn->mul()->cpu_data(), obn->add()->cpu_data(), obn) : dc->packed(ctx, d);
                if (g.act == EXB_ACT_PRELU) {
                    const std::vector<float> sl = slopes_of_op(g.slope_op, Cout);
                    std::vector<float> rep((size_t)d.Cout);
                    for (int c = 0; c < d.Cout; ++c) rep[c] = sl[c % Cout];
                    exb_check(exb_conv_weights_set_slopes(ctx, ow, rep.data(), (int)rep.size()), "exb_conv_weights_set_slopes");
                }
                y.f32_only = y.need_f32 = true;
                y.N = x.N; y.C = Cout; y.H = x.H * rh; y.W = x.W * rw; y.cs = Cout;
                float* dst = static_cast<float*>(form_f32(y));
                const int n = x.N, h = x.H, wd = x.W, xs = d.cout_stride;
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    (void)mid;
                    exb_check(exb_conv2d_fwd(ctx, &d, xin, ow, nullptr, tmp, nullptr, st), "exb_conv2d_fwd");
                    exb_check(exb_depth_to_space_nchw_f32(ctx, tmp, dst, n, h, wd, rh, rw, Cout, xs, st),
                              "exb_depth_to_space_nchw_f32");
                }, 2);
                y.produced = true;
                return;
            }
            y.need_f16 = true;
            set_shape(y, x.N, Cout, x.H * rh, x.W * rw);
            void* yo = form_f16(y);
            const operation_batchnorm<float>* bn =
                g.bn >= 0 ? dynamic_cast<operation_batchnorm<float>*>(ops_[g.bn].get()) : nullptr;
            exb_conv_weights* w = bn ? dc->packed(ctx, d, bn->mul()->cpu_data(), bn->add()->cpu_data(), bn) : dc->packed(ctx, d);
            if (g.act == EXB_ACT_PRELU) {       // inner output channel t*Cout + co carries the slope of co
                const std::vector<float> sl = slopes_of_op(g.slope_op, Cout);
                std::vector<float> rep((size_t)d.Cout);
                for (int c = 0; c < d.Cout; ++c) rep[c] = sl[c % Cout];
                exb_check(exb_conv_weights_set_slopes(ctx, w, rep.data(), (int)rep.size()), "exb_conv_weights_set_slopes");
            }
            const int n = x.N, h = x.H, wd = x.W, xs = d.cout_stride, ys = y.cs;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                (void)mid;       // keeps the intermediate tensor alive as long as the step
                exb_check(exb_conv2d_fwd(ctx, &d, xin, w, nullptr, tmp, nullptr, st), "exb_conv2d_fwd");
                exb_check(exb_depth_to_space_fwd(ctx, tmp, yo, n, h, wd, rh, rw, Cout, xs, ys, EXB_F16, st),
                          "exb_depth_to_space_fwd");
            }, 2);
            finish_forms(y, false);
            return;
        }
        auto* conv = dynamic_cast<operation_convolution<float>*>(ops_[i].get());
        CHECK_EQ(x.C, conv->in_channels()) << params_[i].name_ << ": input channels do not match the weights";
        const bool int8 = conv->is_int8() && conv->group_ == 1;
        exb_conv_desc d = conv->base_desc(x.N, x.H, x.W);
        d.in_dtype = int8 ? EXB_I8 : EXB_F16;
        d.cin_stride = conv->group_ == 1 ? x.cs : x.C;
        d.x_w_pitch = x.w_pitch;
        d.x_w_pad = x.w_pad;
        d.act = g.act;
        d.fuse_pool = g.pool >= 0 ? 1 : 0;
        int OH, OW;
        exb_check(exb_conv_out_dims(&d, &OH, &OW), "exb_conv_out_dims");
        if (g.cat >= 0) {
            // this group's channels are a slice of a Concat's output: stored there by the epilogue
            const int Cout = conv->output_channel_;
            if (y.N == 0) {
                y.need_f16 = true;
                set_shape(y, x.N, g.cat_total, OH, OW);
                void* whole = form_f16(y);
                // the padding channels are never written afterwards and must stay finite
                if (y.cs > g.cat_total) CUDA_CHECK(cudaMemset(whole, 0, (size_t)y.N * y.H * y.W * y.cs * 2));
            } else if (y.N != x.N || y.H != OH || y.W != OW) {
                PLAN_REFUSE << "(Concat " << params_[g.cat].name_ << ": operands differ in shape)";
            }
            d.out_dtype = EXB_F16;
            d.cout_stride = Cout;
            d.y_pitch = y.cs;
            const void* xin = int8 ? int8_form_for(x, conv->act_scale()) : form_f16(x);
            void* y1 = static_cast<char*>(form_f16(y)) + (size_t)g.cat_off * 2;
            exb_conv_weights* w = nullptr;
            if (g.cat_bn >= 0) {
                auto* cbn = dynamic_cast<operation_batchnorm<float>*>(ops_[g.cat_bn].get());
                const float* m = cbn->mul()->cpu_data() + g.cat_off;
                w = conv->packed(ctx, d, m, cbn->add()->cpu_data() + g.cat_off, m);
            } else {
                const operation_batchnorm<float>* own = g.bn >= 0 ? dynamic_cast<operation_batchnorm<float>*>(ops_[g.bn].get()) : nullptr;
                w = own ? conv->packed(ctx, d, own->mul()->cpu_data(), own->add()->cpu_data(), own) : conv->packed(ctx, d);
            }
            if (g.act == EXB_ACT_PRELU) {
                // slopes of an activation behind the Concat are indexed by the Concat's channels
                const std::vector<float> sl = slopes_of_op(g.slope_op, Cout, g.cat_bn >= 0 ? g.cat_off : 0);
                exb_check(exb_conv_weights_set_slopes(ctx, w, sl.data(), (int)sl.size()), "exb_conv_weights_set_slopes");
            }
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_conv2d_fwd(ctx, &d, xin, w, nullptr, y1, nullptr, st), "exb_conv2d_fwd");
            });
            if (--cat_left[g.cat] == 0) finish_forms(y, false);
            return;
        }
        set_shape(y, x.N, conv->output_channel_, OH, OW);
        if (conv->group_ != 1) CHECK_EQ(x.cs, x.C) << "grouped convolution needs unpadded channels";
        d.cout_stride = y.cs;
        const void* xin = int8 ? int8_form_for(x, conv->act_scale()) : form_f16(x);
        const void* res = nullptr;
        if (g.residual >= 0) {
            fmap_info& r = fmaps_[g.residual];
            CHECK(r.produced) << "residual " << r.name << " is not available when " << params_[i].name_ << " runs";
            CHECK(r.N == y.N && r.C == y.C && r.H == y.H && r.W == y.W && r.cs == y.cs) << "residual shape mismatch";
            res = form_f16(r);
            d.res_dtype = EXB_F16;
        }
        void* y1 = nullptr;
        void* y2 = nullptr;
        bool wrote_i8 = false;
        if (y.need_f16 || !y.need_i8) {
            y.need_f16 = true;
            d.out_dtype = EXB_F16;
            y1 = form_f16(y);
            if (y.need_i8) {
                d.out2_dtype = EXB_I8;
                d.out2_scale = y.i8_scale;
                y2 = form_i8(y);
                wrote_i8 = true;
            }
        } else {
            d.out_dtype = EXB_I8;
            d.out_scale = y.i8_scale;
            y1 = form_i8(y);
            wrote_i8 = true;
        }
        const operation_batchnorm<float>* bn =
            g.bn >= 0 ? dynamic_cast<operation_batchnorm<float>*>(ops_[g.bn].get()) : nullptr;
        exb_conv_weights* w = bn ? conv->packed(ctx, d, bn->mul()->cpu_data(), bn->add()->cpu_data(), bn)
                                 : conv->packed(ctx, d);
        if (g.act == EXB_ACT_PRELU) {
            const std::vector<float> sl = slopes_of_op(g.slope_op, conv->output_channel_);
            exb_check(exb_conv_weights_set_slopes(ctx, w, sl.data(), (int)sl.size()), "exb_conv_weights_set_slopes");
        }
        add_step(params_[i].name_, [=](cudaStream_t st) {
            exb_check(exb_conv2d_fwd(ctx, &d, xin, w, res, y1, y2, st), "exb_conv2d_fwd");
        });
        finish_forms(y, wrote_i8);
    };

    for (size_t i = 0; i < n_ops; ++i) {
        const std::string t = lower_type(params_[i]);
        if (run_group_at[i] >= 0) {
            run_conv_group(groups[run_group_at[i]]);
            continue;
        }
        if (absorbed[i] || alias_op[i] || t == "convolution" || t == "convolutiondepthwise" || t == "deconvolution") continue;
        fmap_info& x = fmaps_[root(in_ids[i][0])];
        fmap_info& y = fmaps_[root(out_ids[i][0])];
        CHECK(x.produced) << "feature map " << x.name << " is consumed before it is produced";
        bool plain_copy = false;
        if (t == "reshape" && !x.f32_only && !x.need_f32)
            plain_copy = dynamic_cast<operation_reshape<float>*>(ops_[i].get())->out_shape({x.N, x.C, x.H, x.W}) ==
                         std::vector<int>{x.N, x.C, x.H, x.W};
        if (t == "flatten" && !x.f32_only && !x.need_f32 && x.H == 1 && x.W == 1) {
            // a feature vector on its way into InnerProducts, which read it as C values whatever its shape says
            const int fy = root(out_ids[i][0]);
            plain_copy = !output_roots.count(fy) && !consumers[fy].empty();
            for (int cj : consumers[fy]) plain_copy = plain_copy && lower_type(params_[cj]) == "innerproduct";
        }
        if (plain_copy) {
            // a Reshape that changes nothing (the (N,C,1,1) vectors around the InnerProducts of a gate): a copy
            y.need_f16 = true;
            set_shape(y, x.N, x.C, x.H, x.W);
            y.cs = x.cs;
            const void* src = form_f16(x);
            void* dst = form_f16(y);
            const size_t bytes = (size_t)x.N * x.H * x.W * x.cs * 2;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                CUDA_CHECK(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, st));
            });
            finish_forms(y, false);
            continue;
        }
        if (t == "reshape" && !x.f32_only && !x.need_f32) {
            // detection head: (N, A*K, H, W) -> Reshape (N, A, K, H*W) -> Transpose of the last two axes, read by
            // nothing else: one gather from the channel-last fp16 map straight into the fp32 result
            const std::vector<int> shp = dynamic_cast<operation_reshape<float>*>(ops_[i].get())->out_shape({x.N, x.C, x.H, x.W});
            const int ry = root(out_ids[i][0]);
            const int j = sole_consumer(ry);
            auto* tr2 = j > (int)i && !absorbed[j] && lower_type(params_[j]) == "transpose"
                            ? dynamic_cast<operation_transpose<float>*>(ops_[j].get()) : nullptr;
            if (tr2 && tr2->is_swap_hw() && shp[0] == x.N && shp[1] * shp[2] == x.C && shp[3] == x.H * x.W) {
                fmap_info& out = fmaps_[root(out_ids[j][0])];
                out.f32_only = out.need_f32 = out.produced = true;
                out.N = x.N; out.C = shp[1]; out.H = shp[3]; out.W = shp[2]; out.cs = out.C;
                const void* h16 = form_f16(x);
                float* dst = static_cast<float*>(form_f32(out));
                const int n = x.N, P = shp[3], cs = x.cs, A = shp[1], K = shp[2];
                add_step(params_[i].name_ + "+" + params_[j].name_, [=](cudaStream_t st) {
                    exb_check(exb_nhwc_f16_split_heads_f32(ctx, h16, dst, n, P, cs, A, K, st), "exb_nhwc_f16_split_heads_f32");
                });
                absorbed[j] = 1;
                continue;
            }
        }
        if (t == "reshape" || t == "transpose" || t == "flatten" || t == "softmax") {
            // Shape surgery is defined on NCHW data: it runs on the fp32 NCHW copy of the tensor, and what it
            // produces exists in that form only (the graph's tail: detection heads).
            float* src = static_cast<float*>(form_f32(x));
            if (!x.f32_only) {
                const void* h16 = form_f16(x);
                const int n = x.N, c = x.C, h = x.H, w = x.W, cs = x.cs;
                add_step("emit " + x.name, [=](cudaStream_t st) {
                    exb_check(exb_nhwc_to_nchw_f32(ctx, h16, EXB_F16, src, n, c, h, w, cs, 1.f, st), "exb_nhwc_to_nchw_f32");
                });
            }
            y.f32_only = y.need_f32 = y.produced = true;
            auto* tr = t == "transpose" ? dynamic_cast<operation_transpose<float>*>(ops_[i].get()) : nullptr;
            if (t == "reshape" || t == "flatten") {
                const std::vector<int> in_shape{x.N, x.C, x.H, x.W};
                const std::vector<int> shp = t == "reshape" ? dynamic_cast<operation_reshape<float>*>(ops_[i].get())->out_shape(in_shape)
                                                            : dynamic_cast<operation_flatten<float>*>(ops_[i].get())->out_shape(in_shape);
                y.N = shp[0]; y.C = shp[1]; y.H = shp[2]; y.W = shp[3]; y.cs = y.C;
                y.f32 = x.f32;       // same bytes, new shape
            } else if (t == "softmax") {
                if (dynamic_cast<operation_softmax<float>*>(ops_[i].get())->axis_ != 0) PLAN_REFUSE << "(Softmax is implemented over the channel axis, key 0=0)";
                y.N = x.N; y.C = x.C; y.H = x.H; y.W = x.W; y.cs = y.C;
                float* dst = static_cast<float*>(form_f32(y));
                const int n = x.N, c = x.C;
                const int64_t inner = (int64_t)x.H * x.W;
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_softmax_channels_f32(ctx, src, dst, n, c, inner, 0, st), "exb_softmax_channels_f32");
                });
            } else if (tr->is_identity()) {
                y.N = x.N; y.C = x.C; y.H = x.H; y.W = x.W; y.cs = y.C;
                y.f32 = x.f32;
            } else {
                if (!tr->is_swap_hw()) PLAN_REFUSE << "(Transpose is implemented for the permutations 0,1,2 and 1,0,2)";
                y.N = x.N; y.C = x.C; y.H = x.W; y.W = x.H; y.cs = y.C;
                float* dst = static_cast<float*>(form_f32(y));
                const int64_t planes = (int64_t)x.N * x.C;
                const int h = x.H, w = x.W;
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_transpose_hw_f32(ctx, src, dst, planes, h, w, st), "exb_transpose_hw_f32");
                });
            }
            continue;
        }
        for (int f : in_ids[i])
            if (fmaps_[root(f)].f32_only)
                PLAN_REFUSE << "(fused plan: " << params_[i].type_ << " " << params_[i].name_
                                << " reads the result of a Reshape / Transpose; call set_fusion(false))";
        if (t == "pooling") {
            auto* pool = dynamic_cast<operation_pooling<float>*>(ops_[i].get());
            exb_pool_desc d = pool->desc(x.N, x.H, x.W, x.C, x.cs, EXB_F16);
            int PH, PW;
            exb_check(exb_pool_out_dims(&d, &PH, &PW), "exb_pool_out_dims");
            y.need_f16 = true;
            set_shape(y, x.N, x.C, PH, PW);
            y.cs = x.cs;
            const void* xin = form_f16(x);
            // SPP: a stride-1 "same" max pooling of window k is the window-5 pooling of the window-(k-4) pooling of
            // the same map (clipped windows compose exactly), 25 loads per output instead of k*k
            auto same_max = [](const exb_pool_desc& q, int k) {
                return q.type == 0 && !q.global_pool && q.kh == k && q.kw == k && q.stride_h == 1 && q.stride_w == 1 &&
                       q.pad_t == k / 2 && q.pad_b == k / 2 && q.pad_l == k / 2 && q.pad_r == k / 2;
            };
            if (d.kh >= 9 && (d.kh & 1) && same_max(d, d.kh)) {
                for (size_t j = 0; j < i; ++j) {
                    if (lower_type(params_[j]) != "pooling" || absorbed[j] || root(in_ids[j][0]) != root(in_ids[i][0])) continue;
                    auto* pj = dynamic_cast<operation_pooling<float>*>(ops_[j].get());
                    const exb_pool_desc dj = pj->desc(x.N, x.H, x.W, x.C, x.cs, EXB_F16);
                    fmap_info& yj = fmaps_[root(out_ids[j][0])];
                    if (!same_max(dj, d.kh - 4) || !yj.produced || !yj.f16) continue;
                    xin = form_f16(yj);
                    d.kh = d.kw = 5;
                    d.pad_t = d.pad_b = d.pad_l = d.pad_r = 2;
                    break;
                }
            }
            void* y1 = form_f16(y);
            void* y2 = nullptr;
            const bool fuse_q = y.need_i8 && d.type == 0;   // max commutes with the monotone quantiser
            if (fuse_q) {
                d.out2_dtype = EXB_I8;
                d.out2_scale = y.i8_scale;
                y2 = form_i8(y);
            }
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_pool2d_fwd(ctx, &d, xin, y1, y2, st), "exb_pool2d_fwd");
            });
            finish_forms(y, fuse_q);
        } else if (t == "innerproduct") {
            auto* fc = dynamic_cast<operation_innerproduct<float>*>(ops_[i].get());
            if (x.H != 1 || x.W != 1) PLAN_REFUSE << "(fused InnerProduct needs a 1x1 input map; call set_fusion(false))";
            CHECK_EQ(x.C, fc->in_features());
            exb_conv_desc d = fc->fc_desc(x.N, x.cs);
            const int fy = root(out_ids[i][0]);
            if (!output_roots.count(fy)) {
                // feeds other operations (the bottleneck of a gate): an fp16 (N,C,1,1) map like any other
                y.need_f16 = true;
                set_shape(y, x.N, fc->num_output_, 1, 1);
                d.out_dtype = EXB_F16;
                d.cout_stride = y.cs;
                const void* xin = form_f16(x);
                void* yo = form_f16(y);
                exb_conv_weights* w = fc->packed(ctx, d);
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_conv2d_fwd(ctx, &d, xin, w, nullptr, yo, nullptr, st), "exb_conv2d_fwd");
                });
                finish_forms(y, false);
                continue;
            }
            y.N = x.N; y.C = fc->num_output_; y.H = 1; y.W = 1; y.cs = y.C;
            y.need_f32 = true;
            // rows padded to 16 floats so the conv epilogue keeps its vector stores; the pad is dropped by the
            // pitched device-to-host copy
            y.f32_pitch = round_up(y.C, 16);
            d.cout_stride = y.f32_pitch;
            const void* xin = form_f16(x);
            void* yo = form_f32(y);
            exb_conv_weights* w = fc->packed(ctx, d);
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_conv2d_fwd(ctx, &d, xin, w, nullptr, yo, nullptr, st), "exb_conv2d_fwd");
            });
            y.produced = true;
            if (!output_roots.count(root(out_ids[i][0])) || consumers[root(out_ids[i][0])].size())
                PLAN_REFUSE << "(fused plan: InnerProduct must be a pipeline output)";
        } else if (t == "concat") {
            auto* cc = dynamic_cast<operation_concat<float>*>(ops_[i].get());
            if (!cc->is_channel_concat()) PLAN_REFUSE << "(Concat is implemented along the channel axis, key 0=-1)";
            auto xs = std::make_shared<std::vector<const void*>>();
            auto widths = std::make_shared<std::vector<int64_t>>();
            auto strides = std::make_shared<std::vector<int64_t>>();
            int ctot = 0;
            for (size_t k = 0; k < in_ids[i].size(); ++k) {
                fmap_info& xi = fmaps_[root(in_ids[i][k])];
                CHECK(xi.produced && xi.N == x.N && xi.H == x.H && xi.W == x.W) << "Concat operands differ in shape";
                xs->push_back(form_f16(xi));
                widths->push_back(xi.C);
                strides->push_back(xi.cs);
                ctot += xi.C;
            }
            y.need_f16 = true;
            set_shape(y, x.N, ctot, x.H, x.W);
            void* yo = form_f16(y);
            const int64_t rows = (int64_t)y.N * y.H * y.W;
            const int64_t ys = y.cs;
            // the padding channels are never written afterwards and must stay finite
            CUDA_CHECK(cudaMemset(yo, 0, (size_t)rows * ys * 2));
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_concat_fwd(ctx, (int)xs->size(), xs->data(), widths->data(), strides->data(), yo, ys, rows,
                                         EXB_F16, st), "exb_concat_fwd");
            });
            finish_forms(y, false);
        } else if (t == "interp") {
            auto* ip = dynamic_cast<operation_interp<float>*>(ops_[i].get());
            if (in_ids[i].size() != 1) PLAN_REFUSE << "(Interp with a size tensor as second input)";
            if (ip->resize_type_ != 1 || ip->align_corner_ != 0)
                PLAN_REFUSE << "(Interp is implemented for nearest mode, keys 0=1 6=0)";
            int OH = 0, OW = 0;
            ip->out_dims(x.H, x.W, &OH, &OW);
            y.need_f16 = true;
            set_shape(y, x.N, x.C, OH, OW);
            y.cs = x.cs;
            const void* xin = form_f16(x);
            void* yo = form_f16(y);
            const int n = x.N, h = x.H, w = x.W, c = x.C, cs = x.cs;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_interp_nearest_fwd(ctx, xin, yo, n, h, w, c, cs, OH, OW, EXB_F16, 1, st), "exb_interp_nearest_fwd");
            });
            finish_forms(y, false);
        } else if (t == "yolov5focus") {
            y.need_f16 = true;
            set_shape(y, x.N, 4 * x.C, x.H / 2, x.W / 2);
            const void* xin = form_f16(x);
            void* yo = form_f16(y);
            const int n = x.N, c = x.C, h = x.H, w = x.W, ics = x.cs, ocs = y.cs;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_focus_fwd(ctx, xin, yo, n, c, h, w, ics, ocs, EXB_F16, 1, st), "exb_focus_fwd");
            });
            finish_forms(y, false);
        } else if (t == "input") {
            // an Input op that is not at the network input: per-channel affine on the fp16 form
            auto* inp = dynamic_cast<operation_input<float>*>(ops_[i].get());
            y.need_f16 = true;
            set_shape(y, x.N, x.C, x.H, x.W);
            y.cs = x.cs;
            const void* xin = form_f16(x);
            void* yo = form_f16(y);
            const float* mul = nullptr;
            const float* add = nullptr;
            inp->coefficients(x.C, &mul, &add);
            const int64_t rows = (int64_t)x.N * x.H * x.W;
            const int c = x.C, cs = x.cs;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_channel_affine_fwd(ctx, xin, yo, mul, add, rows, c, cs, 1, EXB_F16, 1, EXB_ACT_NONE, st),
                          "exb_channel_affine_fwd");
            });
            finish_forms(y, false);
        } else if (t == "batchnorm") {
            auto* bn = dynamic_cast<operation_batchnorm<float>*>(ops_[i].get());
            CHECK_EQ(x.C, bn->channels_);
            // a PReLU / LeakyRelu / plain activation that alone reads the result runs in the same pass
            fmap_info* yy = &y;
            int act = EXB_ACT_NONE;
            const float* slope = nullptr;
            int n_slope = 0;
            const int j = sole_consumer(root(out_ids[i][0]));
            if (j > (int)i && !absorbed[j] && in_ids[j].size() == 1 && act_of_op(j) > 0) {
                const std::string tj = lower_type(params_[j]);
                if (tj == "prelu") {
                    auto* pr = dynamic_cast<operation_prelu<float>*>(ops_[j].get());
                    if (pr->num_slope_ != 1) CHECK_EQ(pr->num_slope_, x.C) << params_[j].name_ << ": slopes do not match the channels";
                    slope = pr->slopes_gpu();
                    n_slope = pr->num_slope_;
                } else if (tj == "leakyrelu") {
                    slope = dynamic_cast<operation_leakyrelu<float>*>(ops_[j].get())->slope_gpu();
                    n_slope = 1;
                } else {
                    act = act_of_op(j);
                }
                absorbed[j] = 1;
                yy = &fmaps_[root(out_ids[j][0])];
            }
            yy->need_f16 = true;
            set_shape(*yy, x.N, x.C, x.H, x.W);
            yy->cs = x.cs;
            const void* xin = form_f16(x);
            void* yo = form_f16(*yy);
            const float* mul = bn->mul()->gpu_data();
            const float* add = bn->add()->gpu_data();
            const int64_t rows = (int64_t)x.N * x.H * x.W;
            const int c = x.C, cs = x.cs;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                if (slope)
                    exb_check(exb_channel_affine_prelu_fwd(ctx, xin, yo, mul, add, slope, n_slope, rows, c, cs, 1, EXB_F16, 1, st),
                              "exb_channel_affine_prelu_fwd");
                else
                    exb_check(exb_channel_affine_fwd(ctx, xin, yo, mul, add, rows, c, cs, 1, EXB_F16, 1, act, st),
                              "exb_channel_affine_fwd");
            });
            finish_forms(*yy, false);
        } else if (t == "binaryop" && in_ids[i].size() == 2 &&
                   !dynamic_cast<operation_binaryop<float>*>(ops_[i].get())->with_scalar_ &&
                   (fmaps_[root(in_ids[i][1])].H != x.H || fmaps_[root(in_ids[i][1])].W != x.W)) {
            // (N,C,H,W) with (N,C,1,1) in either order: a per-channel gate
            fmap_info& o = fmaps_[root(in_ids[i][1])];
            fmap_info& big = (int64_t)x.H * x.W >= (int64_t)o.H * o.W ? x : o;
            fmap_info& sm = &big == &x ? o : x;
            if (!(sm.produced && big.produced && sm.H == 1 && sm.W == 1 && sm.C == big.C && sm.N == big.N && sm.cs == big.cs && !sm.f32_only))
                PLAN_REFUSE << "BinaryOp " << params_[i].name_ << ": operands differ in shape";
            y.need_f16 = true;
            set_shape(y, big.N, big.C, big.H, big.W);
            y.cs = big.cs;
            const void* a = form_f16(big);
            const void* g8 = form_f16(sm);
            void* yo = form_f16(y);
            const int op = dynamic_cast<operation_binaryop<float>*>(ops_[i].get())->op_type_;
            const int n = big.N, c = big.C, cs = big.cs, small_first = &big == &x ? 0 : 1;
            const int64_t inner = (int64_t)big.H * big.W;
            add_step(params_[i].name_, [=](cudaStream_t st) {
                exb_check(exb_binaryop_channel_bcast_fwd(ctx, op, a, g8, small_first, yo, n, n, c, cs, inner, EXB_F16, 1, st),
                          "exb_binaryop_channel_bcast_fwd");
            });
            finish_forms(y, false);
        } else {
            // element-wise ops on the fp16 form
            y.need_f16 = true;
            set_shape(y, x.N, x.C, x.H, x.W);
            y.cs = x.cs;
            const int64_t count = (int64_t)x.N * x.H * x.W * x.cs;
            void* yo = form_f16(y);
            if (t == "hardswish" && act_of_op((int)i) < 0) {
                auto* hs = dynamic_cast<operation_hardswish<float>*>(ops_[i].get());
                const float alpha = hs->alpha_, beta = hs->beta_;
                const void* xin = form_f16(x);
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_hardswish_fwd(ctx, xin, yo, count, EXB_F16, alpha, beta, st), "exb_hardswish_fwd");
                });
            } else if (t == "hardsigmoid") {
                auto* hs = dynamic_cast<operation_hardsigmoid<float>*>(ops_[i].get());
                const float alpha = hs->alpha_, beta = hs->beta_;
                const void* xin = form_f16(x);
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_hardsigmoid_fwd(ctx, xin, yo, count, EXB_F16, alpha, beta, st), "exb_hardsigmoid_fwd");
                });
            } else if (t == "prelu" || t == "leakyrelu") {
                const float* slope = nullptr;
                int n_slope = 1;
                if (t == "prelu") {
                    auto* pr = dynamic_cast<operation_prelu<float>*>(ops_[i].get());
                    if (pr->num_slope_ != 1) CHECK_EQ(pr->num_slope_, x.C) << params_[i].name_ << ": slopes do not match the channels";
                    slope = pr->slopes_gpu();
                    n_slope = pr->num_slope_;
                } else {
                    slope = dynamic_cast<operation_leakyrelu<float>*>(ops_[i].get())->slope_gpu();
                }
                const void* xin = form_f16(x);
                const int64_t rows = (int64_t)x.N * x.H * x.W;
                const int c = x.C, cs = x.cs;
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_prelu_fwd(ctx, xin, yo, slope, n_slope, rows, c, cs, 1, EXB_F16, 1, st), "exb_prelu_fwd");
                });
            } else if (t == "relu" || t == "relu6" || t == "clip" || t == "sigmoid" || t == "hardswish") {
                const int act = act_of_op((int)i);
                if (act < 0) PLAN_REFUSE << "(" << params_[i].type_ << " parameters)";
                const void* xin = form_f16(x);
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_activation_fwd(ctx, act, xin, yo, count, EXB_F16, st), "exb_activation_fwd");
                });
            } else if (t == "binaryop") {
                auto* b = dynamic_cast<operation_binaryop<float>*>(ops_[i].get());
                const void* a = form_f16(x);
                const int op = b->op_type_;
                if (b->with_scalar_) {
                    const float s = b->coef_;
                    add_step(params_[i].name_, [=](cudaStream_t st) {
                        exb_check(exb_binaryop_scalar_fwd(ctx, op, a, s, yo, count, EXB_F16, st), "exb_binaryop_scalar_fwd");
                    });
                } else {
                    fmap_info& x2 = fmaps_[root(in_ids[i][1])];
                    if (!(x2.produced && x2.N == x.N && x2.C == x.C && x2.H == x.H && x2.W == x.W)) PLAN_REFUSE << "BinaryOp " << params_[i].name_ << ": operands differ in shape";
                    const void* bb = form_f16(x2);
                    add_step(params_[i].name_, [=](cudaStream_t st) {
                        exb_check(exb_binaryop_fwd(ctx, op, a, bb, yo, count, EXB_F16, st), "exb_binaryop_fwd");
                    });
                }
            } else if (t == "eltwise") {
                auto* e = dynamic_cast<operation_eltwise<float>*>(ops_[i].get());
                auto xs = std::make_shared<std::vector<const void*>>();
                auto cf = std::make_shared<std::vector<float>>();
                for (size_t k = 0; k < in_ids[i].size(); ++k) {
                    fmap_info& xi = fmaps_[root(in_ids[i][k])];
                    CHECK(xi.produced && xi.C == x.C && xi.H == x.H && xi.W == x.W) << "Eltwise operands differ in shape";
                    xs->push_back(form_f16(xi));
                    cf->push_back(k < e->coeffs_.size() ? e->coeffs_[k] : 1.f);
                }
                const int type = e->type_;
                add_step(params_[i].name_, [=](cudaStream_t st) {
                    exb_check(exb_eltwise_fwd(ctx, type, (int)xs->size(), xs->data(), cf->data(), yo, count, EXB_F16, st),
                              "exb_eltwise_fwd");
                });
            } else {
                LOG(FATAL) << "fused plan: unexpected operation type " << params_[i].type_;
            }
            finish_forms(y, false);
        }
    }

    // ---- 5. outputs: fp32 NCHW on the device, then one D2H each -------------------------------
    host_out_.clear();
    for (const auto& name : outputs_) {
        fmap_info& f = fmaps_[root(fid(name))];
        CHECK(f.produced) << "output " << name << " is never produced";
        auto t = std::shared_ptr<memory::tensor<float>>(
            new memory::tensor<float>(std::vector<int>{f.N, f.C, f.H, f.W}, device_, memory::NCHW, nullptr));
        host_out_[name] = t;
        if (f.need_f32 && f.f32 && f.H == 1 && f.W == 1 && !f.f32_only) continue;   // already fp32 [N][C]
        if (f.f32_only) continue;                                    // Reshape / Transpose results are fp32 NCHW already
        const void* src = form_f16(f);
        float* dst = static_cast<float*>(form_f32(f));
        const int n = f.N, c = f.C, h = f.H, w = f.W, cs = f.cs;
        add_step("emit " + name, [=](cudaStream_t st) {
            exb_check(exb_nhwc_to_nchw_f32(ctx, src, EXB_F16, dst, n, c, h, w, cs, 1.f, st), "exb_nhwc_to_nchw_f32");
        });
    }
    N_ = N; C_ = C; H_ = H; W_ = W;
    built_ = true;
}

void fused_plan::run(const float* host_input, bool use_graph, bool profile, std::vector<trace_event>* trace) {
    CUDA_CHECK(cudaSetDevice(device_));
    const size_t in_bytes = (size_t)N_ * C_ * H_ * W_ * 4;
    CUDA_CHECK(cudaMemcpyAsync(staging_in_.p, host_input, in_bytes, cudaMemcpyHostToDevice, stream_));
    ingest_src_ = staging_in_.p;
    ingest_src_f16_ = false;
    launches_ = 0;
    for (auto& s : steps_) launches_ += s.launches;
    if (profile) {
        // per-step device times; never replayed from the graph so every step can be bracketed
        std::vector<cudaEvent_t> evs(steps_.size() + 1);
        for (auto& e : evs) CUDA_CHECK(cudaEventCreate(&e));
        CUDA_CHECK(cudaEventRecord(evs[0], stream_));
        for (size_t i = 0; i < steps_.size(); ++i) {
            steps_[i].run(stream_);
            CUDA_CHECK(cudaEventRecord(evs[i + 1], stream_));
        }
        CUDA_CHECK(cudaStreamSynchronize(stream_));
        if (trace) {
            trace->clear();
            for (size_t i = 0; i < steps_.size(); ++i) {
                float b = 0, e = 0;
                cudaEventElapsedTime(&b, evs[0], evs[i]);
                cudaEventElapsedTime(&e, evs[0], evs[i + 1]);
                trace->push_back({steps_[i].name, b, e});
            }
        }
        float total = 0;
        cudaEventElapsedTime(&total, evs[0], evs.back());
        device_ms_ = total;
        for (auto& e : evs) cudaEventDestroy(e);
    } else {
        CUDA_CHECK(cudaEventRecord(ev0_, stream_));
        launch_body(use_graph);
        CUDA_CHECK(cudaEventRecord(ev1_, stream_));
    }
    for (auto& kv : host_out_) {
        fmap_info& f = fmaps_[root(index_[kv.first])];
        if (f.f32_pitch)
            CUDA_CHECK(cudaMemcpy2DAsync(kv.second->mutable_cpu_data(), (size_t)f.C * 4, f.f32->p, (size_t)f.f32_pitch * 4,
                                         (size_t)f.C * 4, f.N, cudaMemcpyDeviceToHost, stream_));
        else
            CUDA_CHECK(cudaMemcpyAsync(kv.second->mutable_cpu_data(), f.f32->p, (size_t)f.N * f.C * f.H * f.W * 4,
                                       cudaMemcpyDeviceToHost, stream_));
    }
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    if (!profile) {
        float ms = 0;
        cudaEventElapsedTime(&ms, ev0_, ev1_);
        device_ms_ = ms;
    }
    exb_check(exb_ctx_sync_check(ctx_, stream_), "fused forward");
}

// The ingest step reads `ingest_src_` when it is launched and is therefore launched eagerly; the rest
// of the plan runs eagerly the first time and as one CUDA graph afterwards.
void fused_plan::launch_body(bool use_graph) {
    steps_[0].run(stream_);
    if (use_graph && warmed_ && steps_.size() > 1) {
        if (!graph_exec_) {
            cudaGraph_t graph = nullptr;
            CUDA_CHECK(cudaStreamBeginCapture(stream_, cudaStreamCaptureModeThreadLocal));
            for (size_t i = 1; i < steps_.size(); ++i) steps_[i].run(stream_);
            CUDA_CHECK(cudaStreamEndCapture(stream_, &graph));
            CUDA_CHECK(cudaGraphInstantiate(&graph_exec_, graph, 0));
            cudaGraphDestroy(graph);
        }
        CUDA_CHECK(cudaGraphLaunch(graph_exec_, stream_));
    } else {
        for (size_t i = 1; i < steps_.size(); ++i) steps_[i].run(stream_);
        warmed_ = true;
    }
}

double fused_plan::run_resident(int iters, bool use_graph) {
    if (!built_) return -1.0;
    CUDA_CHECK(cudaSetDevice(device_));
    ingest_src_ = staging_in_.p;
    ingest_src_f16_ = false;
    if (!warmed_) launch_body(false);      // make sure every kernel has run eagerly once
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    CUDA_CHECK(cudaEventRecord(ev0_, stream_));
    for (int i = 0; i < iters; ++i) launch_body(use_graph);
    CUDA_CHECK(cudaEventRecord(ev1_, stream_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    float ms = 0;
    cudaEventElapsedTime(&ms, ev0_, ev1_);
    exb_check(exb_ctx_sync_check(ctx_, stream_), "resident run");
    return ms;
}

void fused_plan::run_chunked(const float* host_input, int k, bool use_graph, int host_threads, const uint16_t* host_f16) {
    CUDA_CHECK(cudaSetDevice(device_));
    CHECK(built_ && k >= 1);
    const size_t chunk_elems = (size_t)N_ * C_ * H_ * W_;
    if (host_f16) CHECK(ingest_f16_capable_) << "this plan's ingest step cannot read fp16 planes";
    const bool convert = !host_f16 && host_threads > 0 && ingest_f16_capable_;
    const bool f16 = host_f16 != nullptr || convert;
    float* stage = static_cast<float*>(chunk_stage_.ensure(chunk_elems * 4 * k, device_));
    uint16_t* stage16 = reinterpret_cast<uint16_t*>(stage);
    if (convert) {
        if (host_f16_bytes_ < chunk_elems * 2 * k) {
            if (host_f16_) cudaFreeHost(host_f16_);
            host_f16_ = nullptr;
            CUDA_CHECK(cudaHostAlloc(&host_f16_, chunk_elems * 2 * k, cudaHostAllocDefault));
            host_f16_bytes_ = chunk_elems * 2 * k;
        }
        if (!pool_ || pool_->threads() != host_threads) pool_.reset(new convert_pool(host_threads));
    }
    if (!copy_stream_) CUDA_CHECK(cudaStreamCreateWithFlags(&copy_stream_, cudaStreamNonBlocking));
    while ((int)copied_.size() < k) {
        cudaEvent_t e;
        CUDA_CHECK(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        copied_.push_back(e);
    }
    for (auto& kv : host_out_) {
        auto& t = chunk_out_[kv.first];
        const std::vector<int> shp = kv.second->data_shape();
        if (!t || t->num() != shp[0] * k)
            t = std::shared_ptr<memory::tensor<float>>(
                new memory::tensor<float>(std::vector<int>{shp[0] * k, shp[1], shp[2], shp[3]}, device_, memory::NCHW, nullptr));
    }
    launches_ = 0;
    for (auto& s : steps_) launches_ += s.launches;
    launches_ *= k;
    // every copy is queued at once on its own stream; compute of chunk c waits for copy c only
    if (!convert) {
        for (int c = 0; c < k; ++c) {
            if (host_f16)
                CUDA_CHECK(cudaMemcpyAsync(stage16 + c * chunk_elems, host_f16 + c * chunk_elems, chunk_elems * 2,
                                           cudaMemcpyHostToDevice, copy_stream_));
            else
                CUDA_CHECK(cudaMemcpyAsync(stage + c * chunk_elems, host_input + c * chunk_elems, chunk_elems * 4,
                                           cudaMemcpyHostToDevice, copy_stream_));
            CUDA_CHECK(cudaEventRecord(copied_[c], copy_stream_));
        }
    }
    CUDA_CHECK(cudaEventRecord(ev0_, stream_));
    for (int c = 0; c < k; ++c) {
        if (convert) {
            // the host converts chunk c while the copy of chunk c-1 and the kernels of chunk c-2 run
            uint16_t* h16 = static_cast<uint16_t*>(host_f16_) + c * chunk_elems;
            pool_->run(host_input + c * chunk_elems, h16, chunk_elems);
            CUDA_CHECK(cudaMemcpyAsync(stage16 + c * chunk_elems, h16, chunk_elems * 2, cudaMemcpyHostToDevice, copy_stream_));
            CUDA_CHECK(cudaEventRecord(copied_[c], copy_stream_));
        }
        CUDA_CHECK(cudaStreamWaitEvent(stream_, copied_[c], 0));
        ingest_src_ = f16 ? static_cast<const void*>(stage16 + c * chunk_elems) : static_cast<const void*>(stage + c * chunk_elems);
        ingest_src_f16_ = f16;
        launch_body(use_graph);
        for (auto& kv : host_out_) {
            fmap_info& f = fmaps_[root(index_[kv.first])];
            const size_t per = (size_t)f.N * f.C * f.H * f.W;
            float* dst = chunk_out_[kv.first]->mutable_cpu_data() + c * per;
            if (f.f32_pitch)
                CUDA_CHECK(cudaMemcpy2DAsync(dst, (size_t)f.C * 4, f.f32->p, (size_t)f.f32_pitch * 4, (size_t)f.C * 4, f.N,
                                             cudaMemcpyDeviceToHost, stream_));
            else
                CUDA_CHECK(cudaMemcpyAsync(dst, f.f32->p, per * 4, cudaMemcpyDeviceToHost, stream_));
        }
    }
    CUDA_CHECK(cudaEventRecord(ev1_, stream_));
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    CUDA_CHECK(cudaStreamSynchronize(copy_stream_));
    float ms = 0;
    cudaEventElapsedTime(&ms, ev0_, ev1_);
    device_ms_ = ms;
    ingest_src_f16_ = false;
    exb_check(exb_ctx_sync_check(ctx_, stream_), "chunked forward");
}

std::shared_ptr<memory::tensor<float>> fused_plan::fetch(const std::string& name_in) {
    // "<feature map>:int8" asks for the quantised tensor the plan hands to int8 convolutions, as the raw integers
    // (-128..127 in fp32, not dequantised): what a parity test compares with quantize(reference map, scale).
    static const std::string kInt8Suffix = ":int8";
    const bool want_i8 = name_in.size() > kInt8Suffix.size() &&
                         name_in.compare(name_in.size() - kInt8Suffix.size(), kInt8Suffix.size(), kInt8Suffix) == 0;
    const std::string name = want_i8 ? name_in.substr(0, name_in.size() - kInt8Suffix.size()) : name_in;
    auto it = index_.find(name);
    if (it == index_.end()) return nullptr;
    fmap_info& f = fmaps_[root(it->second)];
    if (want_i8) {
        if (!f.produced || !f.i8 || f.w_pitch) return nullptr;
        auto t = std::shared_ptr<memory::tensor<float>>(
            new memory::tensor<float>(std::vector<int>{f.N, f.C, f.H, f.W}, device_, memory::NCHW, nullptr));
        CUDA_CHECK(cudaStreamSynchronize(stream_));
        exb_check(exb_nhwc_to_nchw_f32(ctx_, f.i8->p, EXB_I8, t->mutable_gpu_data(), f.N, f.C, f.H, f.W, f.cs, 1.f, nullptr),
                  "exb_nhwc_to_nchw_f32");
        CUDA_CHECK(cudaDeviceSynchronize());
        t->cpu_data();
        return t;
    }
    if (f.w_pitch) {
        LOG(WARNING) << "feature map " << name << " is kept in a padded row layout and is not exported";
        return nullptr;
    }
    if (!f.produced) {
        LOG(WARNING) << "feature map " << name << " was fused into its consumer and is not materialised; "
                        "call set_fusion(false) to inspect it";
        return nullptr;
    }
    auto t = std::shared_ptr<memory::tensor<float>>(
        new memory::tensor<float>(std::vector<int>{f.N, f.C, f.H, f.W}, device_, memory::NCHW, nullptr));
    if (f.f32 && f.need_f32 && !f.f16) {
        CUDA_CHECK(cudaStreamSynchronize(stream_));
        if (f.f32_pitch)
            CUDA_CHECK(cudaMemcpy2D(t->mutable_cpu_data(), (size_t)f.C * 4, f.f32->p, (size_t)f.f32_pitch * 4,
                                    (size_t)f.C * 4, f.N, cudaMemcpyDeviceToHost));
        else
            CUDA_CHECK(cudaMemcpy(t->mutable_cpu_data(), f.f32->p, (size_t)t->count() * 4, cudaMemcpyDeviceToHost));
        return t;
    }
    const void* src = f.f16 ? f.f16->p : (f.i8 ? f.i8->p : nullptr);
    if (!src) return nullptr;
    const int dt = f.f16 ? EXB_F16 : EXB_I8;
    const float scale = f.f16 ? 1.f : 1.f / f.i8_scale;
    CUDA_CHECK(cudaStreamSynchronize(stream_));
    exb_check(exb_nhwc_to_nchw_f32(ctx_, src, dt, t->mutable_gpu_data(), f.N, f.C, f.H, f.W, f.cs, scale, nullptr),
              "exb_nhwc_to_nchw_f32");
    CUDA_CHECK(cudaDeviceSynchronize());
    t->cpu_data();
    return t;
}

}  // namespace

// ------------------------------------------------------------------------------------------
// impl
// ------------------------------------------------------------------------------------------
template <typename Dtype>
class pipeline<Dtype>::impl {
public:
    impl() {}
    impl(std::string_view param_file, std::string_view model_file, int device)
        : impl(read_lines(param_file), model_file, device) {}
    impl(const std::vector<std::string>& lines, std::string_view model_file, int device) {
        device_ = device;
        lines_ = lines;
        model_file_ = std::string(model_file);
        if (device >= 0) CUDA_CHECK(cudaSetDevice(device));   // select the device BEFORE creating any handle
        if (lines.empty()) LOG(FATAL) << "Incorrect param file.";
        auto head = split_string(lines[0], " ");
        if (head.empty() || (head[0] != "glsv1" && head[0] != "7767517")) LOG(FATAL) << "Incorrect param file version.";
        if (head.size() > 1) name_ = head[1];
        for (size_t i = 2; i < lines.size(); ++i) {   // line 1 (op / feature map counts) is not used
            std::vector<std::string> tok;
            for (auto& s : split_string(lines[i], " "))
                if (!s.empty()) tok.push_back(s);
            if (tok.empty()) continue;
            if (tok.size() < 4) LOG(FATAL) << "malformed operation line: " << lines[i];
            operation_param p;
            p.type_ = tok[0];
            p.name_ = tok[1];
            p.device_ = device_;
            p.input_count_ = std::atoi(tok[2].c_str());
            p.output_count_ = std::atoi(tok[3].c_str());
            const int n_in = p.input_count_ > 0 ? p.input_count_ : 0, n_out = p.output_count_ > 0 ? p.output_count_ : 0;
            if ((int)tok.size() < 4 + n_in + n_out) LOG(FATAL) << "operation line lists fewer feature maps than it declares: " << lines[i];
            for (int j = 0; j < n_out; ++j) p.output_featmaps_.push_back(tok[4 + n_in + j]);
            for (size_t j = 4 + n_in + n_out; j < tok.size(); ++j) p.specific_params_ += tok[j] + " ";
            if (p.input_count_ <= 0) {
                p.input_count_ = 1;   // an op without inputs takes the implicit "<name>_input"
                p.input_featmaps_ = {p.name_ + "_input"};
            } else {
                for (int j = 0; j < n_in; ++j) p.input_featmaps_.push_back(tok[4 + j]);
            }
            op_params_.push_back(p);
        }
        for (auto& p : op_params_) operations_.push_back(operation_reflector<Dtype>::instance().create_object(p));
        if (model_file.empty()) {
            LOG(WARNING) << "THIS PIPELINE IS LOADED WITH DUMMY DATA.";
            for (auto& op : operations_) weights_mem_cost_ += op->init_weights();
        } else {
            FILE* fp = fopen(std::string(model_file).c_str(), "rb");
            if (!fp) LOG(FATAL) << "Cannot open " << model_file;
            for (auto& op : operations_) weights_mem_cost_ += op->init_weights(fp);
            CHECK_EQ(fclose(fp), 0) << "Cannot close " << model_file;
        }
        // feature map table; inputs = consumed but never produced, outputs = produced but never consumed
        std::set<std::string> produced, consumed;
        for (auto& p : op_params_) {
            for (auto& n : p.output_featmaps_) produced.insert(n);
            for (auto& n : p.input_featmaps_) consumed.insert(n);
        }
        for (auto& p : op_params_) {
            for (auto& n : p.input_featmaps_) {
                index_of(n);
                if (!produced.count(n) && std::find(input_names_.begin(), input_names_.end(), n) == input_names_.end())
                    input_names_.push_back(n);
            }
            for (auto& n : p.output_featmaps_) {
                index_of(n);
                if (!consumed.count(n)) output_names_.push_back(n);
            }
        }
        featmaps_.resize(featmap_index_.size());
        if (input_names_.empty()) LOG(FATAL) << "the graph has no input feature map";
    }
    ~impl() {
        chunk_plan_.reset();
        plan_.reset();
        if (ctx_) exb_ctx_destroy(ctx_);
    }

    result_map forward(const std::shared_ptr<memory::tensor<Dtype>>& input) {
        if (device_ >= 0) return forward_gpu(input);
        return forward_cpu(input);
    }
    result_map forward_cpu(const std::shared_ptr<memory::tensor<Dtype>>&) {
        NO_CPU;
        return {};
    }
    result_map forward_gpu(const std::shared_ptr<memory::tensor<Dtype>>& input);
    std::shared_ptr<memory::tensor<Dtype>> get_featmap(std::string_view name);

    int index_of(const std::string& n) {
        auto it = featmap_index_.find(n);
        if (it != featmap_index_.end()) return it->second;
        int id = (int)featmap_index_.size();
        featmap_index_[n] = id;
        return id;
    }
    result_map forward_unfused(const std::shared_ptr<memory::tensor<Dtype>>& input);

    // fp16 input already on the host (pipeline<unsigned short>): the fused plan copies it as it is (half the bytes of
    // the fp32 form); false when this graph's plan cannot ingest fp16 planes (nothing has run then).
    bool forward_f16_input(const uint16_t* host_f16, int N, int C, int H, int W, result_map& out);

    std::string name_;
    int device_ = -1;
    std::vector<std::string> lines_;
    std::string model_file_;
    // pipeline<unsigned short> runs its fused plan through a float pipeline of the same graph (the plan keeps fp16 /
    // int8 tensors on the device whatever the host type is); built on the first forward that can use it
    std::unique_ptr<typename pipeline<float>::impl> inner_;
    bool inner_unusable_ = false;
    // fp16 result tensors of the fused path, reused from forward to forward: allocating and freeing pinned host
    // memory per call synchronises the whole device, which serialises two callers that share a GPU
    std::unordered_map<std::string, std::shared_ptr<memory::tensor<Dtype>>> f16_results_;
    std::vector<operation_param> op_params_;
    std::vector<std::shared_ptr<operation<Dtype>>> operations_;
    std::unordered_map<std::string, int> featmap_index_;
    std::vector<std::shared_ptr<memory::tensor<Dtype>>> featmaps_;
    std::vector<std::string> input_names_, output_names_;
    int weights_mem_cost_ = 0;
    bool profile_ = false, fusion_ = true, graph_ = true;
    bool used_fused_ = false;
    int h2d_chunks_ = 1;
    int host_f16_threads_ = 0;
    std::string plan_refused_;      // why this graph's fused plan could not be built (then: op by op for good)
    bool used_chunked_ = false;
    std::unique_ptr<fused_plan> chunk_plan_;
    exb_ctx* ctx_ = nullptr;
    std::unique_ptr<fused_plan> plan_;
    std::vector<trace_event> trace_;
    int launches_ = 0;
    double device_ms_ = 0.0;
};

template <>
std::shared_ptr<memory::tensor<float>> pipeline<float>::impl::get_featmap(std::string_view name);
template <>
std::shared_ptr<memory::tensor<unsigned short>> pipeline<unsigned short>::impl::get_featmap(std::string_view name);
template <>
bool pipeline<float>::impl::forward_f16_input(const uint16_t* host_f16, int N, int C, int H, int W, result_map& out);
template <>
pipeline<float>::result_map pipeline<float>::impl::forward_gpu(const std::shared_ptr<memory::tensor<float>>& input);
template <>
pipeline<unsigned short>::result_map pipeline<unsigned short>::impl::forward_gpu(
    const std::shared_ptr<memory::tensor<unsigned short>>& input);

// Op-by-op execution in file order with the reference's tensor semantics.
template <typename Dtype>
typename pipeline<Dtype>::result_map pipeline<Dtype>::impl::forward_unfused(
    const std::shared_ptr<memory::tensor<Dtype>>& input) {
    CUDA_CHECK(cudaSetDevice(device_));
    if (!ctx_) exb_check(exb_ctx_create(device_, &ctx_), "exb_ctx_create");
    std::shared_ptr<memory::tensor<Dtype>> in0 = input;
    if (input->device() != device_) {
        // A tensor made for another device would be uploaded there (and switch this thread's current
        // device): work on a copy that lives on the pipeline's device.
        in0 = std::shared_ptr<memory::tensor<Dtype>>(
            new memory::tensor<Dtype>(input->data_shape(), device_, input->order(), input->allocator()));
        std::memcpy(in0->mutable_cpu_data(), input->cpu_data(), (size_t)input->count() * sizeof(Dtype));
    }
    featmaps_[featmap_index_[input_names_[0]]] = in0;
    trace_.clear();
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    if (profile_) {
        CUDA_CHECK(cudaEventCreate(&e0));
        CUDA_CHECK(cudaEventCreate(&e1));
    }
    float t_acc = 0.f;
    for (size_t i = 0; i < operations_.size(); ++i) {
        const auto& p = op_params_[i];
        std::vector<std::shared_ptr<memory::tensor<Dtype>>> in(p.input_featmaps_.size()), out(p.output_featmaps_.size());
        for (size_t j = 0; j < in.size(); ++j) {
            in[j] = featmaps_[featmap_index_[p.input_featmaps_[j]]];
            if (!in[j]) LOG(FATAL) << "feature map " << p.input_featmaps_[j] << " is not available for " << p.name_;
        }
        if (profile_) CUDA_CHECK(cudaEventRecord(e0, nullptr));
        operations_[i]->forward_gpu(ctx_, in, out);
        if (profile_) {
            CUDA_CHECK(cudaEventRecord(e1, nullptr));
            CUDA_CHECK(cudaEventSynchronize(e1));
            float ms = 0;
            cudaEventElapsedTime(&ms, e0, e1);
            trace_.push_back({p.name_, t_acc, t_acc + ms});
            t_acc += ms;
        }
        for (size_t j = 0; j < out.size(); ++j) featmaps_[featmap_index_[p.output_featmaps_[j]]] = out[j];
    }
    if (profile_) {
        cudaEventDestroy(e0);
        cudaEventDestroy(e1);
    }
    exb_check(exb_ctx_sync_check(ctx_, nullptr), "forward");
    result_map results;
    for (auto& n : output_names_) {
        results[n] = featmaps_[featmap_index_[n]];
        if (results[n]) results[n]->cpu_data();   // bring the result to the host, as a caller of the reference would read it
    }
    launches_ = -1;
    return results;
}

template <typename Dtype>
typename pipeline<Dtype>::result_map pipeline<Dtype>::impl::forward_gpu(
    const std::shared_ptr<memory::tensor<Dtype>>& input) {
    if (device_ < 0) NO_GPU;
    CHECK(input != nullptr && !input->empty()) << "empty input tensor";
    used_fused_ = false;
    return forward_unfused(input);
}

template <>
pipeline<float>::result_map pipeline<float>::impl::forward_gpu(const std::shared_ptr<memory::tensor<float>>& input) {
    if (device_ < 0) NO_GPU;
    CHECK(input != nullptr && !input->empty()) << "empty input tensor";
    if (fusion_) {
        if (!plan_) plan_.reset(new fused_plan(op_params_, operations_, input_names_, output_names_, device_));
        std::string why = plan_refused_.empty() ? plan_->unsupported_reason() : plan_refused_;
        if (why.empty()) try {
            if (input->order() == memory::NHWC) input->convert_order();
            const int N = input->num(), C = input->channels(), H = input->height(), W = input->width();
            used_chunked_ = false;
            if ((h2d_chunks_ > 1 || host_f16_threads_ > 0) && !profile_ && N % h2d_chunks_ == 0) {
                if (!chunk_plan_)
                    chunk_plan_.reset(new fused_plan(op_params_, operations_, input_names_, output_names_, device_));
                const int nc = N / h2d_chunks_;
                if (!chunk_plan_->built_for(nc, C, H, W)) chunk_plan_->build(nc, C, H, W);
                chunk_plan_->run_chunked(input->cpu_data(), h2d_chunks_, graph_, host_f16_threads_);
                launches_ = chunk_plan_->launches();
                device_ms_ = chunk_plan_->device_ms();
                used_fused_ = true;
                used_chunked_ = true;
                return chunk_plan_->chunk_out_;
            }
            if (!plan_->built_for(N, C, H, W)) plan_->build(N, C, H, W);
            plan_->run(input->cpu_data(), graph_, profile_, &trace_);
            launches_ = plan_->launches();
            device_ms_ = plan_->device_ms();
            used_fused_ = true;
            return plan_->host_out_;
        } catch (const plan_refusal& e) {
            // nothing has run yet: the refusal comes from building the plan
            plan_refused_ = e.what();
            why = plan_refused_;
            plan_.reset();
            chunk_plan_.reset();
        }
        LOG(WARNING) << "running op by op: " << why;
    }
    used_fused_ = false;
    return forward_unfused(input);
}

template <typename Dtype>
bool pipeline<Dtype>::impl::forward_f16_input(const uint16_t*, int, int, int, int, result_map&) { return false; }
template <>
bool pipeline<float>::impl::forward_f16_input(const uint16_t* host_f16, int N, int C, int H, int W, result_map& out) {
    if (!fusion_ || !plan_refused_.empty()) return false;
    if (!chunk_plan_) chunk_plan_.reset(new fused_plan(op_params_, operations_, input_names_, output_names_, device_));
    if (!chunk_plan_->unsupported_reason().empty()) return false;
    const int k = (h2d_chunks_ > 1 && N % h2d_chunks_ == 0) ? h2d_chunks_ : 1;
    try {
        if (!chunk_plan_->built_for(N / k, C, H, W)) chunk_plan_->build(N / k, C, H, W);
    } catch (const plan_refusal& e) {
        plan_refused_ = e.what();
        chunk_plan_.reset();
        return false;
    }
    if (!chunk_plan_->host_f16_capable()) return false;
    chunk_plan_->run_chunked(nullptr, k, graph_, 0, host_f16);
    launches_ = chunk_plan_->launches();
    device_ms_ = chunk_plan_->device_ms();
    used_fused_ = true;
    used_chunked_ = true;
    out = chunk_plan_->chunk_out_;
    return true;
}

namespace {
std::shared_ptr<memory::tensor<unsigned short>> to_f16_tensor(const std::shared_ptr<memory::tensor<float>>& t, int device) {
    if (!t) return nullptr;
    auto h = std::shared_ptr<memory::tensor<unsigned short>>(
        new memory::tensor<unsigned short>(t->data_shape(), device, memory::NCHW, nullptr));
    convert_f32_to_f16(t->cpu_data(), h->mutable_cpu_data(), (size_t)t->count());
    return h;
}
}  // namespace

// pipeline<unsigned short> (the reference's fp16 Dtype: tensors of IEEE half bits, src/Excalibur/operation.cpp:74-93,
// 124-126).  A network whose fused plan can read fp16 planes (a 3-channel image in front of an fp16 stem convolution)
// runs that plan: the caller's fp16 input crosses PCIe as it is, results come back as fp16 tensors.  Everything else
// runs op by op on operation<unsigned short> objects.
template <>
pipeline<unsigned short>::result_map pipeline<unsigned short>::impl::forward_gpu(
    const std::shared_ptr<memory::tensor<unsigned short>>& input) {
    if (device_ < 0) NO_GPU;
    CHECK(input != nullptr && !input->empty()) << "empty input tensor";
    used_fused_ = false;
    if (fusion_ && !inner_unusable_) {
        if (input->order() == memory::NHWC) input->convert_order();
        if (!inner_) inner_.reset(new pipeline<float>::impl(lines_, model_file_, device_));
        inner_->graph_ = graph_;
        inner_->h2d_chunks_ = h2d_chunks_;
        pipeline<float>::result_map res;
        if (inner_->forward_f16_input(input->cpu_data(), input->num(), input->channels(), input->height(), input->width(), res)) {
            launches_ = inner_->launches_;
            device_ms_ = inner_->device_ms_;
            used_fused_ = true;
            result_map out;
            for (auto& kv : res) {
                auto& h = f16_results_[kv.first];
                if (!kv.second) {
                    h.reset();
                } else {
                    if (!h || h->data_shape() != kv.second->data_shape())
                        h = std::shared_ptr<memory::tensor<unsigned short>>(
                            new memory::tensor<unsigned short>(kv.second->data_shape(), device_, memory::NCHW, nullptr));
                    convert_f32_to_f16(kv.second->cpu_data(), h->mutable_cpu_data(), (size_t)kv.second->count());
                }
                out[kv.first] = h;
            }
            return out;
        }
        inner_unusable_ = true;
        inner_.reset();
        LOG(WARNING) << "running op by op: the fused plan of this graph cannot read an fp16 input";
    }
    if (input->order() == memory::NCHW) {
        // the fp16 operations work on channel-last tensors (as the reference's fp16 GPU path does): reorder on the host
        const int n = input->num(), c = input->channels(), h = input->height(), w = input->width();
        auto t = std::shared_ptr<memory::tensor<unsigned short>>(
            new memory::tensor<unsigned short>(std::vector<int>{n, h, w, c}, device_, memory::NHWC, input->allocator()));
        const unsigned short* src = input->cpu_data();
        unsigned short* dst = t->mutable_cpu_data();
        for (int in = 0; in < n; ++in)
            for (int ic = 0; ic < c; ++ic)
                for (int ih = 0; ih < h; ++ih)
                    for (int iw = 0; iw < w; ++iw)
                        dst[(((size_t)in * h + ih) * w + iw) * c + ic] = src[(((size_t)in * c + ic) * h + ih) * w + iw];
        return forward_unfused(t);
    }
    return forward_unfused(input);
}

template <typename Dtype>
std::shared_ptr<memory::tensor<Dtype>> pipeline<Dtype>::impl::get_featmap(std::string_view name) {
    auto it = featmap_index_.find(std::string(name));
    if (it == featmap_index_.end()) return nullptr;
    return featmaps_[it->second];
}
template <>
std::shared_ptr<memory::tensor<float>> pipeline<float>::impl::get_featmap(std::string_view name) {
    if (used_fused_ && used_chunked_ && chunk_plan_) {
        auto o = chunk_plan_->chunk_out_.find(std::string(name));
        if (o != chunk_plan_->chunk_out_.end()) return o->second;
        return chunk_plan_->fetch(std::string(name));
    }
    if (used_fused_ && plan_) return plan_->fetch(std::string(name));
    auto it = featmap_index_.find(std::string(name));
    if (it == featmap_index_.end()) return nullptr;
    return featmaps_[it->second];
}
template <>
std::shared_ptr<memory::tensor<unsigned short>> pipeline<unsigned short>::impl::get_featmap(std::string_view name) {
    if (used_fused_ && inner_) return to_f16_tensor(inner_->get_featmap(name), device_);
    auto it = featmap_index_.find(std::string(name));
    if (it == featmap_index_.end()) return nullptr;
    return featmaps_[it->second];
}

// chrome://tracing JSON: one "B" / "E" event pair per entry, timestamps in microseconds; names are escaped.
bool write_chrome_trace(std::string_view path, const std::vector<std::string>& names, const std::vector<double>& begin_ms,
                        const std::vector<double>& end_ms) {
    if (names.size() != begin_ms.size() || names.size() != end_ms.size()) return false;
    std::ofstream out{std::string(path)};
    if (!out) return false;
    auto escaped = [](const std::string& s) {
        std::string r;
        for (char c : s) {
            if (c == '"' || c == '\\') {
                r += '\\';
                r += c;
            } else if ((unsigned char)c < 0x20) {
                char buf[8];
                std::snprintf(buf, sizeof(buf), "\\u%04x", (unsigned)(unsigned char)c);
                r += buf;
            } else {
                r += c;
            }
        }
        return r;
    };
    out << "{\"traceEvents\":[";
    for (size_t i = 0; i < names.size(); ++i) {
        for (int k = 0; k < 2; ++k) {
            if (i || k) out << ",";
            out << "{\"name\":\"" << escaped(names[i]) << "\",\"cat\":\"op\",\"ph\":\"" << (k ? "E" : "B")
                << "\",\"pid\":0,\"tid\":0,\"ts\":" << (k ? end_ms[i] : begin_ms[i]) * 1000.0 << "}";
        }
    }
    out << "]}";
    return (bool)out;
}

// ------------------------------------------------------------------------------------------
// public wrappers
// ------------------------------------------------------------------------------------------
template <typename Dtype> pipeline<Dtype>::pipeline() : impl_{new impl} {}
template <typename Dtype>
pipeline<Dtype>::pipeline(std::string_view param_file, std::string_view model_file, int device)
    : impl_{new impl{param_file, model_file, device}} {}
template <typename Dtype>
pipeline<Dtype>::pipeline(std::string_view param_file, int device) : impl_{new impl{param_file, std::string_view{}, device}} {}
template <typename Dtype>
pipeline<Dtype>::pipeline(const std::vector<std::string>& lines, std::string_view model_file, int device)
    : impl_{new impl{lines, model_file, device}} {}
template <typename Dtype> pipeline<Dtype>::~pipeline() { delete impl_; }

template <typename Dtype>
typename pipeline<Dtype>::result_map pipeline<Dtype>::forward(const std::shared_ptr<memory::tensor<Dtype>>& t) { return impl_->forward(t); }
template <typename Dtype>
typename pipeline<Dtype>::result_map pipeline<Dtype>::forward_cpu(const std::shared_ptr<memory::tensor<Dtype>>& t) { return impl_->forward_cpu(t); }
template <typename Dtype>
typename pipeline<Dtype>::result_map pipeline<Dtype>::forward_gpu(const std::shared_ptr<memory::tensor<Dtype>>& t) { return impl_->forward_gpu(t); }
template <typename Dtype>
std::shared_ptr<memory::tensor<Dtype>> pipeline<Dtype>::get_featmap(std::string_view n) { return impl_->get_featmap(n); }
template <typename Dtype> void pipeline<Dtype>::enable_profiler() { impl_->profile_ = true; }
template <typename Dtype> void pipeline<Dtype>::disable_profiler() { impl_->profile_ = false; }
template <typename Dtype> int pipeline<Dtype>::device() const { return impl_->device_; }
template <typename Dtype> void pipeline<Dtype>::set_fusion(bool on) { impl_->fusion_ = on; }
template <typename Dtype> void pipeline<Dtype>::set_cuda_graph(bool on) { impl_->graph_ = on; }
template <typename Dtype> void pipeline<Dtype>::set_h2d_chunks(int k) { impl_->h2d_chunks_ = k < 1 ? 1 : k; }
template <typename Dtype> void pipeline<Dtype>::set_host_f16_threads(int t) { impl_->host_f16_threads_ = t < 0 ? 0 : t; }
template <typename Dtype> int pipeline<Dtype>::launches_last_forward() const { return impl_->launches_; }
template <typename Dtype> double pipeline<Dtype>::run_resident(int iters) {
    if (!impl_->plan_ || !impl_->used_fused_ || !impl_->plan_->built()) return -1.0;
    return impl_->plan_->run_resident(iters, impl_->graph_);
}
template <typename Dtype> int pipeline<Dtype>::trace_size() const { return (int)impl_->trace_.size(); }
template <typename Dtype>
bool pipeline<Dtype>::trace_entry(int i, std::string& name, double& b, double& e) const {
    if (i < 0 || i >= (int)impl_->trace_.size()) return false;
    name = impl_->trace_[i].name;
    b = impl_->trace_[i].begin_ms;
    e = impl_->trace_[i].end_ms;
    return true;
}
template <typename Dtype> double pipeline<Dtype>::device_ms_last_forward() const { return impl_->device_ms_; }
template <typename Dtype> std::vector<std::string> pipeline<Dtype>::input_names() const { return impl_->input_names_; }
template <typename Dtype> std::vector<std::string> pipeline<Dtype>::output_names() const { return impl_->output_names_; }
template <typename Dtype> std::string pipeline<Dtype>::version() { return exb_version(); }

template <typename Dtype>
bool pipeline<Dtype>::dump_profile(std::string_view path) {
    std::vector<std::string> names;
    std::vector<double> b, e;
    for (auto& ev : impl_->trace_) {
        names.push_back(ev.name);
        b.push_back(ev.begin_ms);
        e.push_back(ev.end_ms);
    }
    return write_chrome_trace(path, names, b, e);
}

INSTANCE_CLASS(pipeline);

}  // namespace excalibur
}  // namespace glasssix
