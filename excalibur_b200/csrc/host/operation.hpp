// The operation plug-in interface of the reference (include/Excalibur/operation.hpp:27-89,109-374,
// include/Excalibur/operation_reflector.hpp:16-93, src/Excalibur/operation.cpp:12-126), restated
// for this library: same operation_param fields and CHECKs, same Dtype set {float, double,
// unsigned short = fp16 bits}, same dtype dispatch, same string-keyed factory and REGISTE macros.
// Differences, all forced by "GPU only, no cuBLAS": forward_gpu takes this library's context
// (exb_ctx*&) where the reference takes cublasHandle_t&, and every forward_cpu_* is a fatal
// error (there is no CPU fallback).
#pragma once
#include <algorithm>
#include <cstdio>
#include <functional>
#include <map>
#include <string>
#include <vector>

#include "../../../include/excalibur_b200.h"
#include "primitives.hpp"

namespace glasssix {
namespace excalibur {

struct operation_param {
    std::string type_;
    std::string name_;
    int input_count_;
    int output_count_;
    std::vector<std::string> input_featmaps_;
    std::vector<std::string> output_featmaps_;
    bool int8_quantization_;
    bool brain_float16_;
    bool float16_;
    bool inplace_;
    int device_;
    std::string specific_params_;  // "k=v k=v ..."

    operation_param(std::string type = "N/A", std::string name = "N/A", int input_count = 1, int output_count = 1,
                    std::vector<std::string> input_featmaps = {}, std::vector<std::string> output_featmaps = {},
                    bool int8_quantization = false, bool brain_float16 = false, bool float16 = false,
                    bool inplace = false, int device = -1, std::string specific_params = "")
        : type_(type), name_(name), input_count_(input_count), output_count_(output_count),
          input_featmaps_(input_featmaps), output_featmaps_(output_featmaps),
          int8_quantization_(int8_quantization), brain_float16_(brain_float16), float16_(float16),
          inplace_(inplace), device_(device), specific_params_(specific_params) {
        CHECK(!(brain_float16_ && float16_));
        CHECK(!(brain_float16_ && int8_quantization_));
        CHECK(!(float16_ && int8_quantization_));
    }
    void set_int8_quantization(bool v) { int8_quantization_ = v; }
    void set_brain_float16(bool v) { brain_float16_ = v; }
    void set_float16(bool v) { float16_ = v; }
};

inline std::vector<std::string> split_string(const std::string& s, const std::string& sep) {
    std::vector<std::string> out;
    size_t from = 0, at;
    while ((at = s.find(sep, from)) != std::string::npos) {
        out.push_back(s.substr(from, at - from));
        from = at + sep.size();
    }
    if (from != s.length()) out.push_back(s.substr(from));
    return out;
}

// Parsed "k=v" list of an op line; keys are the reference's integer keys.
struct param_list {
    std::vector<std::pair<int, std::string>> kv;
    explicit param_list(const std::string& specific_params) {
        for (const auto& tok : split_string(specific_params, " ")) {
            if (tok.empty()) continue;
            auto parts = split_string(tok, "=");
            if (parts.size() != 2) LOG(FATAL) << "malformed parameter token '" << tok << "'";
            kv.emplace_back(std::atoi(parts[0].c_str()), parts[1]);
        }
    }
};

template <typename Dtype>
class operation {
public:
    typedef std::vector<std::shared_ptr<memory::tensor<Dtype>>> tensor_list;
    typedef std::vector<std::shared_ptr<memory::tensor<float>>> f32_list;
    typedef std::vector<std::shared_ptr<memory::tensor<unsigned short>>> f16_list;

    operation() {}
    explicit operation(const operation_param& param);
    virtual ~operation() {}

    virtual int init_weights() { return 0; }          // seeded dummy weights
    virtual int init_weights(FILE*) { return 0; }     // returns the bytes consumed

    void forward_cpu(const tensor_list& bottoms, tensor_list& tops);
    void forward_gpu(exb_ctx*& handle, const tensor_list& bottoms, tensor_list& tops);

    std::vector<std::shared_ptr<memory::tensor<float>>>& weights_f32() { return weights_f32_; }
    std::vector<std::shared_ptr<memory::tensor<unsigned short>>>& weights_f16() { return weights_f16_; }
    std::vector<std::shared_ptr<memory::tensor<signed char>>>& weights_i8() { return weights_i8_; }
    std::shared_ptr<memory::tensor<float>>& weights_scaletable_i8() { return weights_scaletable_i8_; }
    std::shared_ptr<memory::tensor<float>>& featmap_scaletable_i8() { return featmap_scaletable_i8_; }
    const operation_param& param() const { return params_; }
    virtual const char* type() const { return "Unknown Type"; }

protected:
    std::vector<std::shared_ptr<memory::tensor<float>>> weights_f32_;
    std::vector<std::shared_ptr<memory::tensor<unsigned short>>> weights_f16_;
    std::vector<std::shared_ptr<memory::tensor<signed char>>> weights_i8_;
    operation_param params_;
    std::shared_ptr<memory::tensor<float>> weights_scaletable_i8_;
    std::shared_ptr<memory::tensor<float>> featmap_scaletable_i8_;

    virtual void forward_cpu_f32(const f32_list&, f32_list&) { NO_CPU; }
    virtual void forward_cpu_f16(const f16_list&, f16_list&) { NO_CPU; }
    virtual void forward_cpu_i8(const f32_list&, f32_list&) { NO_CPU; }
    virtual void forward_gpu_f32(exb_ctx*&, const f32_list&, f32_list&) { NOT_IMPLEMENTED; }
    virtual void forward_gpu_f16(exb_ctx*&, const f16_list&, f16_list&) { NOT_IMPLEMENTED; }
    virtual void forward_gpu_i8(exb_ctx*&, const f32_list&, f32_list&) {
        NOT_IMPLEMENTED << " This function should be overrided in derived class";
    }

private:
    DISABLE_COPY_AND_ASSIGN(operation);
};

template <typename Dtype>
class operation_reflector {
public:
    typedef std::function<std::shared_ptr<operation<Dtype>>(const operation_param&)> generator;
    static operation_reflector& instance();   // one registry per Dtype for the whole library
    std::shared_ptr<operation<Dtype>> create_object(const operation_param& param) {
        std::string type = param.type_;
        std::transform(type.begin(), type.end(), type.begin(), ::tolower);
        auto it = object_map_.find(std::string("operation_") + type);
        if (it != object_map_.end()) return it->second(param);
        LOG(FATAL) << "Un-suppoted operation type: " << param.type_ << ". ";
        return nullptr;
    }
    // Last registration of a name wins.
    void registe(const std::string& class_name, generator&& g) { object_map_[class_name] = g; }
    bool has(const std::string& class_name) const { return object_map_.count(class_name) != 0; }

private:
    std::map<std::string, generator> object_map_;
};

template <typename Dtype>
class register_action {
public:
    register_action(const std::string& class_name, typename operation_reflector<Dtype>::generator&& g) {
        operation_reflector<Dtype>::instance().registe(class_name, std::move(g));
    }
};

#define INSTANCE_CLASS(CLASS_NAME)     \
    template class CLASS_NAME<float>;  \
    template class CLASS_NAME<double>; \
    template class CLASS_NAME<unsigned short>;

#define REGISTE_ONE(CLASS_NAME, DTYPE, TAG)                                                   \
    static ::glasssix::excalibur::register_action<DTYPE> g_##TAG##_register_action_##CLASS_NAME( \
        #CLASS_NAME, [](const ::glasssix::excalibur::operation_param& param) {                \
            return std::shared_ptr<::glasssix::excalibur::operation<DTYPE>>(new CLASS_NAME<DTYPE>(param)); \
        });
#define REGISTE_SHORT(CLASS_NAME) REGISTE_ONE(CLASS_NAME, unsigned short, us)
#define REGISTE_FLOAT(CLASS_NAME) REGISTE_ONE(CLASS_NAME, float, f)
#define REGISTE_DOUBLE(CLASS_NAME) REGISTE_ONE(CLASS_NAME, double, d)
#define REGISTE(CLASS_NAME) REGISTE_SHORT(CLASS_NAME) REGISTE_FLOAT(CLASS_NAME) REGISTE_DOUBLE(CLASS_NAME)

}  // namespace excalibur
}  // namespace glasssix
