// Dtype dispatch of operation<Dtype> (reference src/Excalibur/operation.cpp:12-126) and the
// per-Dtype registries.
#include "operation.hpp"

namespace glasssix {

static fatal_handler_t g_fatal_handler = nullptr;
static bool g_log_quiet = false;
void set_fatal_handler(fatal_handler_t h) { g_fatal_handler = h; }
fatal_handler_t get_fatal_handler() { return g_fatal_handler; }
void set_log_quiet(bool q) { g_log_quiet = q; }
bool log_quiet() { return g_log_quiet; }

namespace excalibur {

template <typename Dtype>
operation<Dtype>::operation(const operation_param& param) : params_(param) {}

template <>
operation<unsigned short>::operation(const operation_param& param) : params_(param) {
    params_.set_float16(true);
}

template <>
void operation<float>::forward_cpu(const tensor_list& bottoms, tensor_list& tops) {
    if (params_.int8_quantization_) forward_cpu_i8(bottoms, tops);
    else forward_cpu_f32(bottoms, tops);
}
template <>
void operation<float>::forward_gpu(exb_ctx*& h, const tensor_list& bottoms, tensor_list& tops) {
    if (params_.int8_quantization_) forward_gpu_i8(h, bottoms, tops);
    else forward_gpu_f32(h, bottoms, tops);
}
template <>
void operation<unsigned short>::forward_cpu(const tensor_list& bottoms, tensor_list& tops) {
    forward_cpu_f16(bottoms, tops);
}
template <>
void operation<unsigned short>::forward_gpu(exb_ctx*& h, const tensor_list& bottoms, tensor_list& tops) {
    forward_gpu_f16(h, bottoms, tops);
}
// The reference routes double tensors to *_d64 entry points that no operation on this path
// implements; here that is stated directly.
template <>
void operation<double>::forward_cpu(const tensor_list&, tensor_list&) { NO_CPU; }
template <>
void operation<double>::forward_gpu(exb_ctx*&, const tensor_list&, tensor_list&) {
    NOT_IMPLEMENTED << " (double tensors have no kernel on this path)";
}

template class operation<float>;
template class operation<double>;
template class operation<unsigned short>;

template <typename Dtype>
operation_reflector<Dtype>& operation_reflector<Dtype>::instance() {
    static operation_reflector<Dtype> inst;
    return inst;
}
template class operation_reflector<float>;
template class operation_reflector<double>;
template class operation_reflector<unsigned short>;

}  // namespace excalibur
}  // namespace glasssix
