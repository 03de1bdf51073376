// Reference-side binding: what a maintainer of the reference adds to ITS tree (next to
// src/Excalibur/cuda/operation_convolution.cu) to route Convolution layers to libexcalibur_b200.so.
//
// It compiles against the reference's own headers (USE_CUDA, no cuDNN) and this library's C header only:
//     g++ -std=c++17 -fsyntax-only -DUSE_CUDA -I<reference>/include -I<reference>/include/Primitives \
//         -I<reference>/include/Excalibur -I<cuda>/include -I<this repo>/include operation_convolution_b200.cpp
// (tests/test_integration_file.py runs exactly that where the reference tree is present).
//
// The class derives from the reference's operation_convolution<Dtype>, so parameter parsing (keys 0..21, -23330)
// and weight loading (.racy records, tag 0 / 871224) stay the reference's own code; only forward_gpu_f32 and
// forward_gpu_i8 are replaced.  Registration under the stock key "operation_convolution" after the stock class
// makes the reflector hand out this class (operation_reflector<Dtype>::registe is a map assignment: the last
// registration of a name wins, include/Excalibur/operation_reflector.hpp:24-51).
#include <cstring>
#include <memory>
#include <vector>

#include "Excalibur/operation_convolution.hpp"
#include "Excalibur/operation_reflector.hpp"
#include "excalibur_b200.h"

namespace glasssix {
namespace excalibur {

template <typename Dtype>
class operation_convolution_b200 : public operation_convolution<Dtype> {
public:
    explicit operation_convolution_b200(const operation_param& param) : operation_convolution<Dtype>(param) {}
    virtual ~operation_convolution_b200() {
        if (packed_) exb_conv_weights_destroy(packed_);
        if (x_nhwc_) cudaFree(x_nhwc_);
        if (y_nhwc_) cudaFree(y_nhwc_);
        if (ctx_) exb_ctx_destroy(ctx_);
    }

protected:
    typedef std::vector<std::shared_ptr<memory::tensor<float>>> f32_list;

    // reference signature: include/Excalibur/operation.hpp (USE_CUDA, no cuDNN); the cuBLAS handle is not used
    virtual void forward_gpu_f32(cublasHandle_t&, const f32_list& bottoms, f32_list& tops) { run(bottoms, tops, false); }
    virtual void forward_gpu_i8(cublasHandle_t&, const f32_list& bottoms, f32_list& tops) { run(bottoms, tops, true); }

private:
    static void check(int rc, const char* what) {
        if (rc != EXB_OK) LOG(FATAL) << what << " failed (" << rc << "): " << exb_last_error_string();
    }

    void run(const f32_list& bottoms, f32_list& tops, bool int8) {
        CHECK_EQ(bottoms.size(), (size_t)1);
        const std::shared_ptr<memory::tensor<float>>& x = bottoms[0];
        const int device = x->device();
        if (!ctx_) check(exb_ctx_create(device, &ctx_), "exb_ctx_create");
        const int N = x->num(), C = x->channels(), H = x->height(), W = x->width();

        exb_conv_desc d;
        std::memset(&d, 0, sizeof(d));
        d.N = N; d.H = H; d.W = W; d.Cin = C; d.Cout = this->output_channel_;
        d.kh = this->kernel_size_h_; d.kw = this->kernel_size_w_;
        d.stride_h = this->stride_h_; d.stride_w = this->stride_w_;
        d.pad_t = this->pad_top_; d.pad_b = this->pad_bottom_; d.pad_l = this->pad_left_; d.pad_r = this->pad_right_;
        d.dilation = 1;
        d.group = this->group_;
        d.in_dtype = int8 ? EXB_I8 : EXB_F16;
        d.cin_stride = this->group_ == 1 ? (C + (int8 ? 31 : 15)) / (int8 ? 32 : 16) * (int8 ? 32 : 16) : C;
        d.out_dtype = EXB_F32; d.out2_dtype = -1; d.res_dtype = -1;
        d.out_scale = 1.f; d.out2_scale = 1.f;
        // conv key 9: 0 none, 1 ReLU, 3 the reference's ReLU6 (0 above 6), 4 sigmoid, 5 Mish
        d.act = this->activation_type_;
        int OH = 0, OW = 0;
        check(exb_conv_out_dims(&d, &OH, &OW), "exb_conv_out_dims");

        if (!packed_) {   // once, where the reference runs its own weight transforms
            const float* bias = this->bias_term_ && this->bias_data ? this->bias_data->cpu_data() : nullptr;
            if (int8)
                check(exb_conv_weights_pack_i8(ctx_, &d, this->weights_i8_[0]->cpu_data(), bias,
                                               this->weights_scaletable_i8_->cpu_data(), this->output_channel_,
                                               this->featmap_scaletable_i8_->cpu_data()[0], &packed_),
                      "exb_conv_weights_pack_i8");
            else
                check(exb_conv_weights_pack_f16(ctx_, &d, this->weights_f32_[0]->cpu_data(), bias, &packed_),
                      "exb_conv_weights_pack_f16");
        }
        tops.resize(1);
        tops[0].reset(new memory::tensor<float>(std::vector<int>{N, this->output_channel_, OH, OW}, device, memory::NCHW,
                                                x->allocator()));
        const size_t in_bytes = (size_t)N * H * W * d.cin_stride * (int8 ? 1 : 2);
        const size_t out_bytes = (size_t)N * OH * OW * this->output_channel_ * sizeof(float);
        grow(&x_nhwc_, &x_cap_, in_bytes);
        grow(&y_nhwc_, &y_cap_, out_bytes);
        // fp32 NCHW -> NHWC fp16 / int8 (the reference's quantisation: x * scale, half away from zero, saturate)
        const float fs = int8 ? this->featmap_scaletable_i8_->cpu_data()[0] : 1.f;
        check(exb_nchw_f32_to_nhwc(ctx_, x->gpu_data(), x_nhwc_, d.in_dtype, N, C, H, W, d.cin_stride, fs, 0, nullptr),
              "exb_nchw_f32_to_nhwc");
        check(exb_conv2d_fwd(ctx_, &d, x_nhwc_, packed_, nullptr, y_nhwc_, nullptr, nullptr), "exb_conv2d_fwd");
        check(exb_nhwc_to_nchw_f32(ctx_, y_nhwc_, EXB_F32, tops[0]->mutable_gpu_data(), N, this->output_channel_, OH, OW,
                                   this->output_channel_, 1.f, nullptr),
              "exb_nhwc_to_nchw_f32");
        check(exb_ctx_sync_check(ctx_, nullptr), "exb_ctx_sync_check");
    }

    static void grow(void** p, size_t* cap, size_t bytes) {
        if (bytes <= *cap) return;
        if (*p) cudaFree(*p);
        CUDA_CHECK(cudaMalloc(p, bytes));
        *cap = bytes;
    }

    exb_ctx* ctx_ = nullptr;
    exb_conv_weights* packed_ = nullptr;
    void* x_nhwc_ = nullptr;
    void* y_nhwc_ = nullptr;
    size_t x_cap_ = 0, y_cap_ = 0;
};

// compiled into libexcalibur after the stock classes: the same key, so this factory replaces the stock one
static register_action<float> g_b200_convolution("operation_convolution", [](const operation_param& p) {
    return std::shared_ptr<operation<float>>(new operation_convolution_b200<float>(p));
});

}  // namespace excalibur
}  // namespace glasssix
