// The operation classes on the CNN forward hot path, registered under the reference's keys
// (operation_convolution, operation_convolutiondepthwise, operation_pooling, operation_eltwise,
// operation_binaryop, operation_relu) plus the glue ops the benchmark graphs need
// (operation_split, operation_innerproduct, operation_input, operation_clip, operation_sigmoid).
// Constructors parse the same integer-keyed "k=v" lists; unknown keys are fatal; key -23330 is
// ignored (reference src/Excalibur/operation_general_conv.cpp:9-124, operation_pooling.cpp:10-77,
// operation_eltwise.cpp:11-40, operation_binaryop.cpp:369-391, operation_relu.cpp:9-28).
#pragma once
#include <cmath>
#include "operation.hpp"

namespace glasssix {
namespace excalibur {

// Raises LOG(FATAL) with the library's error string when a C-ABI call fails.
void exb_check(int rc, const char* what);

// Scratch device buffer that grows on demand (an op instance is not re-entrant, like the
// reference's member scratch tensors, include/Excalibur/operation_convolution.hpp:102-141).
class device_scratch {
public:
    ~device_scratch();
    void* get(size_t bytes, int device);
private:
    void* ptr_ = nullptr;
    size_t cap_ = 0;
};

template <typename Dtype>
class operation_general_conv : public operation<Dtype> {
public:
    explicit operation_general_conv(const operation_param& param);
    virtual const char* type() const { return this->params_.type_.c_str(); }

    int output_channel_ = 0, kernel_size_w_ = 0, kernel_size_h_ = 0, dilation_w_ = 1, dilation_h_ = 1;
    int stride_w_ = 1, stride_h_ = 1, group_ = 1, pad_left_ = 0, pad_right_ = 0, pad_top_ = 0, pad_bottom_ = 0;
    bool int8_scale_term_ = false, bias_term_ = false;
    int weight_data_size_ = 0, activation_type_ = 0, impl_type_ = 0;
    int input_channel_ = 0;   // known after init_weights: weight_data_size / (Cout/group * kh * kw) * ... 
};

template <typename Dtype>
class operation_convolution : public operation_general_conv<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_convolution(const operation_param& param);
    virtual ~operation_convolution();
    virtual int init_weights();
    virtual int init_weights(FILE* fp);

    // --- used by the fused executor ---------------------------------------------------------
    bool is_int8() const { return !this->weights_i8_.empty(); }
    int in_channels() const { return this->input_channel_; }
    float act_scale() const;                  // the conv's input quantisation multiplier (int8)
    // Packed weights for a given input layout; cached per (in_dtype, cin_stride, cout_stride).
    // post_mul / post_add (Cout entries each, or null): a per-channel affine map applied to the conv's
    // result, folded into the packed weights / epilogue constants (an inference BatchNorm behind the
    // conv: y = (conv + bias) * post_mul + post_add).  `tag` identifies the map in the cache.
    exb_conv_weights* packed(exb_ctx* ctx, const exb_conv_desc& d, const float* post_mul = nullptr,
                             const float* post_add = nullptr, const void* tag = nullptr);
    // Descriptor skeleton for an input of N x H x W (dtypes / fusion fields left to the caller).
    exb_conv_desc base_desc(int N, int H, int W) const;
    // Drop the fp32 host weights that only a CPU path would read (keeps bias and scales).
    int exb_activation() const;               // key 9 mapped to exb_act (fatal if unsupported)

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_i8(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
    void forward_nchw_f32(exb_ctx* h, const f32_list& bottoms, f32_list& tops, bool int8);

    struct packed_entry { int in_dtype, cin_stride, cout_stride, w_pitch, w_pad; exb_conv_weights* w; const void* tag; };
    std::vector<packed_entry> packed_;
    device_scratch scratch_in_, scratch_out_;
};

template <typename Dtype>
class operation_convolutiondepthwise : public operation_convolution<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_convolutiondepthwise(const operation_param& param);
    virtual ~operation_convolutiondepthwise();
    exb_dwconv_desc dw_desc(int N, int H, int W, int c_stride) const;
    exb_dw_weights* dw_packed(exb_ctx* ctx, const exb_dwconv_desc& d, const float* post_mul = nullptr,
                              const float* post_add = nullptr, const void* tag = nullptr);
    // fp32 [C][kh][kw] weights; int8 files are dequantised once, like the reference
    // (src/Excalibur/operation_convolutiondepthwise.cpp:184-222).
    const float* dw_weights_f32();

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_i8(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
    exb_dw_weights* dw_w_ = nullptr;
    int dw_cs_ = 0;
    const void* dw_tag_ = nullptr;
    std::vector<float> dequantized_;
};

template <typename Dtype>
class operation_pooling : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    enum pooling_type { MAX = 0, AVE = 1 };
    explicit operation_pooling(const operation_param& param);
    virtual const char* type() const { return "Pooling"; }
    exb_pool_desc desc(int N, int H, int W, int C, int c_stride, int dtype) const;

    int type_ = MAX, kernel_size_w_ = 0, kernel_size_h_ = 0, stride_w_ = 1, stride_h_ = 1;
    int pad_left_ = 0, pad_right_ = 0, pad_top_ = 0, pad_bottom_ = 0;
    bool global_pooling_ = false;
    int pad_mode_ = 1, avgpool_count_include_pad_ = 0;

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
    device_scratch scratch_in_, scratch_out_;
};

template <typename Dtype>
class operation_eltwise : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    enum eltwise_type { PROD = 0, SUM = 1, MAX = 2 };
    explicit operation_eltwise(const operation_param& param);
    virtual const char* type() const { return "Eltwise"; }
    int type_ = SUM;
    std::vector<float> coeffs_;

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
};

template <typename Dtype>
class operation_binaryop : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_binaryop(const operation_param& param);
    virtual const char* type() const { return "BinaryOp"; }
    int op_type_ = 0;
    int with_scalar_ = 0;
    float coef_ = 0.f;

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
};

template <typename Dtype>
class operation_relu : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_relu(const operation_param& param);
    virtual const char* type() const { return "ReLU"; }
    float slope_ = 0.f;   // parsed, unused (as in the reference)

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
};

// The reference's ReLU6 operation (src/Excalibur/operation_relu6.cpp:35-105): keys 0, 1 and -23330 are accepted and
// ignored, anything else is fatal; y = x for 0 <= x <= 6 and 0 elsewhere - values ABOVE 6 become 0, not 6 (the
// reference masks with x <= 6 instead of taking the minimum).  True ReLU6 is Clip 0=0 1=6.
template <typename Dtype>
class operation_relu6 : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_relu6(const operation_param& param);
    virtual const char* type() const { return "ReLU6"; }

protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    virtual void forward_gpu_f16(exb_ctx*& h, const f16_list& bottoms, f16_list& tops);
};

// ---- glue ops around the hot path -----------------------------------------------------------
template <typename Dtype>
class operation_split : public operation<Dtype> {   // aliases its input to every output
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    typedef typename operation<Dtype>::f16_list f16_list;
    explicit operation_split(const operation_param& param) : operation<Dtype>(param) {}
    virtual const char* type() const { return "Split"; }
protected:
    virtual void forward_gpu_f32(exb_ctx*&, const f32_list& bottoms, f32_list& tops) {
        CHECK_EQ(bottoms.size(), (size_t)1);
        for (auto& t : tops) t = bottoms[0];
    }
    virtual void forward_gpu_f16(exb_ctx*&, const f16_list& bottoms, f16_list& tops) {
        CHECK_EQ(bottoms.size(), (size_t)1);
        for (auto& t : tops) t = bottoms[0];
    }
};

template <typename Dtype>
class operation_clip : public operation<Dtype> {    // keys 0 = min, 1 = max
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_clip(const operation_param& param);
    virtual const char* type() const { return "Clip"; }
    float min_ = -3.402823466e+38f, max_ = 3.402823466e+38f;
    bool is_relu6() const { return min_ == 0.f && max_ == 6.f; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

template <typename Dtype>
class operation_sigmoid : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_sigmoid(const operation_param& param) : operation<Dtype>(param) {}
    virtual const char* type() const { return "Sigmoid"; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Fully connected layer: keys 0 num_output, 1 bias_term, 2 weight_data_size, 8 int8, 9 activation
// (reference src/Excalibur/operation_innerproduct.cpp:35-120).  Runs as a 1x1 convolution on a
// 1x1 map through the tensor-core kernel in fp16.
template <typename Dtype>
class operation_innerproduct : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_innerproduct(const operation_param& param);
    virtual ~operation_innerproduct();
    virtual const char* type() const { return "InnerProduct"; }
    virtual int init_weights();
    virtual int init_weights(FILE* fp);
    int num_output_ = 0, weight_data_size_ = 0, activation_type_ = 0;
    bool bias_term_ = false, int8_scale_term_ = false;
    int in_features() const { return num_output_ ? weight_data_size_ / num_output_ : 0; }
    exb_conv_desc fc_desc(int N, int cin_stride) const;
    exb_conv_weights* packed(exb_ctx* ctx, const exb_conv_desc& d);
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    exb_conv_weights* w_ = nullptr;
    int w_cin_stride_ = 0, w_cout_stride_ = 0;
    device_scratch scratch_in_, scratch_out_;
};

// Channel concatenation: key 0 = axis in the reference's ncnn-derived convention (axis + 2 indexes
// {N, C, H, W}, so -1 is the channel axis; reference src/Excalibur/operation_concat.cpp:10-46).
template <typename Dtype>
class operation_concat : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_concat(const operation_param& param);
    virtual const char* type() const { return "Concat"; }
    int axis_ = 0;
    bool is_channel_concat() const { return axis_ + 2 == 1; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Resize: keys 0 type (1 nearest, 2 bilinear), 1 / 2 width / height scale, 3 / 4 output width /
// height, 6 align_corner (reference src/Excalibur/operation_interp.cpp:185-217).  Only the nearest
// mode without corner alignment is implemented.
template <typename Dtype>
class operation_interp : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_interp(const operation_param& param);
    virtual const char* type() const { return "Interp"; }
    int resize_type_ = 0, output_width_ = 0, output_height_ = 0, align_corner_ = 0;
    float width_scale_ = 1.f, height_scale_ = 1.f;
    void out_dims(int H, int W, int* OH, int* OW) const;
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Inference batch norm: keys 0 channels, 1 eps; weights in file order slope, mean, var, bias with
// no quantize tag (reference src/Excalibur/operation_batchnorm.cpp:10-69).  y = b * x + a with
// b = slope / sqrt(var + eps), a = bias - slope * mean / sqrt(var + eps).
template <typename Dtype>
class operation_batchnorm : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_batchnorm(const operation_param& param);
    virtual const char* type() const { return "BatchNorm"; }
    virtual int init_weights();
    virtual int init_weights(FILE* fp);
    int channels_ = 0;
    float eps_ = 0.f;
    const std::shared_ptr<memory::tensor<float>>& mul() const { return b_; }
    const std::shared_ptr<memory::tensor<float>>& add() const { return a_; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    void derive();
    std::shared_ptr<memory::tensor<float>> a_, b_;
};

// y = x * clamp(alpha*x + beta, 0, 1): keys 0 alpha, 1 beta (reference
// src/Excalibur/operation_hardswish.cpp:9-28).
template <typename Dtype>
class operation_hardswish : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_hardswish(const operation_param& param);
    virtual const char* type() const { return "HardSwish"; }
    float alpha_ = 0.f, beta_ = 0.f;
    // the constants of the activation code EXB_ACT_HARDSWISH
    bool is_standard() const { return std::fabs(alpha_ - 1.f / 6.f) < 1e-6f && beta_ == 0.5f; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Network input normalisation y = (x - mean[c]) * var[c]: keys 0 w, 1 h, 2 c, 3 mean list, 4 var list
// (reference src/Excalibur/operation_input.cpp:9-58); 1 or 3 channels.
template <typename Dtype>
class operation_input : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_input(const operation_param& param);
    virtual const char* type() const { return "Input"; }
    int w_ = 0, h_ = 0, c_ = 0;
    std::vector<float> means_, vars_;
    // y = x * mul[c] + add[c] with mul = var, add = -mean * var; device arrays of `channels` entries
    void coefficients(int channels, const float** mul, const float** add);
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    std::shared_ptr<memory::tensor<float>> mul_, add_;
};

// Space-to-depth 2x2 of YOLOv5's Focus layer, no parameters (reference
// src/Excalibur/operation_yolov5focus.cpp:16-47); every image of the batch is converted.
template <typename Dtype>
class operation_yolov5focus : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_yolov5focus(const operation_param& param) : operation<Dtype>(param) {}
    virtual const char* type() const { return "YoloV5Focus"; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// y = x >= 0 ? x : slope[c] * x: key 0 = number of slopes (1 = shared by all channels); weights are the
// slopes, no quantize tag (reference src/Excalibur/operation_prelu.cpp:10-56).
template <typename Dtype>
class operation_prelu : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_prelu(const operation_param& param);
    virtual const char* type() const { return "PReLU"; }
    virtual int init_weights();
    virtual int init_weights(FILE* fp);
    int num_slope_ = 0;
    const float* slopes_gpu() const { return this->weights_f32_[0]->gpu_data(); }
    const float* slopes_cpu() const { return this->weights_f32_[0]->cpu_data(); }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// y = x < 0 ? alpha * x : x: key 0 = alpha (reference src/Excalibur/operation_leakyrelu.cpp:12-58).
template <typename Dtype>
class operation_leakyrelu : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_leakyrelu(const operation_param& param);
    virtual const char* type() const { return "LeakyRelu"; }
    float alpha_ = 0.f;
    const float* slope_gpu();      // one-element device array holding alpha
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    std::shared_ptr<memory::tensor<float>> slope_;
};

// Transposed convolution, fp32 weights [Cin][Cout][kh][kw] behind a quantize tag of 0 (reference
// src/Excalibur/operation_deconvolution.cpp:14-41): out[co][ih*s + a][iw*s + b] += sum_ci W[ci][co][a][b] *
// in[ci][ih][iw], output (H-1)*s + k - pads (:83-150).  Implemented for kernel == stride, no padding, one
// group - taps never overlap, so it is a 1x1 convolution to kh*kw*Cout channels (tensor cores) followed by
// a depth-to-space copy; other shapes are refused.
template <typename Dtype>
class operation_deconvolution : public operation_general_conv<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_deconvolution(const operation_param& param);
    virtual ~operation_deconvolution();
    virtual int init_weights();
    virtual int init_weights(FILE* fp);
    bool supported() const;
    int in_channels() const { return this->input_channel_; }
    // the 1x1 convolution to kh*kw*Cout channels; cout_stride is left to the caller
    exb_conv_desc inner_desc(int N, int H, int W, int cin_stride) const;
    // packed weights of that convolution (output channel (a*kw + b)*Cout + co), with an optional per-output-
    // channel affine map (Cout entries) folded in as operation_convolution::packed does
    exb_conv_weights* packed(exb_ctx* ctx, const exb_conv_desc& d, const float* post_mul = nullptr,
                             const float* post_add = nullptr, const void* tag = nullptr);
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
    struct entry { int cin_stride, cout_stride; exb_conv_weights* w; const void* tag; };
    std::vector<entry> packed_;
    device_scratch scratch_in_, scratch_mid_, scratch_out_;
};

// y = max(0, min(1, alpha*x + beta)): keys 0 alpha, 1 beta (reference src/Excalibur/operation_hardsigmoid.cpp:12-46).
template <typename Dtype>
class operation_hardsigmoid : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_hardsigmoid(const operation_param& param);
    virtual const char* type() const { return "HardSigmoid"; }
    float alpha_ = 0.f, beta_ = 0.f;
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Softmax over the channel axis: key 0 = axis (0, the channels of an NCHW tensor without its batch axis, is the
// only one implemented), key 1 ignored as in the reference (src/Excalibur/operation_softmax.cpp:10-96).
template <typename Dtype>
class operation_softmax : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_softmax(const operation_param& param);
    virtual const char* type() const { return "Softmax"; }
    int axis_ = 0;
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Same values, shape {n, 1, h, w} with (h, w) = (c*h*w, 1), (c*h, w), (c, h*w) or (1, c*h*w) for key 0 = axis
// 0..3, default 1 (reference src/Excalibur/operation_flatten.cpp:10-63).
template <typename Dtype>
class operation_flatten : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_flatten(const operation_param& param);
    virtual const char* type() const { return "Flatten"; }
    int axis_ = 1;
    std::vector<int> out_shape(const std::vector<int>& in) const;
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// View of the same NCHW data with another shape: keys 0 w, 1 h, 2 c (0 keeps, -1 deduces; n is kept;
// reference src/Excalibur/operation_reshape.cpp:10-84).
template <typename Dtype>
class operation_reshape : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_reshape(const operation_param& param);
    virtual const char* type() const { return "Reshape"; }
    int w_ = 0, h_ = 0, c_ = 0, permute_ = 0;
    // {n, c, h, w} of the result for an NCHW input of that shape
    std::vector<int> out_shape(const std::vector<int>& in) const;
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

// Axis permutation of the (h, w, c) axes: key 0 = list.  The identity and 1,0,2 (swap h and w in every
// channel plane: out[n][c][w][h] = in[n][c][h][w], reference src/Excalibur/operation_transpose.cpp:39-66)
// are implemented; the other permutations are refused.
template <typename Dtype>
class operation_transpose : public operation<Dtype> {
public:
    typedef typename operation<Dtype>::f32_list f32_list;
    explicit operation_transpose(const operation_param& param);
    virtual const char* type() const { return "Transpose"; }
    std::vector<int> perms_;
    bool is_identity() const { return perms_.size() == 3 && perms_[0] == 0 && perms_[1] == 1 && perms_[2] == 2; }
    bool is_swap_hw() const { return perms_.size() == 3 && perms_[0] == 1 && perms_[1] == 0 && perms_[2] == 2; }
protected:
    virtual void forward_gpu_f32(exb_ctx*& h, const f32_list& bottoms, f32_list& tops);
};

}  // namespace excalibur
}  // namespace glasssix
