// Host-side mirror of the reference's Primitives layer for the CNN forward path: logging /
// CHECK macros, the lazily synchronised host+device buffer, the host pool allocator and the
// 4-D tensor.  Same names, argument meaning and error behaviour as the reference
// (include/Primitives/logger.hpp:101-204, syncedmem.hpp:10-49, pool_allocator.hpp:22-159,
// tensor.hpp:15-173), written from scratch on top of the CUDA runtime.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>
#include <cstdlib>
#include <cstring>
#include <exception>
#include <iostream>
#include <list>
#include <memory>
#include <mutex>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#if defined(__GNUC__)
#define EXB_HOST_API __attribute__((visibility("default")))
#else
#define EXB_HOST_API
#endif

namespace glasssix {

enum class log_level { INFO, WARNING, ERROR, FATAL };

// What LOG(FATAL) / a failed CHECK does after printing.  The reference terminates the process
// (logger.hpp:101-118); that stays the default.  A host program that wants to survive (the C
// entry points used by the Python harness do) installs a handler that throws fatal_error.
struct fatal_error : std::runtime_error {
    using std::runtime_error::runtime_error;
};
typedef void (*fatal_handler_t)(const std::string& message);
EXB_HOST_API void set_fatal_handler(fatal_handler_t h);
EXB_HOST_API fatal_handler_t get_fatal_handler();
EXB_HOST_API void set_log_quiet(bool quiet);   // suppress INFO/WARNING lines
EXB_HOST_API bool log_quiet();

class log_line {
public:
    log_line(const char* file, int line, log_level level) : level_(level) {
        static const char* names[] = {"INFO", "WARNING", "ERROR", "FATAL"};
        os_ << "[" << names[(int)level] << " " << (file ? file : "?") << ":" << line << "] ";
    }
    ~log_line() noexcept(false) {
        if (level_ == log_level::FATAL) {
            std::string msg = os_.str();
            std::cerr << msg << std::endl;
            fatal_handler_t h = get_fatal_handler();
            if (h) h(msg);       // may throw
            std::terminate();    // reference behaviour
        }
        if (!log_quiet() || level_ == log_level::ERROR) std::cout << os_.str() << std::endl;
    }
    std::ostringstream& stream() { return os_; }

private:
    log_level level_;
    std::ostringstream os_;
};

}  // namespace glasssix

#define LOG(level) ::glasssix::log_line(__FILE__, __LINE__, ::glasssix::log_level::level).stream()
#define LOG_IF(level, condition) if (condition) LOG(level)
#define CHECK(a) if (!(a)) LOG(FATAL) << "Check failed: " #a " "
#define CHECK_BINARY_OP(op, a, b) if (!((a)op(b))) LOG(FATAL) << "Check failed: " #a " " #op " " #b " (" << (a) << " vs " << (b) << ") "
#define CHECK_LT(x, y) CHECK_BINARY_OP(<, x, y)
#define CHECK_GT(x, y) CHECK_BINARY_OP(>, x, y)
#define CHECK_LE(x, y) CHECK_BINARY_OP(<=, x, y)
#define CHECK_GE(x, y) CHECK_BINARY_OP(>=, x, y)
#define CHECK_EQ(x, y) CHECK_BINARY_OP(==, x, y)
#define CHECK_NE(x, y) CHECK_BINARY_OP(!=, x, y)
#define NOT_IMPLEMENTED LOG(FATAL) << "Not Implemented Yet."
#define NO_GPU LOG(FATAL) << "Cannot use GPU in CPU-only Mode: check mode."
// This library has no CPU compute path at all: calling one is a fatal error, never a fallback.
#define NO_CPU LOG(FATAL) << "This build contains only the sm_100a GPU path: construct the operation with device >= 0."
#define CUDA_CHECK(expr)                                                                      \
    do {                                                                                      \
        cudaError_t e__ = (expr);                                                             \
        if (e__ != cudaSuccess) LOG(FATAL) << #expr << ": " << cudaGetErrorString(e__);       \
    } while (0)
#define DISABLE_COPY_AND_ASSIGN(classname) \
    classname(const classname&) = delete;  \
    classname& operator=(const classname&) = delete

namespace glasssix {
namespace memory {

// Recycling allocator for host buffers with the reference's interface (include/Primitives/pool_allocator.hpp:72-146):
// fastMalloc(bytes, device_id) serves a request from the free list ("budgets") when a buffer of
// size_compare_ratio..100 % fit exists (default 75 %), else allocates - page-locked memory bound to device_id when
// device_id >= 0, 64-byte aligned heap memory otherwise; fastFree(ptr, device_id) moves a buffer from the handed-out
// list ("payouts") back to the free list, and frees a pointer it never handed out after logging an error.
// The two lists have a mutex each and no call ever holds both, so allocating and freeing threads cannot deadlock.
// One deliberate difference: every entry remembers the kind of memory it is (the device id it was pinned for), a
// request only reuses buffers of its own kind and clear() frees each buffer with the matching call; the reference
// keeps one untyped list, so a pinned buffer can come back for a heap request and is then freed as heap memory.
template <typename Object>
class pool_allocator {
public:
    pool_allocator() : ratio_(192) {}   // 0.75 * 256
    ~pool_allocator() {
        clear();
        std::lock_guard<std::mutex> g(payout_lock_);
        for (auto& p : payouts_) LOG(ERROR) << "pool allocator destroyed too early: " << p.ptr << " still in use";
    }
    // ratio in 0..1: how much of a free buffer a request must fill to reuse it
    void set_size_compare_ratio(float r) {
        if (r < 0.f || r > 1.f) {
            LOG(FATAL) << "invalid size compare ratio " << r;
            return;
        }
        ratio_ = (unsigned)(r * 256);
    }
    // release every free buffer now
    void clear() {
        std::list<entry> drop;
        {
            std::lock_guard<std::mutex> g(budget_lock_);
            drop.swap(budgets_);
        }
        for (auto& b : drop) release(b.ptr, b.device);
    }
    void* fastMalloc(size_t size, int device_id = -1) {
        entry e{0, nullptr, device_id};
        {
            std::lock_guard<std::mutex> g(budget_lock_);
            for (auto it = budgets_.begin(); it != budgets_.end(); ++it) {
                if (it->device == device_id && it->size >= size && ((it->size * ratio_) >> 8) <= size) {
                    e = *it;
                    budgets_.erase(it);
                    break;
                }
            }
        }
        if (!e.ptr) {
            e.size = size;
            if (device_id >= 0) {
                CUDA_CHECK(cudaSetDevice(device_id));
                CUDA_CHECK(cudaMallocHost(&e.ptr, size ? size : 16));
            } else if (posix_memalign(&e.ptr, 64, size ? size : 64) != 0) {
                LOG(FATAL) << "out of host memory (" << size << " bytes)";
            }
        }
        std::lock_guard<std::mutex> g(payout_lock_);
        payouts_.push_back(e);
        return e.ptr;
    }
    void fastFree(void* ptr, int device_id = -1) {
        entry e{0, nullptr, device_id};
        {
            std::lock_guard<std::mutex> g(payout_lock_);
            for (auto it = payouts_.begin(); it != payouts_.end(); ++it) {
                if (it->ptr == ptr) {
                    e = *it;
                    payouts_.erase(it);
                    break;
                }
            }
        }
        if (e.ptr) {
            std::lock_guard<std::mutex> g(budget_lock_);
            budgets_.push_back(e);
            return;
        }
        LOG(ERROR) << "pool allocator get wild " << ptr;
        release(ptr, device_id);
    }
    // buffers on the free list / handed out (tests and diagnostics)
    size_t budget_count() {
        std::lock_guard<std::mutex> g(budget_lock_);
        return budgets_.size();
    }
    size_t payout_count() {
        std::lock_guard<std::mutex> g(payout_lock_);
        return payouts_.size();
    }

private:
    struct entry {
        size_t size;
        void* ptr;
        int device;
    };
    static void release(void* ptr, int device) {
        if (device >= 0) CUDA_CHECK(cudaFreeHost(ptr));
        else std::free(ptr);
    }
    unsigned ratio_;   // 0..256
    std::mutex budget_lock_, payout_lock_;
    std::list<entry> budgets_, payouts_;
};

// Host + device copies of one buffer with a head state: data lives where it was last written
// and is copied (synchronously, like the reference's syncedmem.cpp:176-276) on first read from
// the other side.  Device memory is used only when device >= 0; host memory is pinned then.
template <typename Dtype>
class syncedmem {
public:
    enum SyncedHead { UNINITIALIZED, HEAD_AT_CPU, HEAD_AT_GPU, SYNCED };
    syncedmem() : syncedmem(0, -1) {}
    explicit syncedmem(size_t size, int device = -1)
        : cpu_ptr_(nullptr), gpu_ptr_(nullptr), allocator_(nullptr), size_(size), head_(UNINITIALIZED),
          own_cpu_(false), pinned_(false), device_(device) {}
    ~syncedmem() {
        if (cpu_ptr_ && own_cpu_) {   // as the reference's destructor (src/Primitives/syncedmem.cpp:57-80)
            if (allocator_) allocator_->fastFree(cpu_ptr_, device_);
            else if (pinned_) cudaFreeHost(cpu_ptr_);
            else std::free(cpu_ptr_);
        }
        if (gpu_ptr_) cudaFree(gpu_ptr_);
    }
    SyncedHead head() const { return head_; }
    size_t size() const { return size_; }
    void set_allocator(pool_allocator<Dtype>* a) { if (!cpu_ptr_) allocator_ = a; }
    const Dtype* cpu_data() { to_cpu(); return cpu_ptr_; }
    const Dtype* gpu_data() { to_gpu(); return gpu_ptr_; }
    Dtype* mutable_cpu_data() { to_cpu(); head_ = HEAD_AT_CPU; return cpu_ptr_; }
    Dtype* mutable_gpu_data() { to_gpu(); head_ = HEAD_AT_GPU; return gpu_ptr_; }
    // Adopt caller-owned host memory (pinned or not) as the CPU side, without copying.
    void set_external_cpu_data(Dtype* p) {
        CHECK(cpu_ptr_ == nullptr) << "buffer already has host storage";
        cpu_ptr_ = p; own_cpu_ = false; head_ = HEAD_AT_CPU;
    }
    void async_gpu_push(const cudaStream_t& stream) {
        CHECK(head_ == HEAD_AT_CPU) << "async_gpu_push needs the head on the CPU";
        alloc_gpu();
        CUDA_CHECK(cudaMemcpyAsync(gpu_ptr_, cpu_ptr_, bytes(), cudaMemcpyHostToDevice, stream));
        head_ = SYNCED;
    }

private:
    size_t bytes() const { return size_ * sizeof(Dtype); }
    void alloc_cpu() {
        if (cpu_ptr_) return;
        if (allocator_) {   // the allocator hands out pinned memory itself when device_ >= 0 (syncedmem.cpp:182-201)
            cpu_ptr_ = static_cast<Dtype*>(allocator_->fastMalloc(bytes(), device_));
        } else if (device_ >= 0) {
            CUDA_CHECK(cudaSetDevice(device_));
            CUDA_CHECK(cudaMallocHost(reinterpret_cast<void**>(&cpu_ptr_), bytes() ? bytes() : 16));
            pinned_ = true;
        } else {
            void* p = nullptr;
            if (posix_memalign(&p, 64, bytes() ? bytes() : 64) != 0) LOG(FATAL) << "out of host memory";
            cpu_ptr_ = static_cast<Dtype*>(p);
        }
        own_cpu_ = true;
    }
    void alloc_gpu() {
        if (gpu_ptr_) return;
        if (device_ < 0) NO_GPU;
        CUDA_CHECK(cudaSetDevice(device_));
        CUDA_CHECK(cudaMalloc(reinterpret_cast<void**>(&gpu_ptr_), bytes() ? bytes() : 16));
    }
    void to_cpu() {
        switch (head_) {
        case UNINITIALIZED:
            alloc_cpu();
            std::memset(cpu_ptr_, 0, bytes());
            head_ = HEAD_AT_CPU;
            break;
        case HEAD_AT_GPU:
            alloc_cpu();
            CUDA_CHECK(cudaMemcpy(cpu_ptr_, gpu_ptr_, bytes(), cudaMemcpyDeviceToHost));
            head_ = SYNCED;
            break;
        default: break;
        }
    }
    void to_gpu() {
        switch (head_) {
        case UNINITIALIZED:
            alloc_gpu();
            CUDA_CHECK(cudaMemset(gpu_ptr_, 0, bytes()));
            head_ = HEAD_AT_GPU;
            break;
        case HEAD_AT_CPU:
            alloc_gpu();
            CUDA_CHECK(cudaMemcpy(gpu_ptr_, cpu_ptr_, bytes(), cudaMemcpyHostToDevice));
            head_ = SYNCED;
            break;
        default: break;
        }
    }
    Dtype* cpu_ptr_;
    Dtype* gpu_ptr_;
    pool_allocator<Dtype>* allocator_;
    size_t size_;
    SyncedHead head_;
    bool own_cpu_, pinned_;
    int device_;
    DISABLE_COPY_AND_ASSIGN(syncedmem);
};

enum orderType { NCHW, NHWC };

// Dense 4-D tensor {N,C,H,W} or {N,H,W,C}; lower-rank constructors fill leading 1s.
template <typename Dtype>
class tensor {
public:
    explicit tensor(orderType order = NCHW, pool_allocator<Dtype>* allocator = nullptr)
        : allocator_(allocator), shape_{0, 0, 0, 0}, device_(-1), order_(order) {}
    explicit tensor(const int w, int device = -1, orderType order = NCHW, pool_allocator<Dtype>* a = nullptr)
        : tensor(std::vector<int>{1, 1, 1, w}, device, order, a) {}
    explicit tensor(const int h, const int w, int device = -1, orderType order = NCHW, pool_allocator<Dtype>* a = nullptr)
        : tensor(order == NCHW ? std::vector<int>{1, 1, h, w} : std::vector<int>{1, h, w, 1}, device, order, a) {}
    explicit tensor(const int c, const int h, const int w, int device = -1, orderType order = NCHW,
                    pool_allocator<Dtype>* a = nullptr)
        : tensor(order == NCHW ? std::vector<int>{1, c, h, w} : std::vector<int>{1, h, w, c}, device, order, a) {}
    explicit tensor(const std::vector<int>& shape, int device = -1, orderType order = NCHW,
                    pool_allocator<Dtype>* a = nullptr)
        : allocator_(a), shape_(shape), device_(device), order_(order) {
        while (shape_.size() < 4) shape_.insert(shape_.begin(), 1);
        CHECK_EQ(shape_.size(), (size_t)4) << "tensors are 4-dimensional";
        data_.reset(new syncedmem<Dtype>((size_t)count(), device));
        data_->set_allocator(a);
    }
    // Shallow copies share the buffer, like the reference's copy constructor.
    tensor(const tensor&) = default;
    tensor& operator=(const tensor&) = default;

    tensor clone() const {
        tensor t(shape_, device_, order_, allocator_);
        if (count()) std::memcpy(t.mutable_cpu_data(), cpu_data(), sizeof(Dtype) * (size_t)count());
        return t;
    }
    bool empty() const { return data_ == nullptr || count() == 0; }
    const Dtype* cpu_data() const { return data_->cpu_data(); }
    const Dtype* gpu_data() const { return data_->gpu_data(); }
    Dtype* mutable_cpu_data() const { return data_->mutable_cpu_data(); }
    Dtype* mutable_gpu_data() const { return data_->mutable_gpu_data(); }
    std::shared_ptr<syncedmem<Dtype>> data() const { return data_; }
    void fill(Dtype v) {
        Dtype* p = mutable_cpu_data();
        for (int i = 0; i < count(); ++i) p[i] = v;
    }
    void copy_from(const void* src, size_t bytes) {
        CHECK_LE(bytes, sizeof(Dtype) * (size_t)count());
        std::memcpy(mutable_cpu_data(), src, bytes);
    }
    // NHWC -> NCHW on the host (the only direction the reference implements, tensor.cpp:334-377).
    void convert_order() {
        if (order_ != NHWC) return;
        const int n = num(), c = channels(), h = height(), w = width();
        std::vector<Dtype> tmp((size_t)count());
        const Dtype* src = cpu_data();
        for (int in = 0; in < n; ++in)
            for (int ih = 0; ih < h; ++ih)
                for (int iw = 0; iw < w; ++iw)
                    for (int ic = 0; ic < c; ++ic)
                        tmp[(((size_t)in * c + ic) * h + ih) * w + iw] = src[(((size_t)in * h + ih) * w + iw) * c + ic];
        std::memcpy(mutable_cpu_data(), tmp.data(), sizeof(Dtype) * tmp.size());
        shape_ = {n, c, h, w};
        order_ = NCHW;
    }
    int num() const { return shape_[0]; }
    int channels() const { return order_ == NCHW ? shape_[1] : shape_[3]; }
    int height() const { return order_ == NCHW ? shape_[2] : shape_[1]; }
    int width() const { return order_ == NCHW ? shape_[3] : shape_[2]; }
    int count(int start_axis, int end_axis) const {
        int c = 1;
        for (int i = start_axis; i < end_axis; ++i) c *= shape_[i];
        return c;
    }
    int count() const { return count(0, (int)shape_.size()); }
    int device() const { return device_; }
    orderType order() const { return order_; }
    int offset(const int n, const int c = 0, const int h = 0, const int w = 0) const {
        return order_ == NCHW ? ((n * channels() + c) * height() + h) * width() + w
                              : ((n * height() + h) * width() + w) * channels() + c;
    }
    std::vector<int> data_shape() const { return shape_; }
    void reshape(std::vector<int> s) { shape_ = s; }
    void set_allocator(pool_allocator<Dtype>* a) { if (!allocator_) allocator_ = a; }
    pool_allocator<Dtype>* allocator() const { return allocator_; }
    Dtype& operator[](size_t i) { return mutable_cpu_data()[i]; }
    const Dtype& operator[](size_t i) const { return cpu_data()[i]; }

private:
    std::shared_ptr<syncedmem<Dtype>> data_;
    pool_allocator<Dtype>* allocator_;
    std::vector<int> shape_;
    int device_;
    orderType order_;
};

}  // namespace memory
}  // namespace glasssix
