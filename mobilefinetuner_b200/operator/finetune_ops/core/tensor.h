// ops::Tensor with device-resident storage.
//
// Same public surface as the reference's core/tensor.h (constructors, shape /
// dtype accessors, raw host access through data<T>() / data_ptr(), autograd
// hooks, factories), so code written against the reference compiles unchanged.
// Underneath, every tensor owns a host buffer AND (lazily) a device buffer from
// the caching allocator of libmft_cuda.so, with a validity state:
//   - ops:: kernels read/write the device copy (uploading a stale one first);
//   - `const` host accessors bring the host copy up to date and keep both valid;
//   - non-const host accessors additionally mark the device copy stale, so a
//     caller may write through the pointer and the next kernel sees the change;
//     because the caller may KEEP that pointer and write again later (the
//     reference's finite-difference tests do), a tensor whose mutable pointer
//     has been handed out is re-uploaded before every kernel that reads it,
//     until a kernel overwrites it.
// Host-visible reads therefore always observe program-order results.
#pragma once

#include <cassert>
#include <cstdint>
#include <exception>
#include <functional>
#include <initializer_list>
#include <iostream>      // callers written against the reference's header count on <iostream> / <stdexcept> arriving with it
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "types.h"

namespace ops {

class Tensor;
using TensorPtr = std::shared_ptr<Tensor>;
using GradFn = std::function<std::vector<TensorPtr>(const TensorPtr&)>;

namespace autograd {
class Node;
class Engine;
using NodePtr = std::shared_ptr<Node>;
}  // namespace autograd

// A value that is computed on first use.  A tensor built by Tensor::make_deferred has a shape and a dtype but no
// storage; the first host or device access calls materialize(), which must fill the device copy through
// Tensor::device_write().  Consumers that can do better than the dense value (lm_cross_entropy on a model's
// logits) look at deferred() first and never trigger it.
class Deferred {
public:
    virtual ~Deferred() = default;
    virtual void materialize(Tensor& into) = 0;
};

class TensorError : public std::exception {
public:
    explicit TensorError(const std::string& msg) : message_(msg) {}
    const char* what() const noexcept override { return message_.c_str(); }
private:
    std::string message_;
};

class Tensor : public std::enable_shared_from_this<Tensor> {
public:
    Tensor() = default;
    Tensor(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
    Tensor(const std::vector<int64_t>& shape, const void* data, DType dtype = kFloat32, Device device = kCPU);
    // wraps caller-owned host memory (no copy, never freed here)
    Tensor(const std::vector<int64_t>& shape, void* external_data, DType dtype, Device device, bool wrap_external_flag);
    Tensor(const Tensor& other);
    Tensor& operator=(const Tensor& other);
    Tensor(Tensor&& other) noexcept;
    Tensor& operator=(Tensor&& other) noexcept;
    ~Tensor();

    const std::vector<int64_t>& shape() const { return shape_; }
    int64_t size(int dim) const { return shape_[static_cast<size_t>(dim)]; }
    int64_t ndim() const { return static_cast<int64_t>(shape_.size()); }
    int64_t numel() const;
    DType dtype() const { return dtype_; }
    Device device() const { return device_; }

    // ---- host access (see the coherence rules above)
    void* data_ptr() { return host_rw(); }
    const void* data_ptr() const { return host_ro(); }
    template <typename T> T* data() { return static_cast<T*>(host_rw()); }
    template <typename T> const T* data() const { return static_cast<const T*>(host_ro()); }
    template <typename T> T& item() { assert(numel() == 1); return *static_cast<T*>(host_rw()); }
    template <typename T> const T& item() const { assert(numel() == 1); return *static_cast<const T*>(host_ro()); }
    float item() const;

    // ---- device access for kernels (not part of the reference's surface)
    const void* device_read() const;     // valid device copy, uploaded if stale
    void* device_write();                // device copy about to be fully overwritten: host copy becomes stale
    void* device_readwrite();            // valid device copy that a kernel will modify
    size_t nbytes() const { return bytes_; }
    // Makes `dev` (caller-owned device memory of nbytes(), e.g. a slice of a flat parameter bucket) this tensor's
    // device copy.  The current value moves there; from then on kernels that read or update the tensor work on
    // that memory directly.  unbind_device() brings the value back into storage the tensor owns.
    void bind_device(void* dev);
    void unbind_device();
    const void* bound_device() const { return owns_dev_ ? nullptr : dev_; }
    // Counts the mutable host pointers handed out (every one may have been written through).
    uint64_t host_write_count() const { return host_writes_; }
    bool host_dirty() const { return host_escaped_ || !(valid_ & DEV_VALID); }
    // A tensor whose value is produced on first access.
    static TensorPtr make_deferred(const std::vector<int64_t>& shape, DType dtype, std::shared_ptr<Deferred> producer);
    const std::shared_ptr<Deferred>& deferred() const { return deferred_; }

    TensorPtr to(const Device& device) const;
    TensorPtr cpu() const { return to(kCPU); }
    TensorPtr cuda() const { return to(kCUDA); }

    TensorPtr reshape(const std::vector<int64_t>& new_shape) const;
    TensorPtr view(const std::vector<int64_t>& new_shape) const;
    TensorPtr squeeze(int dim = -1) const;
    TensorPtr unsqueeze(int dim) const;
    TensorPtr transpose(int dim0, int dim1) const;
    TensorPtr slice(int dim, int64_t start, int64_t end, int64_t step = 1) const;
    TensorPtr operator[](int64_t index) const;

    bool requires_grad() const { return requires_grad_; }
    void set_requires_grad(bool r) { requires_grad_ = r; }
    TensorPtr grad() const { return grad_; }
    void set_grad(const TensorPtr& g) { grad_ = g; }
    bool is_leaf() const { return grad_node_ == nullptr; }
    void backward(const TensorPtr& gradient = nullptr);
    void zero_grad();
    void set_grad_fn(const GradFn& fn) { grad_fn_ = fn; }
    void retain_grad() { retain_grad_ = true; }
    bool retains_grad() const { return retain_grad_; }

    TensorPtr clone() const;
    TensorPtr detach() const;
    void print() const;
    std::string to_string() const;

    TensorPtr operator+(const Tensor& other) const;
    TensorPtr operator-(const Tensor& other) const;
    TensorPtr operator*(const Tensor& other) const;
    TensorPtr operator/(const Tensor& other) const;
    TensorPtr operator+(float scalar) const;
    TensorPtr operator-(float scalar) const;
    TensorPtr operator*(float scalar) const;
    TensorPtr operator/(float scalar) const;

private:
    enum : uint8_t { HOST_VALID = 1, DEV_VALID = 2 };
    std::vector<int64_t> shape_;
    DType dtype_ = kFloat32;
    Device device_ = kCPU;
    mutable void* host_ = nullptr;
    mutable void* dev_ = nullptr;
    size_t bytes_ = 0;
    bool owns_host_ = true;
    bool owns_dev_ = true;
    uint64_t host_writes_ = 0;
    mutable std::shared_ptr<Deferred> deferred_;
    mutable uint8_t valid_ = HOST_VALID;
    bool host_escaped_ = false;      // a mutable host pointer is out: the device copy can go stale at any time

    bool requires_grad_ = false;
    TensorPtr grad_ = nullptr;
    GradFn grad_fn_ = nullptr;
    bool retain_grad_ = false;
    autograd::NodePtr grad_node_ = nullptr;

    void allocate_host();
    void release();
    void* host_rw();
    const void* host_ro() const;
    void sync_to_host() const;
    void materialize() const;
    void ensure_device() const;
    TensorPtr self() const;

    friend class autograd::Engine;
    friend class autograd::Node;
};

TensorPtr zeros(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr ones(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr randn(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr rand(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr empty(const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr full(const std::vector<int64_t>& shape, float value, DType dtype = kFloat32, Device device = kCPU);
TensorPtr from_blob(void* data, const std::vector<int64_t>& shape, DType dtype = kFloat32, Device device = kCPU);
TensorPtr tensor(const std::vector<float>& data, DType dtype = kFloat32, Device device = kCPU);
TensorPtr tensor(std::initializer_list<float> data, DType dtype = kFloat32, Device device = kCPU);
TensorPtr cast(const TensorPtr& tensor, DType dtype);

TensorPtr operator+(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator-(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator*(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator/(const TensorPtr& a, const TensorPtr& b);
TensorPtr operator+(const TensorPtr& t, float s);
TensorPtr operator-(const TensorPtr& t, float s);
TensorPtr operator*(const TensorPtr& t, float s);
TensorPtr operator/(const TensorPtr& t, float s);
TensorPtr operator+(float s, const TensorPtr& t);
TensorPtr operator-(float s, const TensorPtr& t);
TensorPtr operator*(float s, const TensorPtr& t);
TensorPtr operator/(float s, const TensorPtr& t);
std::ostream& operator<<(std::ostream& os, const Tensor& t);

// Internal helpers shared by the ops:: implementation files.
namespace detail {
void check(int32_t status, const char* what);          // throws TensorError with mft_last_error()
void* stream();                                        // the stream every ops:: kernel is launched on
void ensure_runtime();                                 // mft_init on first use; throws without a GPU
TensorPtr new_like(const std::vector<int64_t>& shape, DType dtype = kFloat32);
bool compute_bf16();                                   // the eager operators use the bf16 tensor-core kernels where they exist
TensorPtr to_bf16(const TensorPtr& t);                 // f32 -> bf16 copy on the device (a bf16 tensor is returned as it is)
TensorPtr bf16_to_f32(const TensorPtr& t, const std::vector<int64_t>& shape);
}  // namespace detail

}  // namespace ops
