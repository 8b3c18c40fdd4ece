// Storage, coherence and shape utilities of ops::Tensor (see tensor.h).
#include "tensor.h"

#include <cstdlib>
#include <cstring>
#include <iostream>
#include <numeric>
#include <random>
#include <sstream>

#include "mft_cuda.h"
#include "autograd_engine.h"
#include "ops.h"

namespace ops {

namespace detail {

void check(int32_t status, const char* what) {
    if (status != MFT_OK) throw TensorError(std::string(what) + ": " + mft_last_error());
}
void* stream() { return nullptr; }
void ensure_runtime() {
    static bool ready = false;
    if (ready) return;
    int dev = 0;
    if (const char* e = std::getenv("MFT_DEVICE")) dev = std::atoi(e);
    check(mft_init(dev), "mft_init");
    ready = true;
}
TensorPtr new_like(const std::vector<int64_t>& shape, DType dtype) { return std::make_shared<Tensor>(shape, dtype, kCPU); }

}  // namespace detail

static int64_t count(const std::vector<int64_t>& shape) {
    int64_t n = 1;
    for (auto d : shape) n *= d;
    return shape.empty() ? 1 : n;
}

int64_t Tensor::numel() const { return count(shape_); }

void Tensor::allocate_host() {
    bytes_ = static_cast<size_t>(numel()) * DTypeUtils::size_of(dtype_);
    host_ = std::calloc(bytes_ ? bytes_ : 1, 1);          // zero-initialised, as every reference factory guarantees
    if (!host_) throw TensorError("out of host memory");
    owns_host_ = true;
    valid_ = HOST_VALID;
}

void Tensor::release() {
    if (dev_ && owns_dev_) mft_free(dev_, detail::stream());
    dev_ = nullptr;
    owns_dev_ = true;
    deferred_.reset();
    if (host_ && owns_host_) std::free(host_);
    host_ = nullptr;
    bytes_ = 0;
}

Tensor::Tensor(const std::vector<int64_t>& shape, DType dtype, Device device) : shape_(shape), dtype_(dtype), device_(device) { allocate_host(); }

Tensor::Tensor(const std::vector<int64_t>& shape, const void* data, DType dtype, Device device) : shape_(shape), dtype_(dtype), device_(device) {
    allocate_host();
    if (data && bytes_) std::memcpy(host_, data, bytes_);
}

Tensor::Tensor(const std::vector<int64_t>& shape, void* external, DType dtype, Device device, bool wrap) : shape_(shape), dtype_(dtype), device_(device) {
    if (!wrap) {
        allocate_host();
        if (external && bytes_) std::memcpy(host_, external, bytes_);
        return;
    }
    bytes_ = static_cast<size_t>(numel()) * DTypeUtils::size_of(dtype_);
    host_ = external;
    owns_host_ = false;
    valid_ = HOST_VALID;
}

Tensor::Tensor(const Tensor& o) : shape_(o.shape_), dtype_(o.dtype_), device_(o.device_), requires_grad_(o.requires_grad_) {
    allocate_host();
    if (bytes_) std::memcpy(host_, o.host_ro(), bytes_);
}

Tensor& Tensor::operator=(const Tensor& o) {
    if (this == &o) return *this;
    release();
    shape_ = o.shape_; dtype_ = o.dtype_; device_ = o.device_; requires_grad_ = o.requires_grad_;
    grad_ = nullptr; grad_node_ = nullptr; grad_fn_ = nullptr;
    allocate_host();
    if (bytes_) std::memcpy(host_, o.host_ro(), bytes_);
    return *this;
}

Tensor::Tensor(Tensor&& o) noexcept { *this = std::move(o); }

Tensor& Tensor::operator=(Tensor&& o) noexcept {
    if (this == &o) return *this;
    release();
    shape_ = std::move(o.shape_); dtype_ = o.dtype_; device_ = o.device_;
    host_ = o.host_; dev_ = o.dev_; bytes_ = o.bytes_; owns_host_ = o.owns_host_; owns_dev_ = o.owns_dev_; valid_ = o.valid_;
    host_escaped_ = o.host_escaped_; host_writes_ = o.host_writes_; deferred_ = std::move(o.deferred_);
    requires_grad_ = o.requires_grad_; grad_ = std::move(o.grad_); grad_fn_ = std::move(o.grad_fn_);
    retain_grad_ = o.retain_grad_; grad_node_ = std::move(o.grad_node_);
    o.host_ = nullptr; o.dev_ = nullptr; o.bytes_ = 0; o.owns_dev_ = true;
    return *this;
}

Tensor::~Tensor() { release(); }

// ---------------------------------------------------------------- coherence
TensorPtr Tensor::make_deferred(const std::vector<int64_t>& shape, DType dtype, std::shared_ptr<Deferred> producer) {
    auto t = std::make_shared<Tensor>();
    t->shape_ = shape;
    t->dtype_ = dtype;
    t->bytes_ = static_cast<size_t>(t->numel()) * DTypeUtils::size_of(dtype);
    t->valid_ = 0;
    t->deferred_ = std::move(producer);
    return t;
}

void Tensor::materialize() const {
    if (!deferred_) return;
    std::shared_ptr<Deferred> p = std::move(deferred_);
    deferred_.reset();
    p->materialize(*const_cast<Tensor*>(this));          // fills the device copy
}

void Tensor::bind_device(void* dev) {
    if (!dev) throw TensorError("bind_device: null pointer");
    materialize();
    if (dev_ == dev) return;
    if (bytes_) {
        if ((valid_ & DEV_VALID) && dev_) detail::check(mft_memcpy_d2d(dev, dev_, bytes_, detail::stream()), "bind_device");
        else {
            detail::check(mft_memcpy_h2d(dev, host_, bytes_, detail::stream()), "bind_device upload");
            detail::check(mft_stream_sync(detail::stream()), "stream sync");
        }
    }
    if (dev_ && owns_dev_) mft_free(dev_, detail::stream());
    dev_ = dev;
    owns_dev_ = false;
    valid_ |= DEV_VALID;
}

void Tensor::unbind_device() {
    if (owns_dev_) return;
    sync_to_host();
    dev_ = nullptr;
    owns_dev_ = true;
    valid_ = HOST_VALID;
}

void Tensor::sync_to_host() const {
    materialize();
    if (!host_) {
        host_ = std::calloc(bytes_ ? bytes_ : 1, 1);
        if (!host_) throw TensorError("out of host memory");
    }
    if (valid_ & HOST_VALID) return;
    if (bytes_) detail::check(mft_memcpy_d2h(host_, dev_, bytes_, detail::stream()), "device -> host copy");
    valid_ |= HOST_VALID;
}

void Tensor::ensure_device() const {
    detail::ensure_runtime();
    materialize();
    if (!dev_) {
        void* p = nullptr;
        detail::check(mft_malloc(bytes_ ? bytes_ : 4, detail::stream(), &p), "mft_malloc");
        dev_ = p;
        valid_ &= ~DEV_VALID;
    }
    // a wrapped external buffer can change behind our back (dataset batches): always re-upload it
    if (!(valid_ & DEV_VALID) || !owns_host_ || host_escaped_) {
        if (bytes_) {
            detail::check(mft_memcpy_h2d(dev_, host_, bytes_, detail::stream()), "host -> device copy");
            detail::check(mft_stream_sync(detail::stream()), "stream sync");   // the host buffer may be pageable and reused at once
        }
        valid_ |= DEV_VALID;
    }
}

const void* Tensor::host_ro() const { sync_to_host(); return host_; }
void* Tensor::host_rw() { sync_to_host(); valid_ = HOST_VALID; host_escaped_ = true; ++host_writes_; return host_; }
const void* Tensor::device_read() const { ensure_device(); return dev_; }
void* Tensor::device_readwrite() { ensure_device(); valid_ = DEV_VALID; host_escaped_ = false; return dev_; }
void* Tensor::device_write() {
    detail::ensure_runtime();
    deferred_.reset();
    if (!dev_) {
        void* p = nullptr;
        detail::check(mft_malloc(bytes_ ? bytes_ : 4, detail::stream(), &p), "mft_malloc");
        dev_ = p;
    }
    valid_ = DEV_VALID;
    host_escaped_ = false;
    return dev_;
}

float Tensor::item() const {
    assert(numel() == 1);
    const void* p = host_ro();
    if (dtype_ == kFloat32) return *static_cast<const float*>(p);
    if (dtype_ == kFloat16) return fp16_bits_to_float32(*static_cast<const uint16_t*>(p));
    if (dtype_ == kBFloat16) return bf16_bits_to_float32(*static_cast<const uint16_t*>(p));
    if (dtype_ == kInt32) return static_cast<float>(*static_cast<const int32_t*>(p));
    return 0.0f;
}

TensorPtr Tensor::self() const {
    if (auto sp = const_cast<Tensor*>(this)->weak_from_this().lock()) return sp;
    return TensorPtr(const_cast<Tensor*>(this), [](Tensor*) {});
}

TensorPtr Tensor::to(const Device& device) const {
    // Residency is implicit: every tensor migrates to the GPU on first kernel use.  `to` only retags.
    auto r = clone();
    r->device_ = device;
    return r;
}

TensorPtr Tensor::clone() const {
    auto r = std::make_shared<Tensor>(shape_, dtype_, device_);
    if (bytes_) {
        if ((valid_ & DEV_VALID) && !(valid_ & HOST_VALID)) {
            detail::check(mft_memcpy_d2d(r->device_write(), dev_, bytes_, detail::stream()), "clone");
        } else {
            std::memcpy(r->host_, host_ro(), bytes_);
        }
    }
    r->requires_grad_ = requires_grad_;
    return r;
}

TensorPtr Tensor::detach() const {
    auto r = clone();
    r->requires_grad_ = false;
    return r;
}

TensorPtr Tensor::reshape(const std::vector<int64_t>& new_shape) const {
    std::vector<int64_t> shp = new_shape;
    int64_t known = 1, infer = -1;
    for (size_t i = 0; i < shp.size(); ++i) {
        if (shp[i] == -1) infer = (int64_t)i; else known *= shp[i];
    }
    if (infer >= 0) shp[(size_t)infer] = known ? numel() / known : 0;
    if (count(shp) != numel()) throw TensorError("reshape: element count mismatch");
    auto r = clone();
    r->shape_ = shp;
    return r;
}
TensorPtr Tensor::view(const std::vector<int64_t>& s) const { return reshape(s); }

TensorPtr Tensor::squeeze(int dim) const {
    std::vector<int64_t> shp;
    for (int i = 0; i < (int)shape_.size(); ++i) {
        const bool drop = shape_[i] == 1 && (dim < 0 ? true : i == dim);
        if (!drop) shp.push_back(shape_[i]);
    }
    return reshape(shp);
}
TensorPtr Tensor::unsqueeze(int dim) const {
    std::vector<int64_t> shp = shape_;
    if (dim < 0) dim += (int)shp.size() + 1;
    shp.insert(shp.begin() + dim, 1);
    return reshape(shp);
}
TensorPtr Tensor::transpose(int d0, int d1) const { return ops::transpose(self(), d0, d1); }

TensorPtr Tensor::operator[](int64_t index) const {
    auto s = slice(0, index, index + 1, 1);
    std::vector<int64_t> shp(shape_.begin() + 1, shape_.end());
    return s->reshape(shp.empty() ? std::vector<int64_t>{1} : shp);
}

void Tensor::backward(const TensorPtr& gradient) {
    if (!requires_grad_) return;
    std::vector<TensorPtr> grads;
    if (gradient) grads.push_back(gradient);
    autograd::Engine::instance().run_backward({self()}, grads);
}

void Tensor::zero_grad() {
    if (!grad_) return;
    if (grad_->valid_ & DEV_VALID) {
        detail::check(mft_memset(grad_->dev_, 0, grad_->bytes_, detail::stream()), "zero_grad");
        grad_->valid_ = DEV_VALID;
    } else {
        std::memset(grad_->host_, 0, grad_->bytes_);
    }
}

std::string Tensor::to_string() const {
    std::ostringstream os;
    os << "Tensor(shape=[";
    for (size_t i = 0; i < shape_.size(); ++i) os << (i ? ", " : "") << shape_[i];
    os << "], dtype=" << DTypeUtils::to_string(dtype_) << ", device=" << device_.to_string();
    if (dtype_ == kFloat32) {
        const float* p = data<float>();
        os << ", data=[";
        const int64_t n = std::min<int64_t>(numel(), 8);
        for (int64_t i = 0; i < n; ++i) os << (i ? ", " : "") << p[i];
        if (numel() > n) os << ", ...";
        os << "]";
    }
    os << ")";
    return os.str();
}
void Tensor::print() const { std::cout << to_string() << std::endl; }
std::ostream& operator<<(std::ostream& os, const Tensor& t) { return os << t.to_string(); }

// ---------------------------------------------------------------- factories
TensorPtr zeros(const std::vector<int64_t>& s, DType d, Device dev) { return std::make_shared<Tensor>(s, d, dev); }
TensorPtr empty(const std::vector<int64_t>& s, DType d, Device dev) { return std::make_shared<Tensor>(s, d, dev); }
TensorPtr full(const std::vector<int64_t>& s, float value, DType d, Device dev) {
    auto t = std::make_shared<Tensor>(s, d, dev);
    const int64_t n = t->numel();
    if (d == kFloat32) { float* p = t->data<float>(); for (int64_t i = 0; i < n; ++i) p[i] = value; }
    else if (d == kInt32) { int32_t* p = t->data<int32_t>(); for (int64_t i = 0; i < n; ++i) p[i] = (int32_t)value; }
    else if (d == kBFloat16) { uint16_t* p = t->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) p[i] = float32_to_bf16_bits(value); }
    else if (d == kFloat16) { uint16_t* p = t->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) p[i] = float32_to_fp16_bits(value); }
    else throw TensorError("full: unsupported dtype");
    return t;
}
TensorPtr ones(const std::vector<int64_t>& s, DType d, Device dev) { return full(s, 1.0f, d, dev); }
static std::mt19937& global_rng() { static std::mt19937 g(std::random_device{}()); return g; }
TensorPtr randn(const std::vector<int64_t>& s, DType d, Device dev) {
    if (d != kFloat32) throw TensorError("randn: float32 only");
    auto t = std::make_shared<Tensor>(s, d, dev);
    std::normal_distribution<float> dist(0.f, 1.f);
    float* p = t->data<float>();
    for (int64_t i = 0; i < t->numel(); ++i) p[i] = dist(global_rng());
    return t;
}
TensorPtr rand(const std::vector<int64_t>& s, DType d, Device dev) {
    if (d != kFloat32) throw TensorError("rand: float32 only");
    auto t = std::make_shared<Tensor>(s, d, dev);
    std::uniform_real_distribution<float> dist(0.f, 1.f);
    float* p = t->data<float>();
    for (int64_t i = 0; i < t->numel(); ++i) p[i] = dist(global_rng());
    return t;
}
TensorPtr from_blob(void* data, const std::vector<int64_t>& s, DType d, Device dev) { return std::make_shared<Tensor>(s, data, d, dev, true); }
TensorPtr tensor(const std::vector<float>& data, DType d, Device dev) {
    auto t = std::make_shared<Tensor>(std::vector<int64_t>{(int64_t)data.size()}, data.data(), kFloat32, dev);
    return d == kFloat32 ? t : cast(t, d);
}
TensorPtr tensor(std::initializer_list<float> data, DType d, Device dev) { return tensor(std::vector<float>(data), d, dev); }

TensorPtr cast(const TensorPtr& t, DType to) {
    if (t->dtype() == to) return t->clone();
    const int64_t n = t->numel();
    std::vector<float> tmp((size_t)n);
    const DType from = t->dtype();
    if (from == kFloat32) std::memcpy(tmp.data(), t->data<float>(), (size_t)n * 4);
    else if (from == kBFloat16) { const uint16_t* p = t->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) tmp[(size_t)i] = bf16_bits_to_float32(p[i]); }
    else if (from == kFloat16) { const uint16_t* p = t->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) tmp[(size_t)i] = fp16_bits_to_float32(p[i]); }
    else if (from == kInt32) { const int32_t* p = t->data<int32_t>(); for (int64_t i = 0; i < n; ++i) tmp[(size_t)i] = (float)p[i]; }
    else throw TensorError("cast: unsupported source dtype");
    auto r = std::make_shared<Tensor>(t->shape(), to, t->device());
    if (to == kFloat32) std::memcpy(r->data<float>(), tmp.data(), (size_t)n * 4);
    else if (to == kBFloat16) { uint16_t* p = r->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) p[i] = float32_to_bf16_bits(tmp[(size_t)i]); }
    else if (to == kFloat16) { uint16_t* p = r->data<uint16_t>(); for (int64_t i = 0; i < n; ++i) p[i] = float32_to_fp16_bits(tmp[(size_t)i]); }
    else if (to == kInt32) { int32_t* p = r->data<int32_t>(); for (int64_t i = 0; i < n; ++i) p[i] = (int32_t)tmp[(size_t)i]; }
    else throw TensorError("cast: unsupported target dtype");
    return r;
}

// ---------------------------------------------------------------- operators
TensorPtr Tensor::operator+(const Tensor& o) const { return ops::add(self(), o.self()); }
TensorPtr Tensor::operator-(const Tensor& o) const { return ops::sub(self(), o.self()); }
TensorPtr Tensor::operator*(const Tensor& o) const { return ops::mul(self(), o.self()); }
TensorPtr Tensor::operator/(const Tensor& o) const { return ops::div(self(), o.self()); }
TensorPtr Tensor::operator+(float s) const { return ops::add(self(), s); }
TensorPtr Tensor::operator-(float s) const { return ops::sub(self(), s); }
TensorPtr Tensor::operator*(float s) const { return ops::mul(self(), s); }
TensorPtr Tensor::operator/(float s) const { return ops::div(self(), s); }
TensorPtr operator+(const TensorPtr& a, const TensorPtr& b) { return ops::add(a, b); }
TensorPtr operator-(const TensorPtr& a, const TensorPtr& b) { return ops::sub(a, b); }
TensorPtr operator*(const TensorPtr& a, const TensorPtr& b) { return ops::mul(a, b); }
TensorPtr operator/(const TensorPtr& a, const TensorPtr& b) { return ops::div(a, b); }
TensorPtr operator+(const TensorPtr& t, float s) { return ops::add(t, s); }
TensorPtr operator-(const TensorPtr& t, float s) { return ops::sub(t, s); }
TensorPtr operator*(const TensorPtr& t, float s) { return ops::mul(t, s); }
TensorPtr operator/(const TensorPtr& t, float s) { return ops::div(t, s); }
TensorPtr operator+(float s, const TensorPtr& t) { return ops::add(s, t); }
TensorPtr operator-(float s, const TensorPtr& t) { return ops::sub(s, t); }
TensorPtr operator*(float s, const TensorPtr& t) { return ops::mul(s, t); }
TensorPtr operator/(float s, const TensorPtr& t) { return ops::div(s, t); }

}  // namespace ops
