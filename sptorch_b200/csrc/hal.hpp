// hal.hpp -- C++ mirror of sptorch's backend surface over the C-ABI (header only, no CUDA needed to compile).
//
//   Backend          crates/hal/src/lib.rs:337-367   name, device_id, allocate, copy_to_host, copy_from_host, synchronize
//   KernelProvider   crates/hal/src/lib.rs:374-458   the f32 kernels, host slices in / out
//   BackendDispatch  crates/core-tensor/src/lib.rs:81-100   the nine methods core-ops consults
//   FfiBackend       crates/hal-ffi/src/lib.rs:176-502      dlopen + symbol resolution + alloc/h2d/op/d2h/free per call
//
// Rust is not available where this library is built, so this is the compiled-language host side; method names,
// argument meaning and failure behaviour follow the traits.  Unlike the Rust wrapper, a non-zero return of an op
// is not ignored: it throws HalError.
#pragma once
#include <dlfcn.h>
#include <cstddef>
#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace sptorch_b200 {

struct HalError : std::runtime_error { using std::runtime_error::runtime_error; };

struct DeviceId { std::string backend; int ordinal; };          // crates/hal/src/lib.rs:44-49

class FfiBackend;

// crates/hal/src/lib.rs RawBuffer + hal-ffi FfiDeviceBuffer (lib.rs:61-118): frees its handle when dropped
class RawBuffer {
public:
    RawBuffer(std::shared_ptr<const FfiBackend> b, void* h, size_t n) : b_(std::move(b)), h_(h), n_(n) {}
    RawBuffer(const RawBuffer&) = delete;
    RawBuffer& operator=(const RawBuffer&) = delete;
    RawBuffer(RawBuffer&& o) noexcept : b_(std::move(o.b_)), h_(o.h_), n_(o.n_) { o.h_ = nullptr; }
    ~RawBuffer();
    void* handle() const { return h_; }
    size_t len() const { return n_; }                           // f32 elements
    std::vector<float> to_host() const;
private:
    std::shared_ptr<const FfiBackend> b_;
    void* h_;
    size_t n_;
};

class FfiBackend : public std::enable_shared_from_this<FfiBackend> {
public:
    // FfiBackend::load (hal-ffi/src/lib.rs:176-214): dlopen, resolve 19 required symbols + 1 optional, init != 0 is an error
    static std::shared_ptr<FfiBackend> load(const std::string& path) {
        void* lib = dlopen(path.c_str(), RTLD_NOW | RTLD_LOCAL);
        if (!lib) throw HalError(std::string("failed to load ") + path + ": " + dlerror());
        std::shared_ptr<FfiBackend> b(new FfiBackend(lib));
        b->resolve();
        if (b->init_() != 0) {
            std::string why = b->last_error_ ? b->last_error_() : "";
            b->initialised_ = false;
            throw HalError("sptorch_backend_init failed: " + why);
        }
        b->initialised_ = true;
        return b;
    }
    ~FfiBackend() {                                             // Drop: hal-ffi/src/lib.rs:146-153
        if (initialised_ && shutdown_) shutdown_();
        if (lib_) dlclose(lib_);
    }

    // ---- Backend ----
    std::string name() const { return name_(); }
    DeviceId device_id() const { return DeviceId{"cuda", device_ ? device_() : 0}; }
    RawBuffer allocate(size_t bytes) const {
        void* h = alloc_((bytes + 3) / 4);
        if (!h) throw HalError("allocate failed: " + err());
        return RawBuffer(shared_from_this(), h, (bytes + 3) / 4);
    }
    void copy_to_host(const RawBuffer& buf, float* dst, size_t n) const {
        if (n != buf.len()) throw HalError("copy_to_host: length mismatch");
        check(d2h_(buf.handle(), dst, n), "copy_d2h");
    }
    void copy_from_host(const float* src, size_t n, RawBuffer& buf) const {
        if (n != buf.len()) throw HalError("copy_from_host: length mismatch");
        check(h2d_(src, buf.handle(), n), "copy_h2d");
    }
    void synchronize() const { check(sync_(), "sync"); }
    RawBuffer upload(const std::vector<float>& data) const {     // hal-ffi/src/lib.rs:218-235
        RawBuffer b = allocate(data.size() * 4);
        check(h2d_(data.data(), b.handle(), data.size()), "copy_h2d");
        return b;
    }
    // hal-ffi/src/lib.rs:276-285: None when the optional hook is absent
    bool query_runtime(uint32_t* queue_depth, bool* online) const {
        if (!query_) return false;
        uint32_t q = 0, o = 0;
        if (query_(&q, &o) != 0) return false;
        *queue_depth = q; *online = o != 0;
        return true;
    }

    // ---- KernelProvider / BackendDispatch: host slices in, host slice out ----
    void add_f32(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& out) const { binary(add_, a, b, out, "add_f32"); }
    void mul_f32(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& out) const { binary(mul_, a, b, out, "mul_f32"); }
    void neg_f32(const std::vector<float>& a, std::vector<float>& out) const { unary(neg_, a, out, "neg_f32"); }
    void exp_f32(const std::vector<float>& a, std::vector<float>& out) const { unary(exp_, a, out, "exp_f32"); }
    void log_f32(const std::vector<float>& a, std::vector<float>& out) const { unary(log_, a, out, "log_f32"); }
    void relu_f32(const std::vector<float>& a, std::vector<float>& out) const { unary(relu_, a, out, "relu_f32"); }
    void gelu_f32(const std::vector<float>& a, std::vector<float>& out) const { unary(gelu_, a, out, "gelu_f32"); }
    void scale_f32(const std::vector<float>& a, float s, std::vector<float>& out) const {
        RawBuffer da = upload(a), dout = allocate(a.size() * 4);
        check(scale_(da.handle(), s, dout.handle(), a.size()), "scale_f32");
        out = dout.to_host();
    }
    void matmul_f32(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& out, size_t m, size_t k, size_t n) const {
        RawBuffer da = upload(a), db = upload(b), dout = allocate(m * n * 4);
        check(matmul_(da.handle(), db.handle(), dout.handle(), m, k, n), "matmul_f32");
        out = dout.to_host();
    }
    void batch_matmul_f32(const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& out, size_t batch, size_t m, size_t k, size_t n) const {
        RawBuffer da = upload(a), db = upload(b), dout = allocate(batch * m * n * 4);
        check(bmm_(da.handle(), db.handle(), dout.handle(), batch, m, k, n), "batch_matmul_f32");
        out = dout.to_host();
    }
    void softmax_f32(const std::vector<float>& a, std::vector<float>& out, size_t rows, size_t cols) const {
        RawBuffer da = upload(a), dout = allocate(rows * cols * 4);
        check(softmax_(da.handle(), dout.handle(), rows, cols), "softmax_f32");
        out = dout.to_host();
    }

    void free_handle(void* h) const { if (h) free_(h); }
    int d2h(const void* dev, float* host, size_t n) const { return d2h_(dev, host, n); }

private:
    explicit FfiBackend(void* lib) : lib_(lib) {}
    template <class F> void sym(F& f, const char* name, bool required = true) {
        f = reinterpret_cast<F>(dlsym(lib_, name));
        if (!f && required) throw HalError(std::string("missing symbol ") + name);   // hal-ffi/src/lib.rs:163-169
    }
    void resolve() {
        sym(init_, "sptorch_backend_init"); sym(shutdown_, "sptorch_backend_shutdown"); sym(name_, "sptorch_backend_name");
        sym(alloc_, "sptorch_alloc"); sym(free_, "sptorch_free"); sym(h2d_, "sptorch_copy_h2d"); sym(d2h_, "sptorch_copy_d2h");
        sym(sync_, "sptorch_sync"); sym(query_, "sptorch_query_runtime", false);
        sym(add_, "sptorch_add_f32"); sym(mul_, "sptorch_mul_f32"); sym(neg_, "sptorch_neg_f32"); sym(exp_, "sptorch_exp_f32");
        sym(log_, "sptorch_log_f32"); sym(relu_, "sptorch_relu_f32"); sym(gelu_, "sptorch_gelu_f32"); sym(scale_, "sptorch_scale_f32");
        sym(matmul_, "sptorch_matmul_f32"); sym(bmm_, "sptorch_batch_matmul_f32"); sym(softmax_, "sptorch_softmax_f32");
        sym(last_error_, "sptorch_ext_last_error", false); sym(device_, "sptorch_ext_device", false);
    }
    std::string err() const { return last_error_ ? last_error_() : "(no error text)"; }
    void check(int rc, const char* what) const { if (rc != 0) throw HalError(std::string(what) + " failed: " + err()); }
    using Un = int (*)(const void*, void*, size_t);
    using Bin = int (*)(const void*, const void*, void*, size_t);
    void unary(Un f, const std::vector<float>& a, std::vector<float>& out, const char* what) const {
        RawBuffer da = upload(a), dout = allocate(a.size() * 4);
        check(f(da.handle(), dout.handle(), a.size()), what);
        out = dout.to_host();
    }
    void binary(Bin f, const std::vector<float>& a, const std::vector<float>& b, std::vector<float>& out, const char* what) const {
        if (a.size() != b.size()) throw HalError(std::string(what) + ": length mismatch");
        RawBuffer da = upload(a), db = upload(b), dout = allocate(a.size() * 4);
        check(f(da.handle(), db.handle(), dout.handle(), a.size()), what);
        out = dout.to_host();
    }

    void* lib_ = nullptr;
    bool initialised_ = false;
    int (*init_)() = nullptr; void (*shutdown_)() = nullptr; const char* (*name_)() = nullptr;
    void* (*alloc_)(size_t) = nullptr; void (*free_)(void*) = nullptr;
    int (*h2d_)(const float*, void*, size_t) = nullptr; int (*d2h_)(const void*, float*, size_t) = nullptr;
    int (*sync_)() = nullptr; int (*query_)(uint32_t*, uint32_t*) = nullptr;
    Bin add_ = nullptr, mul_ = nullptr; Un neg_ = nullptr, exp_ = nullptr, log_ = nullptr, relu_ = nullptr, gelu_ = nullptr;
    int (*scale_)(const void*, float, void*, size_t) = nullptr;
    int (*matmul_)(const void*, const void*, void*, size_t, size_t, size_t) = nullptr;
    int (*bmm_)(const void*, const void*, void*, size_t, size_t, size_t, size_t) = nullptr;
    int (*softmax_)(const void*, void*, size_t, size_t) = nullptr;
    const char* (*last_error_)() = nullptr; int (*device_)() = nullptr;
};

inline RawBuffer::~RawBuffer() { if (h_ && b_) b_->free_handle(h_); }
inline std::vector<float> RawBuffer::to_host() const {
    std::vector<float> v(n_);
    if (b_->d2h(h_, v.data(), n_) != 0) throw HalError("copy_d2h failed");
    return v;
}

// ---- key/value cache metadata (crates/hal/src/lib.rs:129-239): host-side bookkeeping only ----
enum class DType { F32, F16, BF16 };
inline size_t dtype_size_bytes(DType t) { return t == DType::F32 ? 4 : 2; }

// One K or V buffer is [layer, position, head, dim]; `position` is a slot of the window, not an absolute token position.
// The device model's caches use the same order per sequence ([layer][sequence][position][head * dim]).
struct KvCacheBufferSpec {
    DeviceId device; DType dtype; size_t n_layer, max_context, n_head, head_dim;
    KvCacheBufferSpec(DeviceId dev, DType dt, size_t layers, size_t ctx, size_t heads, size_t hd)
        : device(std::move(dev)), dtype(dt), n_layer(layers), max_context(ctx), n_head(heads), head_dim(hd) {
        if (!ctx) throw HalError("max_context must be positive");
        if (!heads) throw HalError("n_head must be positive");
        if (!hd) throw HalError("head_dim must be positive");
    }
    size_t elements_per_kind() const { return n_layer * max_context * n_head * head_dim; }
    size_t total_elements() const { return elements_per_kind() * 2; }
    size_t total_bytes() const { return total_elements() * dtype_size_bytes(dtype); }
    size_t element_offset(size_t layer, size_t position, size_t head, size_t dim) const {
        if (layer >= n_layer) throw HalError("layer out of range");
        if (position >= max_context) throw HalError("position out of range");
        if (head >= n_head) throw HalError("head out of range");
        if (dim >= head_dim) throw HalError("dim out of range");
        return (((layer * max_context + position) * n_head + head) * head_dim) + dim;
    }
    bool operator==(const KvCacheBufferSpec& o) const {
        return device.backend == o.device.backend && device.ordinal == o.device.ordinal && dtype == o.dtype && n_layer == o.n_layer &&
               max_context == o.max_context && n_head == o.n_head && head_dim == o.head_dim;
    }
};

// Which absolute positions the cached window covers (crates/hal/src/lib.rs:186-239).
struct KvCacheWindowState {
    size_t window_start = 0, cached_len = 0, max_context;
    explicit KvCacheWindowState(size_t ctx) : max_context(ctx) { if (!ctx) throw HalError("max_context must be positive"); }
    size_t next_position() const { return window_start + cached_len; }
    bool last_position(size_t* pos) const { if (!cached_len) return false; *pos = window_start + cached_len - 1; return true; }
    void prefill(size_t start_position, size_t len) {
        if (len > max_context) throw HalError("prefill len cannot exceed max_context");
        window_start = start_position; cached_len = len;
    }
    void append(size_t len) {
        const size_t total = cached_len + len;
        const size_t dropped = total > max_context ? total - max_context : 0;
        window_start += dropped;
        cached_len = total < max_context ? total : max_context;
    }
    bool operator==(const KvCacheWindowState& o) const { return window_start == o.window_start && cached_len == o.cached_len && max_context == o.max_context; }
};

}  // namespace sptorch_b200
