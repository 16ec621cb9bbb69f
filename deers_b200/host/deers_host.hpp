// C++ mirror of the deers operator interface for the fused attention op, on top
// of the C ABI in include/deers_b200.h.  The deers host code is Rust; this header
// restates the handful of types the path touches with the same names, argument
// meaning and error behaviour, so that the boundary can be exercised from a
// compiled host language:
//
//   Tensor / Layout / DType            src/tensor.rs:53-108, src/layout.rs:151-202, src/dtype.rs:14-21
//   TensorOp {forward, backward, dependencies, name}      src/ops.rs:82-97
//   GradientStore::accumulate (insert-or-add)             src/backprop.rs:101-112
//   CudaStorage::attention_fwd / attention_bwd            new BackendStorage methods, added the way
//                                                         log_softmax_fwd/bwd were (src/storage.rs:284-302)
//   Error::{LayoutMismatch, DTypeMismatch, DeviceMismatch, Cuda}   src/error.rs:8-42
//   Device::synchronize                                   src/device.rs:66-72
//
//   GPTConfig / GPT {forward, parameters} and the trainer's step     src/models/gpt.rs:259-378,
//                                                         examples/tinystories_train.rs:188-218
//
// Header-only, C++17; link with libdeers_b200.so.  There is no CPU fallback.
#pragma once
#include <cmath>
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/deers_b200.h"

namespace deers {

enum class DType { F16 = DEERS_F16, F32 = DEERS_F32 };
inline size_t dtype_size(DType d) { return d == DType::F16 ? 2 : 4; }

struct Error : std::runtime_error {
    enum class Kind { LayoutMismatch, DTypeMismatch, DeviceMismatch, Cuda };
    Kind kind;
    Error(Kind k, const std::string& what) : std::runtime_error(what), kind(k) {}
};

// One process-wide runtime per device, like CudaRuntime behind its OnceLock (src/storage/cuda.rs:455-521).
class Runtime {
public:
    static Runtime& get(int device = 0) {
        static std::map<int, std::unique_ptr<Runtime>> all;
        auto& slot = all[device];
        if (!slot) slot.reset(new Runtime(device));
        return *slot;
    }
    deers_ctx* ctx() const { return ctx_; }
    void check(int status) const {
        if (status == DEERS_OK) return;
        throw Error(Error::Kind::Cuda, std::string("deers_b200: ") + deers_b200_status_string(status) + " [" +
                                           deers_b200_last_error(ctx_) + "]");
    }
    void synchronize() const { check(deers_b200_sync(ctx_)); }          // Device::synchronize
    ~Runtime() { deers_b200_destroy(ctx_); }

private:
    explicit Runtime(int device) : ctx_(nullptr) {
        const int rc = deers_b200_init(device, nullptr, &ctx_);
        if (rc != DEERS_OK) throw Error(Error::Kind::Cuda, std::string("deers_b200_init: ") + deers_b200_status_string(rc));
    }
    deers_ctx* ctx_;
};

struct Layout {
    std::vector<int64_t> shape, strides;                       // strides in elements (src/layout.rs:101-105)
    static Layout contiguous(const std::vector<int64_t>& shape) {
        Layout l{shape, std::vector<int64_t>(shape.size(), 1)};
        for (int i = (int)shape.size() - 2; i >= 0; --i) l.strides[i] = l.strides[i + 1] * shape[i + 1];
        return l;
    }
    int64_t size() const { int64_t n = 1; for (auto s : shape) n *= s; return n; }
    bool is_compact() const { return strides == contiguous(shape).strides; }
};

// Device buffer owned by the storage value and freed on drop (src/storage/cuda.rs:637-644).
class CudaStorage {
public:
    CudaStorage(size_t bytes, DType dtype, int device = 0) : rt_(&Runtime::get(device)), bytes_(bytes), dtype_(dtype) {
        rt_->check(deers_b200_alloc(rt_->ctx(), bytes, &ptr_));
    }
    CudaStorage(const CudaStorage&) = delete;
    CudaStorage& operator=(const CudaStorage&) = delete;
    ~CudaStorage() { deers_b200_free(rt_->ctx(), ptr_); }
    void* ptr() const { return ptr_; }
    size_t bytes() const { return bytes_; }
    DType dtype() const { return dtype_; }
    Runtime& runtime() const { return *rt_; }
    void upload(const void* host) { rt_->check(deers_b200_memcpy_h2d(rt_->ctx(), ptr_, host, bytes_)); rt_->synchronize(); }
    void download(void* host) const { rt_->check(deers_b200_memcpy_d2h(rt_->ctx(), host, ptr_, bytes_)); }

private:
    Runtime* rt_;
    void* ptr_ = nullptr;
    size_t bytes_;
    DType dtype_;
};

class Tensor;
class GradientStore;

// src/ops.rs:82-97.  forward() consumes the op in Rust; here the op is shared so that the
// output tensor can keep it alive for the backward walk.
class TensorOp {
public:
    virtual ~TensorOp() = default;
    virtual Tensor forward() = 0;
    virtual void backward(GradientStore& grads, const Tensor& out_grad) const = 0;
    virtual std::vector<const Tensor*> dependencies() const = 0;
    virtual const char* name() const = 0;
};

class Tensor {
public:
    Tensor() = default;
    Tensor(std::shared_ptr<CudaStorage> storage, Layout layout, std::shared_ptr<const TensorOp> op = nullptr)
        : in_(std::make_shared<Internal>(Internal{next_id()++, std::move(storage), std::move(layout), std::move(op)})) {}

    template <typename T>
    static Tensor from_vec(const std::vector<T>& data, const std::vector<int64_t>& shape, DType dtype, int device = 0) {
        Layout l = Layout::contiguous(shape);
        if ((int64_t)data.size() != l.size() || sizeof(T) != dtype_size(dtype))
            throw Error(Error::Kind::LayoutMismatch, "from_vec: data does not fit the shape / dtype");
        auto st = std::make_shared<CudaStorage>(data.size() * sizeof(T), dtype, device);
        st->upload(data.data());
        return Tensor(st, l);
    }
    template <typename T>
    std::vector<T> to_vec() const {
        if (!layout().is_compact()) throw Error(Error::Kind::LayoutMismatch, "to_vec: tensor is not compact");
        std::vector<T> out(storage().bytes() / sizeof(T));
        storage().download(out.data());
        return out;
    }
    uint64_t id() const { return in_->id; }
    const Layout& layout() const { return in_->layout; }
    CudaStorage& storage() const { return *in_->storage; }
    std::shared_ptr<CudaStorage> storage_ptr() const { return in_->storage; }
    DType dtype() const { return in_->storage->dtype(); }
    const TensorOp* op() const { return in_->op.get(); }
    bool defined() const { return (bool)in_; }

    // Tensor method of the house style (src/tensor.rs:379-381): CausalAttention::new(..).forward().
    Tensor causal_attention(const Tensor& k, const Tensor& v, float scale) const;

private:
    struct Internal {
        uint64_t id;
        std::shared_ptr<CudaStorage> storage;
        Layout layout;
        std::shared_ptr<const TensorOp> op;
    };
    static uint64_t& next_id() { static uint64_t n = 1; return n; }
    std::shared_ptr<Internal> in_;
};

// src/backprop.rs:74-128: insert-or-add keyed by tensor id.  The fused op produces exactly one
// gradient per input, so the add branch only triggers when an input is used twice; it then sums
// on the host (this mirror has no elementwise add kernel of its own).
class GradientStore {
public:
    void accumulate(const Tensor& t, const Tensor& grad) {
        auto it = grads_.find(t.id());
        if (it == grads_.end()) { grads_.emplace(t.id(), grad); return; }
        if (grad.dtype() != DType::F32) throw Error(Error::Kind::DTypeMismatch, "accumulate: repeated f16 gradient");
        auto a = it->second.to_vec<float>(), b = grad.to_vec<float>();
        for (size_t i = 0; i < a.size(); ++i) a[i] += b[i];
        it->second = Tensor::from_vec(a, grad.layout().shape, DType::F32);
    }
    const Tensor* get(const Tensor& t) const {
        auto it = grads_.find(t.id());
        return it == grads_.end() ? nullptr : &it->second;
    }

private:
    std::map<uint64_t, Tensor> grads_;
};

inline void fill_strides(int64_t (&dst)[4], const Layout& l) { for (int i = 0; i < 4; ++i) dst[i] = l.strides[i]; }

// The fused op for src/models/gpt.rs:139-144 on [B, H, T, D] tensors.
class CausalAttention : public TensorOp, public std::enable_shared_from_this<CausalAttention> {
public:
    // X::new(args) -> Result<Self>: validates, throwing the reference's error kinds (src/ops.rs:1018-1064).
    static std::shared_ptr<CausalAttention> make(const Tensor& q, const Tensor& k, const Tensor& v, float scale,
                                                 bool causal = true) {
        for (const Tensor* t : {&q, &k, &v}) {
            if (t->layout().shape.size() != 4) throw Error(Error::Kind::LayoutMismatch, "CausalAttention: expected [B, H, T, D]");
            if (t->layout().shape != q.layout().shape) throw Error(Error::Kind::LayoutMismatch, "CausalAttention: shapes differ");
            if (t->dtype() != q.dtype()) throw Error(Error::Kind::DTypeMismatch, "CausalAttention: dtypes differ");
            if (&t->storage().runtime() != &q.storage().runtime()) throw Error(Error::Kind::DeviceMismatch, "CausalAttention: devices differ");
        }
        return std::shared_ptr<CausalAttention>(new CausalAttention(q, k, v, scale, causal));
    }

    Tensor forward() override {
        Runtime& rt = q_.storage().runtime();
        const Layout out_layout = Layout::contiguous(q_.layout().shape);
        auto o = std::make_shared<CudaStorage>((size_t)out_layout.size() * dtype_size(q_.dtype()), q_.dtype());
        const auto& s = q_.layout().shape;
        lse_ = std::make_shared<CudaStorage>((size_t)(s[0] * s[1] * s[2]) * sizeof(float), DType::F32);
        deers_attn_desc d = desc(out_layout);
        // scratch only for f16 head dims other than 64 / 128 (zero-padded copies)
        const size_t fwd_ws = deers_b200_attn_workspace_bytes(&d, 0);
        std::shared_ptr<CudaStorage> ws = fwd_ws ? std::make_shared<CudaStorage>(fwd_ws, DType::F32) : nullptr;
        rt.check(deers_b200_attn_fwd(rt.ctx(), &d, q_.storage().ptr(), k_.storage().ptr(), v_.storage().ptr(), o->ptr(),
                                     (float*)lse_->ptr(), ws ? ws->ptr() : nullptr, fwd_ws));
        o_ = Tensor(o, out_layout);                                     // kept for the backward, like LogSumExp.lse
        return Tensor(o, out_layout, shared_from_this());
    }

    void backward(GradientStore& grads, const Tensor& out_grad) const override {
        if (!o_.defined()) throw std::logic_error("CausalAttention::backward before forward");
        if (out_grad.layout().shape != q_.layout().shape) throw Error(Error::Kind::LayoutMismatch, "out_grad shape");
        Runtime& rt = q_.storage().runtime();
        const Layout gl = Layout::contiguous(q_.layout().shape);
        const size_t bytes = (size_t)gl.size() * dtype_size(q_.dtype());
        auto dq = std::make_shared<CudaStorage>(bytes, q_.dtype()), dk = std::make_shared<CudaStorage>(bytes, q_.dtype()),
             dv = std::make_shared<CudaStorage>(bytes, q_.dtype());
        deers_attn_desc d = desc(o_.layout());
        fill_strides(d.do_strides, out_grad.layout());
        fill_strides(d.dq_strides, gl); fill_strides(d.dk_strides, gl); fill_strides(d.dv_strides, gl);
        // The larger (pass 2) workspace lets the f16 backward keep its dS tiles between its kernels; taken when
        // it is a small part of what the device has free, else the backward recomputes (pass 1).
        size_t ws_bytes = deers_b200_attn_workspace_bytes(&d, 1);
        const size_t fast = deers_b200_attn_workspace_bytes(&d, 2);
        size_t free_b = 0, total_b = 0;
        if (fast > ws_bytes && deers_b200_mem_info(rt.ctx(), &free_b, &total_b) == DEERS_OK && fast <= free_b / 4) ws_bytes = fast;
        CudaStorage ws(ws_bytes ? ws_bytes : 256, DType::F32);
        rt.check(deers_b200_attn_bwd(rt.ctx(), &d, q_.storage().ptr(), k_.storage().ptr(), v_.storage().ptr(),
                                     o_.storage().ptr(), (const float*)lse_->ptr(), out_grad.storage().ptr(), dq->ptr(),
                                     dk->ptr(), dv->ptr(), ws.ptr(), ws.bytes()));
        grads.accumulate(q_, Tensor(dq, gl));
        grads.accumulate(k_, Tensor(dk, gl));
        grads.accumulate(v_, Tensor(dv, gl));
    }

    std::vector<const Tensor*> dependencies() const override { return {&q_, &k_, &v_}; }
    const char* name() const override { return "CausalAttention"; }
    const CudaStorage& lse() const { return *lse_; }

private:
    CausalAttention(const Tensor& q, const Tensor& k, const Tensor& v, float scale, bool causal)
        : q_(q), k_(k), v_(v), scale_(scale), causal_(causal) {}
    deers_attn_desc desc(const Layout& o_layout) const {
        const auto& s = q_.layout().shape;
        deers_attn_desc d;
        deers_b200_attn_desc_compact(&d, (int32_t)s[0], (int32_t)s[1], (int32_t)s[2], (int32_t)s[3], (int32_t)q_.dtype(),
                                     causal_ ? 1 : 0, scale_);
        fill_strides(d.q_strides, q_.layout()); fill_strides(d.k_strides, k_.layout());
        fill_strides(d.v_strides, v_.layout()); fill_strides(d.o_strides, o_layout);
        return d;
    }
    Tensor q_, k_, v_, o_;
    float scale_;
    bool causal_;
    std::shared_ptr<CudaStorage> lse_;
};

inline Tensor Tensor::causal_attention(const Tensor& k, const Tensor& v, float scale) const {
    return CausalAttention::make(*this, k, v, scale)->forward();
}

// apply_rotary_emb(x, cos, sin).permute([0,2,1,3]) (src/models/gpt.rs:49-73,135-136) as one op: x is a compact
// [B,T,H,D] tensor, cos / sin are [1,T,1,D/2] (or [T,D/2]) of the same dtype; the result is [B,H,T,D].
class RotaryPack : public TensorOp, public std::enable_shared_from_this<RotaryPack> {
public:
    static std::shared_ptr<RotaryPack> make(const Tensor& x, const Tensor& cos, const Tensor& sin) {
        const auto& s = x.layout().shape;
        if (s.size() != 4) throw Error(Error::Kind::LayoutMismatch, "RoPE expects a 4D attention tensor");
        if (s[3] % 2) throw Error(Error::Kind::LayoutMismatch, "RoPE requires an even head dimension");
        if (cos.layout().shape != sin.layout().shape) throw Error(Error::Kind::LayoutMismatch, "RoPE cos/sin shapes must match");
        if (cos.layout().size() != s[1] * (s[3] / 2)) throw Error(Error::Kind::LayoutMismatch, "RoPE cache must match sequence length and head_dim / 2");
        if (cos.dtype() != x.dtype() || sin.dtype() != x.dtype()) throw Error(Error::Kind::DTypeMismatch, "RoPE cache dtype");
        if (!x.layout().is_compact() || !cos.layout().is_compact() || !sin.layout().is_compact())
            throw Error(Error::Kind::LayoutMismatch, "RotaryPack: compact inputs expected");
        return std::shared_ptr<RotaryPack>(new RotaryPack(x, cos, sin));
    }
    Tensor forward() override {
        const auto& s = x_.layout().shape;                              // [B,T,H,D]
        const Layout out = Layout::contiguous({s[0], s[2], s[1], s[3]});
        auto y = std::make_shared<CudaStorage>((size_t)out.size() * dtype_size(x_.dtype()), x_.dtype());
        call(x_.storage().ptr(), x_.layout(), y->ptr(), out, false);
        return Tensor(y, out, shared_from_this());
    }
    void backward(GradientStore& grads, const Tensor& out_grad) const override {
        const auto& s = x_.layout().shape;
        if (out_grad.layout().shape != std::vector<int64_t>{s[0], s[2], s[1], s[3]})
            throw Error(Error::Kind::LayoutMismatch, "RotaryPack: out_grad shape");
        const Layout dl = Layout::contiguous(s);
        auto dx = std::make_shared<CudaStorage>((size_t)dl.size() * dtype_size(x_.dtype()), x_.dtype());
        call(out_grad.storage().ptr(), dl, dx->ptr(), out_grad.layout(), true);
        grads.accumulate(x_, Tensor(dx, dl));
    }
    std::vector<const Tensor*> dependencies() const override { return {&x_}; }
    const char* name() const override { return "RotaryPack"; }

private:
    RotaryPack(const Tensor& x, const Tensor& cos, const Tensor& sin) : x_(x), cos_(cos), sin_(sin) {}
    // bthd: layout of the [B,T,H,D] side; bhtd: layout of the [B,H,T,D] side; inverse reads bhtd, writes bthd.
    void call(const void* src, const Layout& bthd, void* dst, const Layout& bhtd, bool inverse) const {
        Runtime& rt = x_.storage().runtime();
        const auto& s = x_.layout().shape;
        deers_rope_desc d{};
        d.B = (int32_t)s[0]; d.T = (int32_t)s[1]; d.H = (int32_t)s[2]; d.D = (int32_t)s[3];
        d.dtype = (int32_t)x_.dtype(); d.inverse = inverse ? 1 : 0;
        const int64_t a[4] = {bthd.strides[0], bthd.strides[1], bthd.strides[2], 1};          // (b, t, h, d)
        const int64_t b[4] = {bhtd.strides[0], bhtd.strides[2], bhtd.strides[1], 1};
        for (int i = 0; i < 4; ++i) { d.src_strides[i] = inverse ? b[i] : a[i]; d.dst_strides[i] = inverse ? a[i] : b[i]; }
        rt.check(deers_b200_rope_pack(rt.ctx(), &d, src, cos_.storage().ptr(), sin_.storage().ptr(), dst));
    }
    Tensor x_, cos_, sin_;
};

// RMSNorm::forward (src/nn.rs:244-251) over the last axis of a compact f32 tensor, one launch each way.
class RMSNorm : public TensorOp, public std::enable_shared_from_this<RMSNorm> {
public:
    static std::shared_ptr<RMSNorm> make(const Tensor& x, double eps) {
        if (x.layout().shape.empty()) throw Error(Error::Kind::LayoutMismatch, "RMSNorm: needs at least one axis");
        if (x.dtype() != DType::F32) throw Error(Error::Kind::DTypeMismatch, "RMSNorm: f32 only");
        if (!x.layout().is_compact()) throw Error(Error::Kind::LayoutMismatch, "RMSNorm: compact input expected");
        return std::shared_ptr<RMSNorm>(new RMSNorm(x, eps));
    }
    Tensor forward() override {
        Runtime& rt = x_.storage().runtime();
        const int64_t C = x_.layout().shape.back(), rows = x_.layout().size() / C;
        auto y = std::make_shared<CudaStorage>((size_t)x_.layout().size() * 4, DType::F32);
        inv_ = std::make_shared<CudaStorage>((size_t)(rows ? rows : 1) * 4, DType::F32);
        rt.check(deers_b200_rmsnorm_fwd(rt.ctx(), rows, (int32_t)C, eps_, (const float*)x_.storage().ptr(), (float*)y->ptr(),
                                        (float*)inv_->ptr()));
        return Tensor(y, x_.layout(), shared_from_this());
    }
    void backward(GradientStore& grads, const Tensor& out_grad) const override {
        if (!inv_) throw std::logic_error("RMSNorm::backward before forward");
        if (out_grad.layout().shape != x_.layout().shape || !out_grad.layout().is_compact())
            throw Error(Error::Kind::LayoutMismatch, "RMSNorm: out_grad layout");
        Runtime& rt = x_.storage().runtime();
        const int64_t C = x_.layout().shape.back(), rows = x_.layout().size() / C;
        auto dx = std::make_shared<CudaStorage>((size_t)x_.layout().size() * 4, DType::F32);
        rt.check(deers_b200_rmsnorm_bwd(rt.ctx(), rows, (int32_t)C, (const float*)x_.storage().ptr(), (const float*)inv_->ptr(),
                                        (const float*)out_grad.storage().ptr(), (float*)dx->ptr()));
        grads.accumulate(x_, Tensor(dx, x_.layout()));
    }
    std::vector<const Tensor*> dependencies() const override { return {&x_}; }
    const char* name() const override { return "RMSNorm"; }

private:
    RMSNorm(const Tensor& x, double eps) : x_(x), eps_(eps) {}
    Tensor x_;
    double eps_;
    std::shared_ptr<CudaStorage> inv_;
};

// AdamWConfig + AdamW (src/optim.rs:49-251) over compact f32 parameters, every parameter in one launch; with
// `clip_max_norm > 0` the global gradient-norm clip of clip_grad_norm (optim.rs:257-297) is applied inside it.
class AdamW {
public:
    AdamW(std::vector<Tensor> parameters, double lr, double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8,
          double weight_decay = 0.0)
        : params_(std::move(parameters)), lr_(lr), b1_(beta1), b2_(beta2), eps_(eps), wd_(weight_decay) {}
    void set_lr(double lr) { lr_ = lr; }
    double lr() const { return lr_; }
    size_t step_count() const { return step_; }
    void set_step_count(size_t s) { step_ = s; }
    void step_with_grads(const GradientStore& grads, double clip_max_norm = 0.0) {
        ++step_;
        std::vector<deers_optim_tensor> table;
        Runtime* rt = nullptr;
        for (const Tensor& p : params_) {
            const Tensor* g = grads.get(p);
            if (!g) continue;                                           // optim.rs:221-225
            if (p.dtype() != DType::F32 || g->dtype() != DType::F32) throw Error(Error::Kind::DTypeMismatch, "AdamW: f32 only");
            if (!p.layout().is_compact() || !g->layout().is_compact() || g->layout().shape != p.layout().shape)
                throw Error(Error::Kind::LayoutMismatch, "AdamW: compact parameters and gradients of equal shape expected");
            rt = &p.storage().runtime();
            auto& mv = state_[p.id()];
            if (!mv.first) {                                            // param.zeros_like()
                const std::vector<float> zeros((size_t)p.layout().size(), 0.f);
                mv.first = Tensor::from_vec(zeros, p.layout().shape, DType::F32).storage_ptr();
                mv.second = Tensor::from_vec(zeros, p.layout().shape, DType::F32).storage_ptr();
            }
            table.push_back({p.storage().ptr(), g->storage().ptr(), mv.first->ptr(), mv.second->ptr(), p.layout().size()});
        }
        if (table.empty()) return;
        const deers_adamw_hyper h{lr_, b1_, b2_, eps_, wd_, (int64_t)step_};
        if (clip_max_norm > 0.0) {
            CudaStorage norm(4, DType::F32), scratch(deers_b200_optim_scratch_bytes(), DType::F32);
            rt->check(deers_b200_grad_norm(rt->ctx(), (int)table.size(), table.data(), (float*)norm.ptr(), scratch.ptr(), scratch.bytes()));
            rt->check(deers_b200_adamw_step(rt->ctx(), (int)table.size(), table.data(), &h, (const float*)norm.ptr(), clip_max_norm));
            rt->synchronize();                                          // norm / scratch are freed on return
        } else {
            rt->check(deers_b200_adamw_step(rt->ctx(), (int)table.size(), table.data(), &h, nullptr, 0.0));
        }
    }

private:
    std::vector<Tensor> params_;
    double lr_, b1_, b2_, eps_, wd_;
    size_t step_ = 0;
    std::map<uint64_t, std::pair<std::shared_ptr<CudaStorage>, std::shared_ptr<CudaStorage>>> state_;
};

// Tensor::backward for a graph that consists of this one op (src/backprop.rs:52-66 walks the
// sorted nodes and calls op.backward for each).
inline GradientStore backward(const Tensor& out, const Tensor& out_grad) {
    GradientStore grads;
    if (out.op()) out.op()->backward(grads, out_grad);
    return grads;
}

// GPTConfig (src/models/gpt.rs:259-285) and the model as one device-resident object: GPT::forward
// (gpt.rs:329-355) and one step of the trainer loop (tinystories_train.rs:188-218: forward, cross_entropy,
// backward, clip_grad_norm, AdamW::step_with_grads).  Parameters are addressed by index in the order of
// GPT::parameters (gpt.rs:358-365).
struct GPTConfig {
    int vocab_size, sequence_len, n_layer, n_head, n_embd, mlp_hidden_dim;
    double rms_norm_eps = 1e-5;
    float rope_base = 10000.f;
};

class GPT {
public:
    GPT(const GPTConfig& cfg, int max_batch, int device = 0) : rt_(Runtime::get(device)), cfg_(cfg), model_(nullptr) {
        deers_gpt_config c{cfg.vocab_size, cfg.sequence_len, cfg.n_layer, cfg.n_head, cfg.n_embd, cfg.mlp_hidden_dim,
                           cfg.rms_norm_eps, cfg.rope_base};
        rt_.check(deers_b200_gpt_create(rt_.ctx(), &c, max_batch, &model_));
    }
    ~GPT() { deers_b200_gpt_destroy(model_); }
    GPT(const GPT&) = delete;
    GPT& operator=(const GPT&) = delete;

    int num_parameters() const { return deers_b200_gpt_num_params(model_); }
    std::pair<std::string, std::pair<int64_t, int64_t>> parameter_info(int index) const {
        char name[96];
        int64_t rows = 0, cols = 0;
        rt_.check(deers_b200_gpt_param_info(model_, index, name, sizeof(name), &rows, &cols));
        return {name, {rows, cols}};
    }
    void load_parameter(int index, const std::vector<float>& host) {
        const auto shape = parameter_info(index).second;
        if ((int64_t)host.size() != shape.first * shape.second)
            throw Error(Error::Kind::LayoutMismatch, "GPT::load_parameter: wrong element count for " + parameter_info(index).first);
        rt_.check(deers_b200_gpt_param_set(model_, index, 0, host.data()));
    }
    std::vector<float> read(int index, int what) const {        // 0 weight, 1 gradient, 2 / 3 AdamW moments
        const auto shape = parameter_info(index).second;
        std::vector<float> host((size_t)(shape.first * shape.second));
        rt_.check(deers_b200_gpt_param_get(model_, index, what, host.data()));
        return host;
    }
    // ids: B*T token ids on the host (the trainer's sample_batch + from_vec); returns logits [B*T, vocab].
    std::vector<float> forward(const std::vector<int64_t>& ids, int B, int T) {
        DeviceBuffer d_ids(rt_, ids.size() * sizeof(int64_t)), d_logits(rt_, (size_t)B * T * cfg_.vocab_size * sizeof(float));
        rt_.check(deers_b200_memcpy_h2d(rt_.ctx(), d_ids.ptr, ids.data(), ids.size() * sizeof(int64_t)));
        rt_.check(deers_b200_gpt_forward(model_, (const int64_t*)d_ids.ptr, B, T, (float*)d_logits.ptr));
        std::vector<float> logits((size_t)B * T * cfg_.vocab_size);
        rt_.check(deers_b200_memcpy_d2h(rt_.ctx(), logits.data(), d_logits.ptr, logits.size() * sizeof(float)));
        return logits;
    }
    // forward + cross_entropy + backward; returns the loss, gradients are read with read(index, 1).
    float forward_backward(const std::vector<int64_t>& ids, const std::vector<int64_t>& targets, int B, int T) {
        DeviceBuffer d_ids(rt_, ids.size() * sizeof(int64_t)), d_tgt(rt_, targets.size() * sizeof(int64_t)), d_loss(rt_, 4);
        rt_.check(deers_b200_memcpy_h2d(rt_.ctx(), d_ids.ptr, ids.data(), ids.size() * sizeof(int64_t)));
        rt_.check(deers_b200_memcpy_h2d(rt_.ctx(), d_tgt.ptr, targets.data(), targets.size() * sizeof(int64_t)));
        rt_.check(deers_b200_gpt_forward_backward(model_, (const int64_t*)d_ids.ptr, (const int64_t*)d_tgt.ptr, B, T, (float*)d_loss.ptr));
        float loss = 0.f;
        rt_.check(deers_b200_memcpy_d2h(rt_.ctx(), &loss, d_loss.ptr, 4));
        return loss;
    }
    // One optimizer step on host ids; returns {loss, gradient norm before clipping}.
    std::pair<float, float> train_step(const std::vector<int64_t>& ids, const std::vector<int64_t>& targets, int B, int T,
                                       double lr, double beta1 = 0.9, double beta2 = 0.999, double eps = 1e-8,
                                       double weight_decay = 0.0, double max_grad_norm = 0.0) {
        deers_adamw_hyper h{lr, beta1, beta2, eps, weight_decay, ++step_};
        float loss = 0.f, norm = 0.f;
        rt_.check(deers_b200_gpt_train_step_host(model_, ids.data(), targets.data(), B, T, &h, max_grad_norm, &loss, &norm));
        return {loss, norm};
    }
    int64_t step_count() const { return step_; }

private:
    struct DeviceBuffer {
        Runtime& rt;
        void* ptr = nullptr;
        DeviceBuffer(Runtime& r, size_t bytes) : rt(r) { rt.check(deers_b200_alloc(rt.ctx(), bytes, &ptr)); }
        ~DeviceBuffer() { deers_b200_free(rt.ctx(), ptr); }
    };
    Runtime& rt_;
    GPTConfig cfg_;
    deers_gpt* model_;
    int64_t step_ = 0;
};

}  // namespace deers
