// Test of the C++ host mirror (deers_b200/host/deers_host.hpp) against the CPU oracle: the
// fused op is driven the way deers drives a TensorOp (new -> forward -> backward into a
// GradientStore) and its results are compared with oracle/attn_ref.c on the same seeded inputs.
// Test infrastructure: links the oracle, never shipped.
#include <cstdio>
#include <random>

#include "../../deers_b200/host/deers_host.hpp"

extern "C" int ref_attn_fwd_bwd(const float* q, const float* k, const float* v, const float* d_o, int B, int H, int T,
                                int D, float scale, int causal, float* o, float* lse, float* dq, float* dk, float* dv);

extern "C" void ref_rope_pack(const float* x, const float* cosv, const float* sinv, int B, int T, int H, int D, int inverse,
                              float* y);
extern "C" void ref_rmsnorm(const float* x, long long rows, int C, double eps, const float* dy, float* y, float* dx);
extern "C" void ref_adamw_step(float* w, const float* g, float* m, float* v, long long n, double lr, double beta1,
                               double beta2, double eps, double weight_decay, int step);

static float max_rel(const std::vector<float>& got, const std::vector<float>& want) {
    float err = 0.f, mx = 1e-30f;
    for (size_t i = 0; i < want.size(); ++i) {
        if (!(got[i] == got[i])) return INFINITY;
        err = std::fmax(err, std::fabs(got[i] - want[i]));
        mx = std::fmax(mx, std::fabs(want[i]));
    }
    return err / mx;
}

template <typename T>
static std::vector<float> as_float(const std::vector<T>& v) {
    std::vector<float> out(v.size());
    for (size_t i = 0; i < v.size(); ++i) out[i] = (float)v[i];
    return out;
}

static int run_case(deers::DType dtype, int B, int H, int T, int D, float tol) {
    const size_t n = (size_t)B * H * T * D;
    std::mt19937 rng(1234 + T + D);
    std::normal_distribution<float> dist(0.f, 1.f);
    std::vector<float> host[4];
    for (auto& h : host) {
        h.resize(n);
        for (auto& x : h) { x = dist(rng); if (dtype == deers::DType::F16) x = (float)(_Float16)x; }
    }
    const float scale = (float)(1.0 / std::sqrt((double)D));
    std::vector<float> o(n), lse((size_t)B * H * T), dq(n), dk(n), dv(n);
    ref_attn_fwd_bwd(host[0].data(), host[1].data(), host[2].data(), host[3].data(), B, H, T, D, scale, 1, o.data(),
                     lse.data(), dq.data(), dk.data(), dv.data());

    const std::vector<int64_t> shape{B, H, T, D};
    deers::Tensor t[4];
    for (int i = 0; i < 4; ++i) {
        if (dtype == deers::DType::F16) {
            std::vector<_Float16> h16(n);
            for (size_t e = 0; e < n; ++e) h16[e] = (_Float16)host[i][e];
            t[i] = deers::Tensor::from_vec(h16, shape, dtype);
        } else {
            t[i] = deers::Tensor::from_vec(host[i], shape, dtype);
        }
    }
    deers::Tensor y = t[0].causal_attention(t[1], t[2], scale);
    if (std::string(y.op()->name()) != "CausalAttention" || y.op()->dependencies().size() != 3) return 1;
    deers::GradientStore grads = deers::backward(y, t[3]);
    deers::Runtime::get().synchronize();

    auto fetch = [&](const deers::Tensor& x) {
        return dtype == deers::DType::F16 ? as_float(x.to_vec<_Float16>()) : x.to_vec<float>();
    };
    const float e[4] = {max_rel(fetch(y), o), max_rel(fetch(*grads.get(t[0])), dq), max_rel(fetch(*grads.get(t[1])), dk),
                        max_rel(fetch(*grads.get(t[2])), dv)};
    const bool ok = e[0] <= tol && e[1] <= tol && e[2] <= tol && e[3] <= tol;
    std::printf("%s %s B%d H%d T%d D%d  o %.2e dq %.2e dk %.2e dv %.2e (tol %.0e)\n", ok ? "PASS" : "FAIL",
                dtype == deers::DType::F16 ? "f16" : "f32", B, H, T, D, e[0], e[1], e[2], e[3], tol);
    return ok ? 0 : 1;
}

// The other ops of the mirror (rotary pack, RMSNorm, AdamW) against the oracle's restatements, f32.
static int run_other_ops() {
    int fails = 0;
    std::mt19937 rng(99);
    std::normal_distribution<float> dist(0.f, 1.f);
    {   // RotaryPack: bit-exact forward and backward
        const int B = 2, T = 9, H = 3, D = 16;
        std::vector<float> x((size_t)B * T * H * D), dy(x.size()), cs((size_t)T * D / 2), sn(cs.size());
        for (auto& v : x) v = dist(rng);
        for (auto& v : dy) v = dist(rng);
        for (int t = 0; t < T; ++t)
            for (int i = 0; i < D / 2; ++i) {
                const float f = (float)t * (1.0f / std::pow(10000.0f, (float)(2 * i) / (float)D));
                cs[(size_t)t * D / 2 + i] = std::cos(f); sn[(size_t)t * D / 2 + i] = std::sin(f);
            }
        std::vector<float> want_y(x.size()), want_dx(x.size());
        ref_rope_pack(x.data(), cs.data(), sn.data(), B, T, H, D, 0, want_y.data());
        ref_rope_pack(dy.data(), cs.data(), sn.data(), B, T, H, D, 1, want_dx.data());
        auto tx = deers::Tensor::from_vec(x, {B, T, H, D}, deers::DType::F32);
        auto tc = deers::Tensor::from_vec(cs, {1, T, 1, D / 2}, deers::DType::F32);
        auto ts = deers::Tensor::from_vec(sn, {1, T, 1, D / 2}, deers::DType::F32);
        auto y = deers::RotaryPack::make(tx, tc, ts)->forward();
        auto grads = deers::backward(y, deers::Tensor::from_vec(dy, {B, H, T, D}, deers::DType::F32));
        deers::Runtime::get().synchronize();
        const bool ok = y.to_vec<float>() == want_y && grads.get(tx)->to_vec<float>() == want_dx &&
                        std::string(y.op()->name()) == "RotaryPack";
        std::printf("%s RotaryPack bit-exact\n", ok ? "PASS" : "FAIL");
        fails += !ok;
    }
    {   // RMSNorm
        const int rows = 37, C = 192;
        std::vector<float> x((size_t)rows * C), dy(x.size()), wy(x.size()), wdx(x.size());
        for (auto& v : x) v = dist(rng);
        for (auto& v : dy) v = dist(rng);
        ref_rmsnorm(x.data(), rows, C, 1e-6, dy.data(), wy.data(), wdx.data());
        auto tx = deers::Tensor::from_vec(x, {rows, C}, deers::DType::F32);
        auto y = deers::RMSNorm::make(tx, 1e-6)->forward();
        auto grads = deers::backward(y, deers::Tensor::from_vec(dy, {rows, C}, deers::DType::F32));
        deers::Runtime::get().synchronize();
        const float e1 = max_rel(y.to_vec<float>(), wy), e2 = max_rel(grads.get(tx)->to_vec<float>(), wdx);
        const bool ok = e1 <= 1e-5f && e2 <= 1e-5f;
        std::printf("%s RMSNorm y %.2e dx %.2e\n", ok ? "PASS" : "FAIL", e1, e2);
        fails += !ok;
    }
    {   // AdamW: three steps, bit-exact
        const int n = 5000;
        std::vector<float> w(n), m(n, 0.f), v(n, 0.f);
        for (auto& e : w) e = dist(rng);
        auto tw = deers::Tensor::from_vec(w, {n}, deers::DType::F32);
        deers::AdamW opt({tw}, 1e-3, 0.9, 0.95, 1e-8, 0.1);
        for (int step = 1; step <= 3; ++step) {
            std::vector<float> g(n);
            for (auto& e : g) e = dist(rng);
            deers::GradientStore grads;
            grads.accumulate(tw, deers::Tensor::from_vec(g, {n}, deers::DType::F32));
            opt.step_with_grads(grads);
            ref_adamw_step(w.data(), g.data(), m.data(), v.data(), n, 1e-3, 0.9, 0.95, 1e-8, 0.1, step);
        }
        deers::Runtime::get().synchronize();
        const bool ok = tw.to_vec<float>() == w && opt.step_count() == 3;
        std::printf("%s AdamW bit-exact\n", ok ? "PASS" : "FAIL");
        fails += !ok;
    }
    return fails;
}

// The reference's model test (tests/gpt.rs:38-66: vocab 8, 1 layer, 2 heads, n_embd 4, mlp 8, B=2, T=3, its token
// ids) through deers::GPT, against the C oracle's step: logits, loss, every parameter gradient (2e-3, the
// reference's accelerator tolerance), then one optimizer step.
extern "C" int ref_gpt_step(const int* cfg, double eps, float rope_base, int B, int T, const long long* ids,
                            const long long* targets, const float* const* params, float* logits_out, float* loss_out,
                            float* const* grads);

static int run_gpt() {
    int fails = 0;
    const int V = 8, L = 1, H = 2, C = 4, Hm = 8, B = 2, T = 3;
    deers::GPT model({V, 4, L, H, C, Hm}, B);
    std::mt19937 rng(77);
    std::uniform_real_distribution<float> uni(-0.5f, 0.5f);
    std::vector<std::vector<float>> params, grads;
    for (int i = 0; i < model.num_parameters(); ++i) {
        const auto shape = model.parameter_info(i).second;
        params.emplace_back((size_t)(shape.first * shape.second));
        for (auto& e : params.back()) e = uni(rng);
        grads.emplace_back(params.back().size());
        model.load_parameter(i, params.back());
    }
    const std::vector<int64_t> ids = {1, 2, 3, 4, 3, 2}, targets = {2, 3, 4, 3, 2, 1};
    const std::vector<long long> ids_ll(ids.begin(), ids.end()), tgt_ll(targets.begin(), targets.end());
    std::vector<const float*> pp;
    std::vector<float*> gp;
    for (size_t i = 0; i < params.size(); ++i) { pp.push_back(params[i].data()); gp.push_back(grads[i].data()); }
    const int cfg[5] = {V, L, H, C, Hm};
    std::vector<float> want_logits((size_t)B * T * V);
    float want_loss = 0.f;
    ref_gpt_step(cfg, 1e-5, 10000.f, B, T, ids_ll.data(), tgt_ll.data(), pp.data(), want_logits.data(), &want_loss, gp.data());
    const std::vector<float> logits = model.forward(ids, B, T);
    const float loss = model.forward_backward(ids, targets, B, T);
    float err = std::fabs(loss - want_loss);
    for (size_t i = 0; i < logits.size(); ++i) err = std::max(err, std::fabs(logits[i] - want_logits[i]));
    for (int i = 0; i < model.num_parameters(); ++i) {
        const std::vector<float> g = model.read(i, 1);
        for (size_t e = 0; e < g.size(); ++e) err = std::max(err, std::fabs(g[e] - grads[i][e]));
    }
    bool ok = err < 2e-3f && model.parameter_info(1).first == "blocks.0.attn.q_proj.weight";
    std::printf("%s GPT logits / loss / gradients (max abs err %.2e)\n", ok ? "PASS" : "FAIL", err);
    fails += !ok;
    const auto step = model.train_step(ids, targets, B, T, 1e-2, 0.9, 0.999, 1e-8, 0.1, 1.0);
    const float loss2 = model.forward_backward(ids, targets, B, T);
    ok = std::fabs(step.first - want_loss) < 2e-3f && std::isfinite(step.second) && loss2 < step.first;
    std::printf("%s GPT training step lowers the loss (%.4f -> %.4f, grad norm %.4f)\n", ok ? "PASS" : "FAIL", step.first, loss2,
                step.second);
    fails += !ok;
    return fails;
}

int main() {
    int fails = 0;
    try {
        fails += run_other_ops();
        fails += run_gpt();
        fails += run_case(deers::DType::F32, 2, 3, 96, 32, 1e-4f);
        fails += run_case(deers::DType::F16, 2, 2, 300, 128, 2e-2f);
        fails += run_case(deers::DType::F16, 1, 3, 200, 64, 2e-2f);
        // Error behaviour: mismatched shapes are a LayoutMismatch, like the Rust constructor.
        auto a = deers::Tensor::from_vec(std::vector<float>(64, 0.f), {1, 1, 8, 8}, deers::DType::F32);
        auto b = deers::Tensor::from_vec(std::vector<float>(32, 0.f), {1, 1, 4, 8}, deers::DType::F32);
        try {
            deers::CausalAttention::make(a, b, a, 1.0f);
            std::printf("FAIL no LayoutMismatch\n");
            ++fails;
        } catch (const deers::Error& err) {
            const bool ok = err.kind == deers::Error::Kind::LayoutMismatch;
            std::printf("%s LayoutMismatch raised\n", ok ? "PASS" : "FAIL");
            fails += !ok;
        }
    } catch (const std::exception& ex) {
        std::printf("FAIL exception: %s\n", ex.what());
        return 2;
    }
    return fails ? 1 : 0;
}
