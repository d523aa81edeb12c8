// The SwiGLU feed-forward: down(SiLU(gate(x)) * up(x)), no biases
// (src/llm/model_ffn.c:147-154, src/llm/vmath.h:64-68).  The reference runs a
// dense layer as the single expert of a mixture with router weight exactly 1
// (src/llm/model_load.c:505-514); here it is a part of its own.
#include "part.h"

namespace jb {

namespace {

// params: hidden_size, intermediate_size, names (optional): gate, up, down
class SwiGLU : public FeedForward {
public:
    // Rows from which gate, up and the activation run as one kernel.  Measured on
    // B200 at Qwen3-4B sizes: 167 against 165 + 37 microseconds at 2,048 rows, 103
    // against 109 at 1,024, even at 512; with few rows the one kernel cannot cut k
    // into parts and loses (29 against 20 at 8 rows).
    static constexpr long long FUSED_FROM = 512;
    // Rows up to which the one kernel runs too, in tiles of 64 gate and 64 up
    // features, if the plain product would not cut k either (a wide feed-forward:
    // the tiles alone fill the SMs).  It saves the activation kernel of a decode step
    // and of a short prompt (a prompt of 128 tokens: 3.22 -> 3.13 ms).
    static constexpr long long FUSED_UP_TO = 128;

    SwiGLU(const PartSpec &s, DType dt, Device *d) : FeedForward(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        inter_ = s.get_int("intermediate_size");
        if (hidden_ <= 0 || inter_ <= 0) config_error("swiglu: sizes must be positive");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_gate_ = leaf("gate", "gate_proj.weight");
        n_up_ = leaf("up", "up_proj.weight");
        n_down_ = leaf("down", "down_proj.weight");
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, n_gate_), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, n_up_), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, n_down_), TensorSpec{{hidden_, inter_}, MATRIX, false});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        std::vector<DevTensor> gu = {take(t, name(prefix, n_gate_)), take(t, name(prefix, n_up_))};
        w_gate_up_ = fuse_rows(*dev, gu);
        w_down_ = take(t, name(prefix, n_down_));
    }

    size_t weight_bytes() const override { return w_gate_up_.bytes() + w_down_.bytes(); }

    Stack forward(StepContext &ctx, const void *h) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        Buf act;
        fused_last_ = false;
        if (ctx.dtype == BF16 &&
            (n >= FUSED_FROM || (n <= FUSED_UP_TO && ops::linear_parts(n, 2 * inter_, hidden_) == 1))) {
            // enough rows, or enough features, to fill the SMs without cutting k:
            // gate, up and the activation in one kernel
            act = ops::linear_swiglu(d, h, ctx.dtype, n, hidden_, w_gate_up_);
            fused_last_ = (bool)act;
        }
        if (!act) {
            Stack gu = ops::linear(d, h, ctx.dtype, n, hidden_, w_gate_up_);
            act = ops::swiglu(d, gu, ctx.dtype);
        }
        return ops::linear(d, act.ptr, ctx.dtype, n, inter_, w_down_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("fused_from", FUSED_FROM);
        o.set("fused_up_to", FUSED_UP_TO);
        o.set("fused_last", fused_last_);
        return o;
    }

private:
    long long hidden_, inter_;
    std::string n_gate_, n_up_, n_down_;
    DevTensor w_gate_up_, w_down_;
    bool fused_last_ = false;      // whether the last forward took the one-kernel way
};

// A dense feed-forward with the PolyNorm activation: down(act(up(x))), no biases,
//   act(z) = c0 n(z) + c1 n(z^2) + c2 n(z^3) + c3,   n(u) = u / sqrt(mean(u^2) + eps)
// with powers value by value, the mean over one token's feed-forward values, and
// the four numbers c learned.
// params: hidden_size, intermediate_size, eps, names (optional): up, down, coefficients
class PolyNormFFN : public FeedForward {
public:
    PolyNormFFN(const PartSpec &s, DType dt, Device *d) : FeedForward(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        inter_ = s.get_int("intermediate_size");
        eps_ = (float)s.get_double("eps");
        if (hidden_ <= 0 || inter_ <= 0) config_error("polynorm: sizes must be positive");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_up_ = leaf("up", "up_proj.weight");
        n_down_ = leaf("down", "down_proj.weight");
        n_coef_ = leaf("coefficients", "act.weight");
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, n_up_), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, n_down_), TensorSpec{{hidden_, inter_}, MATRIX, false});
        out.emplace_back(name(prefix, n_coef_), TensorSpec{{4}, PARAM, false, 0.3f, 0.1f});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        w_up_ = take(t, name(prefix, n_up_));
        w_down_ = take(t, name(prefix, n_down_));
        coef_ = take(t, name(prefix, n_coef_));
    }

    size_t weight_bytes() const override { return w_up_.bytes() + w_down_.bytes() + coef_.bytes(); }

    bool take_side_rows(DevTensor &m) override {
        if (!w_up_ || m.shape.size() != 2 || m.shape[1] != hidden_ || side_) return false;
        std::vector<DevTensor> both = {w_up_, m};
        w_up_ = DevTensor();
        m = DevTensor();
        w_up_ = fuse_rows(*dev, both);
        side_ = true;
        return true;
    }

    Stack forward(StepContext &ctx, const void *h) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        Stack z = ops::linear(d, h, ctx.dtype, n, hidden_, w_up_);
        Buf act = ops::polynorm(d, z, inter_, (const float *)coef_.ptr, eps_, ctx.dtype);
        if (side_) {
            ctx.side = std::move(z);
            ctx.side_col0 = inter_;
        }
        z = Stack();
        return ops::linear(d, act.ptr, ctx.dtype, n, inter_, w_down_);
    }

private:
    long long hidden_, inter_;
    float eps_;
    std::string n_up_, n_down_, n_coef_;
    DevTensor w_up_, w_down_, coef_;
    bool side_ = false;     // the up matrix carries side rows after its own
};

// A dense feed-forward of two matrices: down(act(up(x))), no biases, the activation
// value by value.
// params: hidden_size, intermediate_size, activation ("relu2": the square of relu;
// "relu"; "gelu_tanh"), names (optional): up, down
class DenseFFN : public FeedForward {
public:
    DenseFFN(const PartSpec &s, DType dt, Device *d) : FeedForward(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        inter_ = s.get_int("intermediate_size");
        if (hidden_ <= 0 || inter_ <= 0) config_error("dense: sizes must be positive");
        std::string act = s.params.get("activation").is_string() ? s.params.get("activation").as_string() : "";
        act_ = ops::activation_kind(act);
        if (act_ < 0) config_error("dense: activation '" + act + "' is not one of relu2, relu, gelu_tanh");
        const Json &nm = s.params.get("names");
        n_up_ = nm.is_object() && nm.get("up").is_string() ? nm.get("up").as_string() : "up_proj.weight";
        n_down_ = nm.is_object() && nm.get("down").is_string() ? nm.get("down").as_string() : "down_proj.weight";
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, n_up_), TensorSpec{{inter_, hidden_}, MATRIX, false});
        out.emplace_back(name(prefix, n_down_), TensorSpec{{hidden_, inter_}, MATRIX, false});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        w_up_ = take(t, name(prefix, n_up_));
        w_down_ = take(t, name(prefix, n_down_));
    }

    size_t weight_bytes() const override { return w_up_.bytes() + w_down_.bytes(); }

    Stack forward(StepContext &ctx, const void *h) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        Stack z = ops::linear(d, h, ctx.dtype, n, hidden_, w_up_);
        Buf act = ops::activation(d, z, inter_, act_, ctx.dtype);
        z = Stack();
        return ops::linear(d, act.ptr, ctx.dtype, n, inter_, w_down_);
    }

private:
    long long hidden_, inter_;
    int act_;
    std::string n_up_, n_down_;
    DevTensor w_up_, w_down_;
};

}  // namespace

void register_builtin_feed_forwards() {
    register_part("feed_forward", "dense", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new DenseFFN(s, dt, d));
    });
    register_part("feed_forward", "polynorm", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new PolyNormFFN(s, dt, d));
    });
    register_part("feed_forward", "swiglu", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new SwiGLU(s, dt, d));
    });
}

}  // namespace jb
