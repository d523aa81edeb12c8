// RMSNorm: out = (x * 1/sqrt(mean(x^2) + eps)) * w
// (src/llm/model_impl.h:635-644).  The weight is used as it is, not as 1 + w.
#include "part.h"

namespace jb {

namespace {

// params: size, eps; one_plus (default false): the stored weight lies around zero and the
// norm multiplies by 1 + w (the sum is taken once, in float32, when the weight is loaded);
// names (optional): weight: the tensor's leaf below the part's prefix ("" for the prefix itself)
class RMSNorm : public Norm {
public:
    RMSNorm(const PartSpec &s, DType dt, Device *d) : Norm(s, dt, d) {
        size_ = s.get_int("size");
        eps_ = (float)s.get_double("eps");
        one_plus_ = s.has("one_plus") && s.params.get("one_plus").as_bool();
        if (size_ <= 0) config_error("rmsnorm: size must be positive");
        const Json &nm = s.params.get("names");
        w_name_ = nm.is_object() && nm.get("weight").is_string() ? nm.get("weight").as_string() : "weight";
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        if (one_plus_) out.emplace_back(name(prefix, w_name_), TensorSpec{{size_}, PARAM, false, 0.0f, 0.1f});
        else out.emplace_back(name(prefix, w_name_), TensorSpec{{size_}, NORM, false});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        weight_ = take(t, name(prefix, w_name_));
        if (one_plus_) {
            if (weight_.dt != F32) fail(JB_LLM_EFAIL, "rmsnorm: a weight around zero is kept in float32");
            std::vector<float> host((size_t)size_);
            dev->sync();
            cuda_check(cudaMemcpy(host.data(), weight_.ptr, host.size() * 4, cudaMemcpyDeviceToHost),
                       "reading a norm's weight");
            for (float &v : host) v = 1.0f + v;
            cuda_check(cudaMemcpy(weight_.ptr, host.data(), host.size() * 4, cudaMemcpyHostToDevice),
                       "writing a norm's weight");
        }
    }

    size_t weight_bytes() const override { return weight_.bytes(); }

    Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta,
              const int32_t *rows, long long n_out) override {
        return ops::rmsnorm(*ctx.dev, x, n, size_, weight_, eps_, out_dt, delta, rows, n_out);
    }

    long long size() const override { return size_; }

    // a float32 weight can go into the kernel that norms a sublayer's result and adds it
    bool layer_norm(ops::LnParams *out, bool *rms) const override {
        if (!weight_ || weight_.dt != F32) return false;
        out->w = (const float *)weight_.ptr;
        out->b = nullptr;
        out->eps = eps_;
        *rms = true;
        return true;
    }

    Json info() const override {
        Json o = Json::object();
        o.set("size", size_);
        o.set("eps", (double)eps_);
        o.set("weight_dtype", dtype_name(weight_.dt));
        return o;
    }

private:
    long long size_;
    float eps_;
    bool one_plus_ = false;
    std::string w_name_;
    DevTensor weight_;
};

// Dynamic Tanh: out = tanh(alpha x) w + b, value by value; no mean and no
// variance is computed.  alpha is one number.
// params: size; names (optional): weight, bias, alpha: the tensors' leaves below the
// part's prefix ("" for the prefix itself)
class DynamicTanh : public Norm {
public:
    DynamicTanh(const PartSpec &s, DType dt, Device *d) : Norm(s, dt, d) {
        size_ = s.get_int("size");
        if (size_ <= 0) config_error("dynamic_tanh: size must be positive");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        w_name_ = leaf("weight", "weight");
        b_name_ = leaf("bias", "bias");
        a_name_ = leaf("alpha", "alpha");
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, w_name_), TensorSpec{{size_}, PARAM, false, 1.0f, 0.1f});
        out.emplace_back(name(prefix, b_name_), TensorSpec{{size_}, PARAM, false, 0.0f, 0.02f});
        out.emplace_back(name(prefix, a_name_), TensorSpec{{}, PARAM, false, 0.5f, 0.05f});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        w_ = take(t, name(prefix, w_name_));
        b_ = take(t, name(prefix, b_name_));
        alpha_ = take(t, name(prefix, a_name_));
    }

    size_t weight_bytes() const override { return w_.bytes() + b_.bytes() + alpha_.bytes(); }

    Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta, const int32_t *rows,
              long long n_out) override {
        ops::DytParams p;
        dynamic_tanh(&p);
        return ops::dyt(*ctx.dev, x, n, size_, p, out_dt, delta, rows, n_out);
    }

    bool dynamic_tanh(ops::DytParams *out) const override {
        out->w = (const float *)w_.ptr;
        out->b = (const float *)b_.ptr;
        out->alpha = (const float *)alpha_.ptr;
        return true;
    }

    long long size() const override { return size_; }

    Json info() const override {
        Json o = Json::object();
        o.set("size", size_);
        return o;
    }

private:
    long long size_;
    std::string w_name_, b_name_, a_name_;
    DevTensor w_, b_, alpha_;
};

// Layer norm with weight and bias: (x - mean) / sqrt(var + eps) * w + b, the variance
// being the mean of the squared deviations.  Weight and bias are kept in float32.
// params: size, eps, names (optional): weight, bias: the tensors' leaves below the
// part's prefix ("" for the prefix itself); bias null: no bias
class LayerNorm : public Norm {
public:
    LayerNorm(const PartSpec &s, DType dt, Device *d) : Norm(s, dt, d) {
        size_ = s.get_int("size");
        eps_ = (float)s.get_double("eps");
        if (size_ <= 0) config_error("layernorm: size must be positive");
        const Json &nm = s.params.get("names");
        w_name_ = nm.is_object() && nm.get("weight").is_string() ? nm.get("weight").as_string() : "weight";
        has_bias_ = !(nm.is_object() && nm.has("bias") && nm.get("bias").is_null());
        b_name_ = nm.is_object() && nm.get("bias").is_string() ? nm.get("bias").as_string() : "bias";
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        out.emplace_back(name(prefix, w_name_), TensorSpec{{size_}, PARAM, false, 1.0f, 0.1f});
        if (has_bias_) out.emplace_back(name(prefix, b_name_), TensorSpec{{size_}, PARAM, false, 0.0f, 0.02f});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        w_ = take(t, name(prefix, w_name_));
        if (has_bias_) b_ = take(t, name(prefix, b_name_));
    }

    size_t weight_bytes() const override { return w_.bytes() + b_.bytes(); }

    ops::LnParams params() const {
        ops::LnParams p;
        p.w = (const float *)w_.ptr;
        p.b = has_bias_ ? (const float *)b_.ptr : nullptr;
        p.eps = eps_;
        return p;
    }

    Buf apply(StepContext &ctx, float *x, long long n, DType out_dt, const Stack *delta, const int32_t *rows,
              long long n_out) override {
        return ops::layernorm(*ctx.dev, x, n, size_, params(), out_dt, delta, nullptr, 1.0f, rows, n_out);
    }

    Buf apply_after_add(StepContext &ctx, float *x, long long n, DType out_dt, const Stack &a, const Stack *b,
                        float mult) override {
        return ops::layernorm(*ctx.dev, x, n, size_, params(), out_dt, &a, b, mult, nullptr, 0);
    }

    bool layer_norm(ops::LnParams *out, bool *rms) const override {
        *out = params();
        *rms = false;
        return true;
    }

    long long size() const override { return size_; }

    Json info() const override {
        Json o = Json::object();
        o.set("size", size_);
        o.set("eps", (double)eps_);
        o.set("bias", has_bias_);
        return o;
    }

private:
    long long size_;
    float eps_;
    bool has_bias_ = true;
    std::string w_name_, b_name_;
    DevTensor w_, b_;
};

}  // namespace

void register_builtin_norms() {
    register_part("norm", "layernorm", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new LayerNorm(s, dt, d));
    });
    register_part("norm", "dynamic_tanh", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new DynamicTanh(s, dt, d));
    });
    register_part("norm", "rmsnorm", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new RMSNorm(s, dt, d));
    });
}

}  // namespace jb
