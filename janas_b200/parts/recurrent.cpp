// Mixers whose memory of the sequence is a state of fixed size (no keys and values).
//
// mingru: a gated running value whose gates read the current token alone,
//
//   z = sigmoid(Wz h + bz);  u = Wx h + bx;  c = u + 1/2 where u >= 0, sigmoid(u) where u < 0
//   S_t = (1 - z_t) S_{t-1} + z_t c_t   (element by element, S before the first token = 0)
//   out = Wo (S_t * silu(Wg h))
//
// z, x and g are one product over h ([z | x | g], W columns each); gates, candidate,
// the recurrence and the state are float32 in both compute types; what goes into Wo is
// rounded to the compute type.  The state [W] lives in the cache per slot and is carried
// from step to step, so prompts in portions, decoding and batches of unequal rows all
// run the same kernels (csrc/recurrent.cu).
#include "part.h"

namespace jb {

namespace {

// params: hidden_size, width, bias (default true: z and x have one), names (optional):
// z, x, g, o, bias (a suffix)
class MinGRU : public Mixer {
public:
    MinGRU(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        width_ = s.get_int("width");
        bias_ = s.has("bias") ? s.params.get("bias").as_bool() : true;
        if (hidden_ <= 0 || width_ <= 0) config_error("mingru: sizes must be positive");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_z_ = leaf("z", "z_proj.weight");
        n_x_ = leaf("x", "x_proj.weight");
        n_g_ = leaf("g", "g_proj.weight");
        n_o_ = leaf("o", "o_proj.weight");
        n_bias_ = leaf("bias", ".bias");
    }

    void tensors(const std::string &p, TensorList &out) const override {
        out.emplace_back(name(p, n_z_), TensorSpec{{width_, hidden_}, MATRIX, false});
        if (bias_) out.emplace_back(name(p, n_z_ + n_bias_), TensorSpec{{width_}, PARAM, false, 0.0f, 0.5f});
        out.emplace_back(name(p, n_x_), TensorSpec{{width_, hidden_}, MATRIX, false});
        if (bias_) out.emplace_back(name(p, n_x_ + n_bias_), TensorSpec{{width_}, PARAM, false, 0.0f, 0.5f});
        out.emplace_back(name(p, n_g_), TensorSpec{{width_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_o_), TensorSpec{{hidden_, width_}, MATRIX, false});
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> in = {take(t, name(p, n_z_)), take(t, name(p, n_x_)), take(t, name(p, n_g_))};
        w_in_ = fuse_rows(*dev, in);
        if (bias_) {
            // one vector over the product's columns; g has no bias
            std::vector<DevTensor> bs = {take(t, name(p, n_z_ + n_bias_)), take(t, name(p, n_x_ + n_bias_)),
                                         dev->tensor(F32, {width_}, true)};
            for (auto &b : bs) b.shape = {b.numel(), 1};
            b_in_ = fuse_rows(*dev, bs);
        }
        w_o_ = take(t, name(p, n_o_));
    }

    size_t weight_bytes() const override { return w_in_.bytes() + w_o_.bytes() + b_in_.bytes(); }

    StateSpec state_spec() const override { return StateSpec{{width_}, F32}; }
    bool supports(StepKind) const override { return true; }
    bool graph_safe() const override { return true; }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (!cache.state || cache.state_spec.shape.size() != 1 || cache.state_spec.shape[0] != width_)
            fail(JB_LLM_EINVAL, "mingru: the cache holds no state of this mixer's width for the layer");
        long long n = ctx.n_rows;
        Stack P = ops::linear(d, h, ctx.dtype, n, hidden_, w_in_);
        Buf a = ops::mingru(d, P, 0, width_, bias_ ? (const float *)b_in_.ptr : nullptr, (float *)cache.state,
                            ctx.row_seq, ctx.seq_slot, ctx.n_seqs, ctx.kind == DECODE, ctx.dtype);
        P = Stack();
        return ops::linear(d, a.ptr, ctx.dtype, n, width_, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("width", width_);
        return o;
    }

private:
    long long hidden_, width_;
    bool bias_;
    std::string n_z_, n_x_, n_g_, n_o_, n_bias_;
    DevTensor w_in_, b_in_, w_o_;
};

}  // namespace

void register_recurrent_mixers() {
    register_part("mixer", "mingru", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new MinGRU(s, dt, d));
    });
}

}  // namespace jb
