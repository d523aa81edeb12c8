// Mixers whose memory of the sequence is a state of fixed size (no keys and values):
// mingru, mamba2 and decay_attention (the last two are described at their classes).
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
#include <algorithm>

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

// the most rows one sequence brings to the step (0 where the host does not know: a captured step)
long long longest(const StepContext &ctx) {
    long long m = 0;
    for (long long v : ctx.seq_len) m = std::max(m, v);
    return m;
}

// A selective state space mixer in Mamba-2's form (state-space duality): H heads of P values,
// a state of N x P values per head, G groups of heads that share B and C.
//
//   [z | x | B | C | dt] = Win h        (H P, H P, G N, G N and H columns)
//   [x | B | C] <- silu(conv([x | B | C]) + b)      a causal convolution over time per column
//   dt <- softplus(dt + dt_bias)                    no clamp
//   S_t = exp(-exp(A_log_h) dt_t) S_{t-1} + dt_t B_t x_t^T;   y_t = S_t^T C_t + D_h x_t
//   out = Wo (rms in norm_groups equal parts of (y * silu(z)), times w)
//
// The state per sequence: the convolution's last taps - 1 inputs, then S, both float32.
// The steps, decays, exponentials, the recurrence and the norm are float32 in both compute
// types; what goes into Wo is rounded to the compute type.
//
// params: hidden_size, heads, head_dim (P), state (N), groups, conv_taps, norm_groups, eps,
// names (optional): in, conv, conv_bias, dt_bias, a_log, d, norm, o
class Mamba2 : public Mixer {
public:
    Mamba2(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        H_ = s.get_int("heads");
        P_ = s.get_int("head_dim");
        N_ = s.get_int("state");
        G_ = s.get_int("groups", 1);
        taps_ = (int)s.get_int("conv_taps", 1);
        parts_ = s.get_int("norm_groups", 1);
        eps_ = (float)s.get_double("eps");
        if (hidden_ <= 0 || H_ <= 0 || P_ <= 0 || N_ <= 0 || G_ <= 0) config_error("mamba2: sizes must be positive");
        if (H_ % G_) config_error("mamba2: heads must be a multiple of groups");
        if (N_ > 1024) config_error("mamba2: the recurrence's kernel takes states of up to 1024 rows");
        if (taps_ < 1) config_error("mamba2: conv_taps must be positive");
        inner_ = H_ * P_;
        if (parts_ <= 0 || inner_ % parts_) config_error("mamba2: norm_groups must divide heads * head_dim");
        conv_ = inner_ + 2 * G_ * N_;
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_in_ = leaf("in", "in_proj.weight");
        n_conv_ = leaf("conv", "conv1d.weight");
        n_conv_b_ = leaf("conv_bias", "conv1d.bias");
        n_dtb_ = leaf("dt_bias", "dt_bias");
        n_alog_ = leaf("a_log", "A_log");
        n_d_ = leaf("d", "D");
        n_norm_ = leaf("norm", "norm.weight");
        n_o_ = leaf("o", "out_proj.weight");
    }

    void tensors(const std::string &p, TensorList &out) const override {
        out.emplace_back(name(p, n_in_), TensorSpec{{2 * inner_ + 2 * G_ * N_ + H_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_conv_), TensorSpec{{conv_, taps_}, PARAM, false, 0.25f, 0.25f});
        out.emplace_back(name(p, n_conv_b_), TensorSpec{{conv_}, PARAM, false, 0.0f, 0.1f});
        out.emplace_back(name(p, n_dtb_), TensorSpec{{H_}, PARAM, false, -1.0f, 0.5f});
        out.emplace_back(name(p, n_alog_), TensorSpec{{H_}, PARAM, false, 0.0f, 0.5f});
        out.emplace_back(name(p, n_d_), TensorSpec{{H_}, PARAM, false, 1.0f, 0.1f});
        out.emplace_back(name(p, n_norm_), TensorSpec{{inner_}, PARAM, false, 1.0f, 0.1f});
        out.emplace_back(name(p, n_o_), TensorSpec{{hidden_, inner_}, MATRIX, false});
    }

    void load(const std::string &p, TensorMap &t) override {
        w_in_ = take(t, name(p, n_in_));
        conv_w_ = take(t, name(p, n_conv_));
        conv_b_ = take(t, name(p, n_conv_b_));
        dt_bias_ = take(t, name(p, n_dtb_));
        a_log_ = take(t, name(p, n_alog_));
        d_ = take(t, name(p, n_d_));
        norm_ = take(t, name(p, n_norm_));
        w_o_ = take(t, name(p, n_o_));
    }

    size_t weight_bytes() const override {
        return w_in_.bytes() + w_o_.bytes() + conv_w_.bytes() + conv_b_.bytes() + dt_bias_.bytes() + a_log_.bytes() +
               d_.bytes() + norm_.bytes();
    }

    DevTensor *first_matrix() override { return w_in_ ? &w_in_ : nullptr; }
    void share_first_product(long long col0) override {
        shared_ = true;
        col0_ = col0;
    }

    long long conv_state() const { return (long long)(taps_ - 1) * conv_; }
    StateSpec state_spec() const override { return StateSpec{{conv_state() + H_ * N_ * P_}, F32}; }
    bool strided_state() const override { return true; }
    bool graph_safe() const override { return true; }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (!cache.state || cache.state_spec.bytes() < state_spec().bytes())
            fail(JB_LLM_EINVAL, "mamba2: the cache holds no state of this mixer's size for the layer");
        long long n = ctx.n_rows;
        long long stride = cache.state_stride > 0 ? cache.state_stride : state_spec().shape[0];
        float *st = (float *)cache.state;
        Stack own;
        if (!shared_) own = ops::linear(d, h, ctx.dtype, n, hidden_, w_in_);
        else if (!ctx.shared) fail(JB_LLM_EFAIL, "mamba2: the shared first product is missing");
        const Stack &P = shared_ ? *ctx.shared : own;
        const long long c0 = shared_ ? col0_ : 0;
        // [x | B | C] through the convolution and silu, float32
        Stack xbc;
        xbc.S = 1;
        xbc.n = n;
        xbc.m = conv_;
        bool two = ctx.kind == EXTEND && taps_ > 1;
        xbc.buf = ops::causal_conv(d, P, c0 + inner_, conv_, (const float *)conv_w_.ptr, (const float *)conv_b_.ptr, taps_,
                                   st, stride, ctx.row_pos, ctx.row_seq, ctx.seq_slot, true, F32, true, !two);
        if (two)
            ops::causal_conv(d, P, c0 + inner_, conv_, (const float *)conv_w_.ptr, (const float *)conv_b_.ptr, taps_, st,
                             stride, ctx.row_pos, ctx.row_seq, ctx.seq_slot, true, F32, false, true);
        ops::MatrixScan m;
        m.H = (int)H_;
        m.G = (int)G_;
        m.N = (int)N_;
        m.P = (int)P_;
        m.val_col0 = 0;
        m.key_col0 = inner_;
        m.qry_col0 = inner_ + G_ * N_;
        m.dt = &P;
        m.dt_col0 = c0 + inner_ + conv_;
        m.dt_bias = (const float *)dt_bias_.ptr;
        m.a_log = (const float *)a_log_.ptr;
        m.skip = (const float *)d_.ptr;
        Buf y = ops::matrix_state_scan(d, xbc, m, st + conv_state(), stride, ctx.row_seq, ctx.seq_slot, ctx.n_seqs,
                                       ctx.kind == DECODE, longest(ctx));
        xbc = Stack();
        Buf a = ops::gated_part_norm(d, y.as<float>(), n, inner_, (int)parts_, &P, c0, nullptr, 0,
                                     (const float *)norm_.ptr, eps_, ctx.dtype, ctx.kind == DECODE && ctx.dtype == BF16);
        own = Stack();
        return ops::linear(d, a.ptr, ctx.dtype, n, inner_, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("inner", inner_);
        o.set("state_floats", state_spec().shape[0]);
        return o;
    }

private:
    long long hidden_, H_, P_, N_, G_, parts_, inner_ = 0, conv_ = 0;
    int taps_;
    float eps_;
    std::string n_in_, n_conv_, n_conv_b_, n_dtb_, n_alog_, n_d_, n_norm_, n_o_;
    DevTensor w_in_, w_o_, conv_w_, conv_b_, dt_bias_, a_log_, d_, norm_;
    bool shared_ = false;        // the in-product's rows went into a pair's shared first product
    long long col0_ = 0;
};

// Linear attention with a fixed decay per head (lightning attention's recurrence): H heads,
// D query/key values and Dv values a head, a state of D x Dv values per head.
//
//   q = silu(Wq h), k = silu(Wk h), v = silu(Wv h)       laid out head by head
//   S_t = decay_a S_{t-1} + k_t v_t^T;   o_t = S_t^T q_t          no other scale
//   out = Wo (rms(all heads of o) w * sigmoid(Wg h))
//
// q, k, v and the gate are one product over h; the recurrence, the state and the norm are
// float32 in both compute types.
//
// params: hidden_size, heads, head_dim (D), v_head_dim (Dv, default D), decay (a list of one
// number per head), eps, names (optional): q, k, v, g, o, norm
class DecayAttention : public Mixer {
public:
    DecayAttention(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        H_ = s.get_int("heads");
        D_ = s.get_int("head_dim");
        Dv_ = s.get_int("v_head_dim", D_);
        eps_ = (float)s.get_double("eps");
        if (hidden_ <= 0 || H_ <= 0 || D_ <= 0 || Dv_ <= 0) config_error("decay_attention: sizes must be positive");
        if (D_ > 1024) config_error("decay_attention: the recurrence's kernel takes heads of up to 1024 values");
        const Json &dc = s.params.get("decay");
        if (!dc.is_array() || (long long)dc.size() != H_)
            config_error("decay_attention: decay must list one number per head");
        for (size_t i = 0; i < dc.size(); i++) {
            if (!dc[i].is_number()) config_error("decay_attention: decay must list numbers");
            decay_host_.push_back((float)dc[i].as_double());
        }
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_q_ = leaf("q", "q_proj.weight");
        n_k_ = leaf("k", "k_proj.weight");
        n_v_ = leaf("v", "v_proj.weight");
        n_g_ = leaf("g", "g_proj.weight");
        n_o_ = leaf("o", "o_proj.weight");
        n_norm_ = leaf("norm", "norm.weight");
    }

    void tensors(const std::string &p, TensorList &out) const override {
        out.emplace_back(name(p, n_q_), TensorSpec{{H_ * D_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_k_), TensorSpec{{H_ * D_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_v_), TensorSpec{{H_ * Dv_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_g_), TensorSpec{{H_ * Dv_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_o_), TensorSpec{{hidden_, H_ * Dv_}, MATRIX, false});
        out.emplace_back(name(p, n_norm_), TensorSpec{{H_ * Dv_}, PARAM, false, 1.0f, 0.1f});
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> in = {take(t, name(p, n_q_)), take(t, name(p, n_k_)), take(t, name(p, n_v_)),
                                     take(t, name(p, n_g_))};
        w_in_ = fuse_rows(*dev, in);
        w_o_ = take(t, name(p, n_o_));
        norm_ = take(t, name(p, n_norm_));
        decay_ = dev->tensor(F32, {H_});
        cuda_check(cudaMemcpy(decay_.ptr, decay_host_.data(), decay_host_.size() * 4, cudaMemcpyHostToDevice),
                   "copying the heads' decays");
    }

    size_t weight_bytes() const override { return w_in_.bytes() + w_o_.bytes() + norm_.bytes() + decay_.bytes(); }

    DevTensor *first_matrix() override { return w_in_ ? &w_in_ : nullptr; }
    void share_first_product(long long col0) override {
        shared_ = true;
        col0_ = col0;
    }

    StateSpec state_spec() const override { return StateSpec{{H_ * D_ * Dv_}, F32}; }
    bool strided_state() const override { return true; }
    bool graph_safe() const override { return true; }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (!cache.state || cache.state_spec.bytes() < state_spec().bytes())
            fail(JB_LLM_EINVAL, "decay_attention: the cache holds no state of this mixer's size for the layer");
        long long n = ctx.n_rows;
        long long stride = cache.state_stride > 0 ? cache.state_stride : state_spec().shape[0];
        Stack own;
        if (!shared_) own = ops::linear(d, h, ctx.dtype, n, hidden_, w_in_);
        else if (!ctx.shared) fail(JB_LLM_EFAIL, "decay_attention: the shared first product is missing");
        const Stack &P = shared_ ? *ctx.shared : own;
        const long long c0 = shared_ ? col0_ : 0;
        ops::MatrixScan m;
        m.H = (int)H_;
        m.G = (int)H_;
        m.N = (int)D_;
        m.P = (int)Dv_;
        m.qry_col0 = c0;
        m.key_col0 = c0 + H_ * D_;
        m.val_col0 = c0 + 2 * H_ * D_;
        m.silu = true;
        m.decay = (const float *)decay_.ptr;
        // Many rows: q, k and v are activated once, ahead of the recurrence, whose blocks would
        // otherwise each activate the rows they read (several blocks read the same k and q).
        Stack act;
        if (ctx.kind != DECODE && n >= 64) {
            act.buf = ops::activation(d, P, 2 * H_ * D_ + H_ * Dv_, ops::activation_kind("silu"), F32, c0);
            act.S = 1;
            act.n = n;
            act.m = 2 * H_ * D_ + H_ * Dv_;
            m.silu = false;
            m.qry_col0 = 0;
            m.key_col0 = H_ * D_;
            m.val_col0 = 2 * H_ * D_;
        }
        Buf y = ops::matrix_state_scan(d, act ? act : P, m, (float *)cache.state, stride, ctx.row_seq, ctx.seq_slot,
                                       ctx.n_seqs, ctx.kind == DECODE, longest(ctx));
        act = Stack();
        Buf a = ops::gated_part_norm(d, y.as<float>(), n, H_ * Dv_, 1, nullptr, 0, &P, c0 + 2 * H_ * D_ + H_ * Dv_,
                                     (const float *)norm_.ptr, eps_, ctx.dtype, ctx.kind == DECODE && ctx.dtype == BF16);
        own = Stack();
        return ops::linear(d, a.ptr, ctx.dtype, n, H_ * Dv_, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("state_floats", state_spec().shape[0]);
        return o;
    }

private:
    long long hidden_, H_, D_, Dv_;
    float eps_;
    std::vector<float> decay_host_;
    std::string n_q_, n_k_, n_v_, n_g_, n_o_, n_norm_;
    DevTensor w_in_, w_o_, norm_, decay_;
    bool shared_ = false;        // the [q | k | v | g] rows went into a pair's shared first product
    long long col0_ = 0;
};

}  // namespace

void register_recurrent_mixers() {
    register_part("mixer", "mamba2", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new Mamba2(s, dt, d));
    });
    register_part("mixer", "decay_attention", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new DecayAttention(s, dt, d));
    });
    register_part("mixer", "mingru", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new MinGRU(s, dt, d));
    });
}

}  // namespace jb
