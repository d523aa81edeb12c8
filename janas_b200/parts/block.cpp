// Block arrangements.
//
// prenorm: x += mixer(norm(x)); x += ffn(norm(x))  (src/llm/model.c:743-796).
//
// parallel: one norm, both sublayers read its output, and their results join the
// residual stream together, times a factor:
//     h = norm(x);  x += m * (mixer(h) + ffn(h))       (ffn(h) = 0 for a layer without one)
//
// sandwich: a norm before and after each sublayer, and optionally a gate on the
// sublayer's result, computed from the sublayer's own input:
//     h = norm_in(x);  y = sublayer(h);  y *= sigmoid(G h + g);  x += norm_out(y)
// for the mixer and then, where the layer has one, for the feed-forward.
//
// result_norm: no norm in front of a sublayer, one on its result alone; the sublayers read
// the residual stream itself, optionally through a short causal convolution over time on
// every channel (weights [hidden, taps], no bias):
//     h = x + conv(x);  x += norm(sublayer(h))          conv(x)_t = sum_j w[:, j] x_{t - taps + 1 + j}
// for the mixer and then, where the layer has one, for the feed-forward.  The last
// taps - 1 inputs of either convolution are state of the sequence (float32, per slot).
#include "part.h"

namespace jb {

namespace {

class PreNormBlock : public Block {
public:
    explicit PreNormBlock(BlockParts p) : Block(std::move(p)) {
        if (!mixer_norm) config_error("prenorm: the layer needs a norm in front of its mixer");
        if (!feed_forward || !ffn_norm) config_error("prenorm: the layer needs a feed-forward and its norm");
        if (post_mixer_norm || post_ffn_norm) config_error("prenorm: the arrangement has no norms on results");
    }
    void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) override {
        long long n = ctx.n_rows;
        // the add of what the previous part produced is fused into the norm
        Buf h = mixer_norm->apply(ctx, x, n, ctx.dtype, pending ? &pending : nullptr, nullptr, 0);
        Stack d = mixer->forward(ctx, h.ptr, cache);
        h = ffn_norm->apply(ctx, x, n, ctx.dtype, &d, nullptr, 0);
        pending = feed_forward->forward(ctx, h.ptr);
    }
};

// block_params: residual_mult (default 1): the factor m on the sublayers' sum.
// The add is left to the norm that meets the residual stream next where the model
// names one (Block::next_norm): its result then waits in ctx.normed.
class ParallelBlock : public Block {
public:
    ParallelBlock(BlockParts p, const LayerSpec &ls) : Block(std::move(p)) {
        if (!mixer_norm) config_error("parallel: the layer needs its norm");
        if (ffn_norm || post_mixer_norm || post_ffn_norm)
            config_error("parallel: the arrangement has one norm, before both sublayers");
        const Json &m = ls.block_params.get("residual_mult");
        mult_ = m.is_number() ? (float)m.as_double() : 1.0f;
    }

    void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) override {
        long long n = ctx.n_rows;
        Buf h;
        if (ctx.normed && ctx.normed_by == mixer_norm.get()) {
            if (pending) fail(JB_LLM_EFAIL, "parallel: a norm was computed ahead of a pending sum");
            h = std::move(ctx.normed);
        } else {
            h = mixer_norm->apply(ctx, x, n, ctx.dtype, pending ? &pending : nullptr, nullptr, 0);
        }
        ctx.normed.reset();
        ctx.normed_by = nullptr;
        pending = Stack();
        Stack y = mixer->forward(ctx, h.ptr, cache);
        Stack z;
        if (feed_forward) z = feed_forward->forward(ctx, h.ptr);
        if (next_norm) {
            ctx.normed = const_cast<Norm *>(next_norm)->apply_after_add(ctx, x, n, ctx.dtype, y,
                                                                        z ? &z : nullptr, mult_);
            ctx.normed_by = next_norm;
        } else {
            ops::add_scaled_(*ctx.dev, x, n, ctx.hidden, y, z ? &z : nullptr, mult_);
        }
    }

private:
    float mult_ = 1.0f;
};

// block_params: hidden_size; mixer_gate / ffn_gate: the tensor names (below the
// layer's prefix) of the gates' matrices [hidden, hidden], absent or null for no
// gate; gate_bias: the suffix of a gate's bias vector ("" for none); fuse (default
// true): false runs gate, norm and add as kernels of their own; token_side (optional):
// {dim, col0, eps, names {gate, proj, norm}}: an input of the token's own after the sublayers,
// from columns col0 .. col0 + dim - 1 of the model's token table (see token_side()).
class SandwichBlock : public Block {
public:
    SandwichBlock(BlockParts p, const LayerSpec &ls, DType dt, Device *d) : Block(std::move(p)), dev_(d) {
        if (!mixer_norm) config_error("sandwich: the mixer needs a norm in front of it");
        if (!post_mixer_norm || (feed_forward && !post_ffn_norm))
            config_error("sandwich: every sublayer needs a norm on its result");
        if (feed_forward && !ffn_norm) config_error("sandwich: the feed-forward needs its norm");
        const Json &bp = ls.block_params;
        hidden_ = bp.get("hidden_size").is_number() ? bp.get("hidden_size").as_int() : mixer_norm->size();
        if (bp.get("mixer_gate").is_string()) gate_name_[0] = bp.get("mixer_gate").as_string();
        if (bp.get("ffn_gate").is_string() && feed_forward) gate_name_[1] = bp.get("ffn_gate").as_string();
        if (bp.get("gate_bias").is_string()) bias_suffix_ = bp.get("gate_bias").as_string();
        if (bp.get("fuse").is_bool()) fuse_ = bp.get("fuse").as_bool();
        const Json &ts = bp.get("token_side");
        if (ts.is_object()) {
            PartSpec tp{"sandwich: token_side", ts};
            side_dim_ = tp.get_int("dim");
            side_col0_ = tp.get_int("col0", 0);
            side_eps_ = (float)tp.get_double("eps");
            if (side_dim_ <= 0 || side_col0_ < 0) config_error("sandwich: token_side needs dim > 0 and col0 >= 0");
            const Json &nm = ts.get("names");
            auto leaf = [&](const char *key, const char *dflt) {
                return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
            };
            side_name_[0] = leaf("gate", "side.gate");
            side_name_[1] = leaf("proj", "side.proj");
            side_name_[2] = leaf("norm", "side.norm");
        }
        // tensors of an absent feed-forward's surroundings that a file may still
        // hold: tolerated and not read
        if (!feed_forward)
            for (auto &v : bp.get("unused").items())
                if (v.is_object() && v.get("name").is_string()) {
                    std::vector<long long> shape;
                    for (auto &s : v.get("shape").items()) shape.push_back(s.as_int());
                    unused_.emplace_back(v.get("name").as_string(), shape);
                }
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        for (int i = 0; i < 2; i++) {
            if (gate_name_[i].empty()) continue;
            out.emplace_back(Part::name(prefix, gate_name_[i]), TensorSpec{{hidden_, hidden_}, MATRIX, false});
            if (!bias_suffix_.empty())
                out.emplace_back(Part::name(prefix, gate_name_[i] + bias_suffix_),
                                 TensorSpec{{hidden_}, PARAM, false, 0.0f, 0.02f});
        }
        if (side_dim_ > 0) {
            out.emplace_back(Part::name(prefix, side_name_[0]), TensorSpec{{side_dim_, hidden_}, MATRIX, false});
            out.emplace_back(Part::name(prefix, side_name_[1]), TensorSpec{{hidden_, side_dim_}, MATRIX, false});
            out.emplace_back(Part::name(prefix, side_name_[2]), TensorSpec{{hidden_}, PARAM, false, 1.0f, 0.1f});
        }
        for (auto &u : unused_)
            out.emplace_back(Part::name(prefix, u.first),
                             TensorSpec{u.second, u.second.size() == 2 ? MATRIX : PARAM, true});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        for (int i = 0; i < 2; i++) {
            if (gate_name_[i].empty()) continue;
            gate_[i] = Part::take(t, Part::name(prefix, gate_name_[i]));
            if (!bias_suffix_.empty()) gate_bias_[i] = Part::take(t, Part::name(prefix, gate_name_[i] + bias_suffix_));
            // the gate reads what its sublayer reads: one product for both, where the part can
            if (fuse_) {
                Part *p = i == 0 ? (Part *)mixer.get() : (Part *)feed_forward.get();
                in_part_[i] = p->take_side_rows(gate_[i]);
            }
        }
        if (side_dim_ > 0)
            for (int i = 0; i < 3; i++) side_w_[i] = Part::take(t, Part::name(prefix, side_name_[i]));
        for (auto &u : unused_) t.erase(Part::name(prefix, u.first));
    }

    size_t weight_bytes() const override {
        // a gate that went into its sublayer's first product is counted there
        return gate_[0].bytes() + gate_[1].bytes() + gate_bias_[0].bytes() + gate_bias_[1].bytes() +
               side_w_[0].bytes() + side_w_[1].bytes() + side_w_[2].bytes();
    }

    void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) override {
        long long n = ctx.n_rows;
        Buf h = take_normed(ctx, mixer_norm.get());
        if (!h) h = mixer_norm->apply(ctx, x, n, ctx.dtype, pending ? &pending : nullptr, nullptr, 0);
        else if (pending) fail(JB_LLM_EFAIL, "sandwich: a norm was computed ahead of a pending sum");
        pending = Stack();
        {
            Stack g = gate_product(ctx, 0, h.ptr);
            Stack y = mixer->forward(ctx, h.ptr, cache);
            long long col0 = take_side(ctx, 0, g);
            // what the token's own input changes afterwards cannot be normed ahead
            const Norm *next = feed_forward ? ffn_norm.get() : side_dim_ > 0 ? nullptr : next_norm;
            finish(ctx, x, y, g, col0, 0, post_mixer_norm.get(), next);
        }
        if (!feed_forward) {
            token_side(ctx, x);
            return;
        }
        h = take_normed(ctx, ffn_norm.get());
        if (!h) h = ffn_norm->apply(ctx, x, n, ctx.dtype, nullptr, nullptr, 0);
        {
            Stack g = gate_product(ctx, 1, h.ptr);
            Stack y = feed_forward->forward(ctx, h.ptr);
            long long col0 = take_side(ctx, 1, g);
            finish(ctx, x, y, g, col0, 1, post_ffn_norm.get(), side_dim_ > 0 ? nullptr : next_norm);
        }
        token_side(ctx, x);
    }

private:
    static Buf take_normed(StepContext &ctx, const Norm *by) {
        if (!ctx.normed || ctx.normed_by != by) {
            ctx.normed.reset();
            ctx.normed_by = nullptr;
            return Buf();
        }
        ctx.normed_by = nullptr;
        return std::move(ctx.normed);
    }

    // the gate's values out of the sublayer's own first product, where they went into it
    long long take_side(StepContext &ctx, int which, Stack &g) {
        if (!in_part_[which]) return 0;
        if (!ctx.side) fail(JB_LLM_EFAIL, "sandwich: the sublayer took the gate's rows and left no product");
        g = std::move(ctx.side);
        ctx.side = Stack();
        return ctx.side_col0;
    }

    Stack gate_product(StepContext &ctx, int which, const void *h) {
        if (!gate_[which]) return Stack();
        return ops::linear(*ctx.dev, h, ctx.dtype, ctx.n_rows, hidden_, gate_[which]);
    }

    // x += norm_out(y * gate); the next norm of x too where both norms work value by
    // value (its result then waits in ctx.normed)
    void finish(StepContext &ctx, float *x, Stack &y, const Stack &g, long long col0, int which, Norm *post,
                const Norm *next) {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        const float *g_bias = gate_bias_[which] ? (const float *)gate_bias_[which].ptr : nullptr;
        ops::DytParams pp, np;
        if (fuse_ && g && post->dynamic_tanh(&pp)) {
            bool fuse_next = next && next->dynamic_tanh(&np);
            Buf out = ops::gated_dyt_residual(d, x, y, g, col0, g_bias, pp, fuse_next ? &np : nullptr, ctx.dtype);
            if (fuse_next) {
                ctx.normed = std::move(out);
                ctx.normed_by = next;
            }
            return;
        }
        ops::LnParams lp;
        bool rms = false;
        if (fuse_ && !g && post->layer_norm(&lp, &rms)) {
            // no gate and a norm whose kernel adds its result: sums, norm and add in one pass
            ops::norm_residual_(d, x, y, lp, rms, ctx.kind == DECODE && ctx.dtype == BF16);
            return;
        }
        // the steps one by one, for any norm: gate, norm of the result, add
        Buf t;
        Stack one;
        if (g) {
            t = ops::gate_mul(d, y, g, col0, g_bias);
        } else {
            t = d.pool.get((size_t)n * (size_t)hidden_ * 4);
            cuda_check(cudaMemsetAsync(t.ptr, 0, t.bytes, d.stream), "clearing a sum");
            ops::add_(d, t.as<float>(), n, hidden_, y);
        }
        one.buf = post->apply(ctx, t.as<float>(), n, F32, nullptr, nullptr, 0);
        one.S = 1;
        one.n = n;
        one.m = hidden_;
        ops::add_(d, x, n, hidden_, one);
    }

    // The token's own input to the layer, after the sublayers: with e = the token's row of the
    // model's token table, columns col0 .. col0 + dim - 1,
    //   y = P (gelu_tanh(G x) * e);   x += rms(y) w        (a plain weight, eps inside the root)
    void token_side(StepContext &ctx, float *x) {
        if (side_dim_ <= 0) return;
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        if (!ctx.token_table || !ctx.tokens)
            fail(JB_LLM_EINVAL, "sandwich: the model has no token table for the layers' token input");
        if (side_col0_ + side_dim_ > ctx.token_table->shape.at(1))
            fail(JB_LLM_EINVAL, "sandwich: the layer's columns lie outside the token table");
        Buf hx;
        const void *in = x;
        if (ctx.dtype != F32) {
            hx = d.pool.get((size_t)n * (size_t)hidden_ * dtype_size(ctx.dtype));
            if (jb_convert(x, F32, hx.ptr, ctx.dtype, n * hidden_, d.stream) != 0)
                fail(JB_LLM_EFAIL, "sandwich: the conversion could not be launched");
            in = hx.ptr;
        }
        Stack P = ops::linear(d, in, ctx.dtype, n, hidden_, side_w_[0]);
        Buf gt = ops::token_gate(d, P, *ctx.token_table, side_col0_, side_dim_, ctx.tokens, ctx.dtype);
        P = Stack();
        Stack y = ops::linear(d, gt.ptr, ctx.dtype, n, side_dim_, side_w_[1]);
        ops::LnParams lp;
        lp.w = (const float *)side_w_[2].ptr;
        lp.eps = side_eps_;
        ops::norm_residual_(d, x, y, lp, true, ctx.kind == DECODE && ctx.dtype == BF16);
    }

    Device *dev_;
    long long hidden_ = 0;
    long long side_dim_ = 0, side_col0_ = 0;
    float side_eps_ = 0.0f;
    std::string side_name_[3];
    DevTensor side_w_[3];
    bool fuse_ = true;      // false: every step as a kernel of its own (for comparisons)
    std::string gate_name_[2], bias_suffix_;
    DevTensor gate_[2], gate_bias_[2];
    bool in_part_[2] = {false, false};     // the gate's rows lie in the sublayer's first product
    std::vector<std::pair<std::string, std::vector<long long>>> unused_;
};

// block_params: hidden_size; conv_taps (0 or absent: the sublayers read x as it is);
// mixer_conv / ffn_conv: the tensor names (below the layer's prefix) of the convolutions'
// weights.  The norms are the layer's post_mixer_norm and post_ffn_norm; it has no others.
class ResultNormBlock : public Block {
public:
    ResultNormBlock(BlockParts p, const LayerSpec &ls) : Block(std::move(p)) {
        if (mixer_norm || ffn_norm) config_error("result_norm: the arrangement has no norm in front of a sublayer");
        if (!post_mixer_norm || (feed_forward && !post_ffn_norm))
            config_error("result_norm: every sublayer needs a norm on its result");
        const Json &bp = ls.block_params;
        hidden_ = bp.get("hidden_size").is_number() ? bp.get("hidden_size").as_int() : post_mixer_norm->size();
        taps_ = bp.get("conv_taps").is_number() ? (int)bp.get("conv_taps").as_int() : 0;
        if (taps_ < 0) config_error("result_norm: conv_taps must not be negative");
        conv_name_[0] = bp.get("mixer_conv").is_string() ? bp.get("mixer_conv").as_string() : "mixer_conv";
        conv_name_[1] = bp.get("ffn_conv").is_string() ? bp.get("ffn_conv").as_string() : "ffn_conv";
        n_sub_ = feed_forward ? 2 : 1;
    }

    void tensors(const std::string &prefix, TensorList &out) const override {
        if (!taps_) return;
        for (int i = 0; i < n_sub_; i++)
            out.emplace_back(Part::name(prefix, conv_name_[i]), TensorSpec{{hidden_, taps_}, PARAM, false, 0.0f, 0.2f});
    }

    void load(const std::string &prefix, TensorMap &t) override {
        if (!taps_) return;
        for (int i = 0; i < n_sub_; i++) conv_[i] = Part::take(t, Part::name(prefix, conv_name_[i]));
    }

    size_t weight_bytes() const override { return conv_[0].bytes() + conv_[1].bytes(); }

    // the last taps - 1 inputs of each sublayer's convolution
    StateSpec state_spec() const override {
        if (taps_ < 2) return StateSpec();
        return StateSpec{{n_sub_, taps_ - 1, hidden_}, F32};
    }

    void forward(StepContext &ctx, float *x, Stack &pending, LayerCache &cache) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        ctx.normed.reset();
        ctx.normed_by = nullptr;
        if (pending) {
            ops::add_(d, x, n, hidden_, pending);
            pending = Stack();
        }
        if (taps_ >= 2 && (!cache.block_state || cache.block_state_spec.bytes() != state_spec().bytes()))
            fail(JB_LLM_EINVAL, "result_norm: the cache holds no state for the layer's convolutions");
        bool few = ctx.kind == DECODE && ctx.dtype == BF16;
        for (int i = 0; i < n_sub_; i++) {
            Buf h = read(ctx, x, i, cache);
            Stack y = i == 0 ? mixer->forward(ctx, h ? h.ptr : x, cache)
                             : feed_forward->forward(ctx, h ? h.ptr : x);
            Norm *post = i == 0 ? post_mixer_norm.get() : post_ffn_norm.get();
            ops::LnParams lp;
            bool rms = false;
            if (post->layer_norm(&lp, &rms)) {
                ops::norm_residual_(d, x, y, lp, rms, few);
            } else {
                // any other norm: the result summed, normed, added
                Buf t = d.pool.get((size_t)n * (size_t)hidden_ * 4);
                cuda_check(cudaMemsetAsync(t.ptr, 0, t.bytes, d.stream), "clearing a sum");
                ops::add_(d, t.as<float>(), n, hidden_, y);
                Stack one;
                one.buf = post->apply(ctx, t.as<float>(), n, F32, nullptr, nullptr, 0);
                one.S = 1;
                one.n = n;
                one.m = hidden_;
                ops::add_(d, x, n, hidden_, one);
            }
        }
    }

private:
    // what sublayer i reads: x through its convolution in the compute type (an empty
    // handle: x itself, float32 compute and no convolution)
    Buf read(StepContext &ctx, float *x, int i, LayerCache &cache) {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        if (!taps_) {
            if (ctx.dtype == F32) return Buf();
            Buf h = d.pool.get((size_t)n * (size_t)hidden_ * dtype_size(ctx.dtype));
            if (jb_convert(x, F32, h.ptr, ctx.dtype, n * hidden_, d.stream) != 0)
                fail(JB_LLM_EFAIL, "result_norm: the conversion could not be launched");
            return h;
        }
        float *st = taps_ >= 2 ? (float *)cache.block_state + (size_t)i * (size_t)(taps_ - 1) * (size_t)hidden_
                               : nullptr;
        // A slot's state is [n_sub, taps - 1, hidden]: the kernel takes the stride between
        // slots from the sublayers' count.
        const float *w = (const float *)conv_[i].ptr;
        long long slot_stride = (long long)n_sub_ * (taps_ - 1) * hidden_;
        if (ctx.kind == EXTEND && taps_ >= 2) {
            // rows read inputs of earlier steps that other rows of this step replace: two launches
            Buf h = ops::short_conv(d, x, n, hidden_, w, taps_, st, slot_stride, ctx.row_pos, ctx.row_seq,
                                    ctx.seq_slot, ctx.dtype, true, false);
            ops::short_conv(d, x, n, hidden_, w, taps_, st, slot_stride, ctx.row_pos, ctx.row_seq, ctx.seq_slot,
                            ctx.dtype, false, true);
            return h;
        }
        return ops::short_conv(d, x, n, hidden_, w, taps_, st, slot_stride, ctx.row_pos, ctx.row_seq, ctx.seq_slot,
                               ctx.dtype, true, taps_ >= 2);
    }

    long long hidden_ = 0;
    int taps_ = 0, n_sub_ = 1;
    std::string conv_name_[2];
    DevTensor conv_[2];
};

}  // namespace

void register_builtin_blocks() {
    register_block("result_norm", [](BlockParts p, const LayerSpec &ls, DType, Device *) {
        return std::unique_ptr<Block>(new ResultNormBlock(std::move(p), ls));
    });
    register_block("prenorm", [](BlockParts p, const LayerSpec &, DType, Device *) {
        return std::unique_ptr<Block>(new PreNormBlock(std::move(p)));
    });
    register_block("parallel", [](BlockParts p, const LayerSpec &ls, DType, Device *) {
        return std::unique_ptr<Block>(new ParallelBlock(std::move(p), ls));
    });
    register_block("sandwich", [](BlockParts p, const LayerSpec &ls, DType dt, Device *d) {
        return std::unique_ptr<Block>(new SandwichBlock(std::move(p), ls, dt, d));
    });
}

}  // namespace jb
