// Grouped-query attention with optional per-head q/k RMSNorm, a position
// encoding and an optional sliding window.
//
// In order: q, k, v products without biases; per head, RMSNorm of q and of k with
// one weight vector for all heads, before the rotation; the rotation; K and V into
// the cache at the row's position; causal attention, head h reading KV head
// h / (heads / kv_heads), scores scaled by 1/sqrt(head size); the output product
// (src/llm/model_attn.c:75-146,224-285; src/llm/attention.c:874-875,1012).  With a
// window w a token at position p sees positions p + 1 - w .. p
// (src/llm/attention.c:736-739).
#include <cmath>

#include "part.h"

namespace jb {

namespace {

// params: hidden_size, num_heads, num_kv_heads, head_dim, qk_norm_eps (null: no
// q/k norm), window (0: none), position (a part)
class GQAAttention : public Mixer {
public:
    GQAAttention(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        g_.nh = (int)s.get_int("num_heads");
        g_.nkv = (int)s.get_int("num_kv_heads");
        g_.hd = (int)s.get_int("head_dim");
        qk_norm_ = s.has("qk_norm_eps");
        qk_eps_ = qk_norm_ ? (float)s.get_double("qk_norm_eps") : 0.0f;
        g_.window = (int)s.get_int("window", 0);
        if (hidden_ <= 0 || g_.nh <= 0 || g_.nkv <= 0) config_error("gqa_attention: sizes must be positive");
        if (g_.nh % g_.nkv) config_error("gqa_attention: num_heads must be a multiple of num_kv_heads");
        if (g_.hd % 16 || g_.hd < 16 || g_.hd > 512)
            config_error(fmt("gqa_attention: head_dim %d: the kernels take head sizes from 16 to 512 in "
                             "steps of 16", g_.hd));
        if (g_.window < 0) config_error("gqa_attention: window must not be negative");
        position_ = build_position(s.get_part("position"), dt, d);
        if (position_->rotary_dim() != 0 && position_->rotary_dim() != g_.hd)
            config_error(fmt("gqa_attention: only the whole head can be rotated (rotary_dim %d, "
                             "head_dim %d)", position_->rotary_dim(), g_.hd));
        g_.scale = (float)(1.0 / std::sqrt((double)g_.hd));
    }

    // ------------------------------------------------------------- weights
    void tensors(const std::string &p, TensorList &out) const override {
        long long hd = g_.hd;
        out.emplace_back(name(p, "q_proj.weight"), TensorSpec{{g_.nh * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "k_proj.weight"), TensorSpec{{g_.nkv * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "v_proj.weight"), TensorSpec{{g_.nkv * hd, hidden_}, MATRIX, false});
        out.emplace_back(name(p, "o_proj.weight"), TensorSpec{{hidden_, g_.nh * hd}, MATRIX, false});
        if (qk_norm_) {
            out.emplace_back(name(p, "q_norm.weight"), TensorSpec{{hd}, NORM, false});
            out.emplace_back(name(p, "k_norm.weight"), TensorSpec{{hd}, NORM, false});
        }
        position_->tensors(name(p, "position"), out);
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> qkv = {take(t, name(p, "q_proj.weight")), take(t, name(p, "k_proj.weight")),
                                      take(t, name(p, "v_proj.weight"))};
        w_qkv_ = fuse_rows(*dev, qkv);
        w_o_ = take(t, name(p, "o_proj.weight"));
        if (qk_norm_) {
            q_norm_ = take(t, name(p, "q_norm.weight"));
            k_norm_ = take(t, name(p, "k_norm.weight"));
            if (q_norm_.dt != k_norm_.dt) {
                // one kernel reads both: the wider type for both
                std::vector<DevTensor *> both = {&q_norm_, &k_norm_};
                for (DevTensor *w : both) {
                    if (w->dt == F32) continue;
                    DevTensor wide = dev->tensor(F32, w->shape);
                    if (jb_convert(w->ptr, w->dt, wide.ptr, F32, w->numel(), dev->stream) != 0)
                        fail(JB_LLM_EFAIL, "gqa_attention: widening a norm weight failed");
                    dev->sync();
                    *w = wide;
                }
            }
        }
        position_->load(name(p, "position"), t);
    }

    size_t weight_bytes() const override {
        return w_qkv_.bytes() + w_o_.bytes() + q_norm_.bytes() * (qk_norm_ ? 2 : 0);
    }

    // --------------------------------------------------------------- cache
    KVSpec kv_spec() const override { return KVSpec{g_.nkv, g_.hd, g_.window}; }

    void prepare(long long n_positions) override {
        position_->prepare(n_positions);
        chunk_ = ops::attention_chunk();
    }

    // Every kind of step, with a window too: the pages a window group gives back
    // after a step are those that the sequence's NEXT token cannot see, and tokens
    // appended later see no further back than that one.
    bool supports(StepKind) const override { return true; }

    // everything that changes from step to step is read from device arrays, so a
    // captured decode step can be replayed
    bool graph_safe() const override { return true; }

    // ------------------------------------------------------------- forward
    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (ctx.max_pos >= position_->n_positions())
            fail(JB_LLM_EINVAL, fmt("position %lld is beyond the %lld positions the encoding was prepared "
                                    "for", ctx.max_pos, position_->n_positions()));
        if (!chunk_) chunk_ = ops::attention_chunk();
        long long n = ctx.n_rows;
        const DevTensor *qw = qk_norm_ ? &q_norm_ : nullptr, *kw = qk_norm_ ? &k_norm_ : nullptr;
        Stack qkv = ops::linear(d, h, ctx.dtype, n, hidden_, w_qkv_);
        int max_chunks = (int)(ctx.max_pos / chunk_ + 1);
        if (g_.window) max_chunks = std::min(max_chunks, (g_.window - 1) / chunk_ + 2);
        Buf a;
        if (ctx.kind == DECODE && ctx.dtype == BF16) {
            // one new token per sequence: the attention kernel makes q and the new key
            // and value from the product's sums itself, where it takes the sizes
            a = ops::attention_decode_qkv(d, qkv, qw, kw, qk_eps_, position_->cos(), position_->sin(),
                                          cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks);
        }
        if (!a) {
            Buf q = ops::qk_norm_rope_append(d, qkv, qw, kw, qk_eps_, position_->cos(), position_->sin(),
                                             ctx.row_pos, ctx.row_seq, cache.kv, g_, ctx.dtype);
            qkv.buf.reset();
            bool decode = ctx.kind == DECODE;
            const int32_t *blocks = nullptr;
            int n_blocks = 0;
            if (!decode && ctx.dtype == BF16 && ops::attention_tc_ok(g_.nh, g_.nkv, g_.hd) &&
                !ctx.seq_len.empty()) {
                // runs of consecutive positions, for the tensor-core kernel; the same
                // for every layer of the step with this grouping of heads
                int per = ops::attention_block_positions(g_.nh, g_.nkv);
                std::string key = "attention_blocks/" + std::to_string(per);
                auto it = ctx.extras.find(key);
                if (it == ctx.extras.end()) {
                    StepContext::Extra e;
                    e.buf = ops::attention_blocks(d, ctx.seq_row0.data(), ctx.seq_pos0.data(),
                                                  ctx.seq_len.data(), ctx.n_seqs, per, &e.n);
                    it = ctx.extras.emplace(key, std::move(e)).first;
                }
                blocks = it->second.buf.as<int32_t>();
                n_blocks = it->second.n;
            }
            a = ops::attention(d, q.ptr, n, cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks, blocks,
                               n_blocks, decode);
        }
        return ops::linear(d, a.ptr, ctx.dtype, n, (long long)g_.nh * g_.hd, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("position", position_->info());
        o.set("position_kind", position_->spec.kind);
        return o;
    }

private:
    long long hidden_;
    ops::AttnGeometry g_;
    bool qk_norm_;
    float qk_eps_;
    std::unique_ptr<PositionEncoding> position_;
    DevTensor w_qkv_, w_o_, q_norm_, k_norm_;
    int chunk_ = 0;
};

// Grouped-query attention without a rotation, with what some designs add to it:
// biases on the four products, a scale given as a constant, a learned factor per
// head on the scores, a learned sink per head in the softmax's denominator, values
// of another head size than the keys, and keys and values taken from another
// layer's cache.
//
//   q = Wq h + bq, k = Wk h + bk, v = Wv h + bv            (k, v only with own_kv)
//   s_ij = (q_i . k_j) * scale * temp_a,  j <= i  (and within the window, if any)
//   p_ij = exp(s_ij) / (exp(sink_a) + sum_j exp(s_ij));   out = Wo concat(p v) + bo
//
// Further, each optional: a cap on the scores, s <- softcap * tanh(s / softcap); a
// distance bias, slope_a * (i - j) taken off the score of key j for the query at i,
// with slope_a = 2^(-e (a + 1) / H) for head a of H (distance_slope_exponent = e); a
// query temperature, q_i multiplied by 1 + coef * ln(floor((i + 1) / every) + 1).
//
// Also optional: an RMS norm of q and of k per head (one weight vector each for all
// heads, before any rotation); a rotation of the first rotary_dim values of each q and k
// head with the position (a `position` part of kind rope_neox: value i turns with value
// i + rotary_dim / 2, the rest of the head passes unchanged); first positions that stay
// visible beside the window, j < keep_first, at their true positions; and weights that
// are no softmax: with score_bias the weight of a visible key is
// sigmoid(s_ij + score_bias_a), a learned number per head, not normalized over the keys.
//
// And: a short causal convolution over time on every column of q, k and v, directly after
// the products (conv_taps; weights [columns, taps] beside each matrix, no bias; the last
// taps - 1 sums of a sequence are its state); a position part of kind rope_pairs turns
// neighbours (2i, 2i + 1); qk_unit_norm_eps: q and k are divided by their root mean square per
// head AFTER the rotation, without a weight; gate: the joined heads are multiplied by
// sigmoid(Wg h) before the output product (Wg's rows go into the q, k, v product).
//
// params: hidden_size, num_heads, num_kv_heads, head_dim, v_head_dim (default: head_dim),
// scale (default 1/sqrt(head_dim)), window (0: none), keep_first (0: none), qk_norm_eps
// (absent: no q/k norm), qk_unit_norm_eps (absent: none), conv_taps (0: none), gate (boolean),
// position (a part; absent: none), score_bias (boolean),
// softcap (0 or absent: none),
// distance_slope_exponent (absent: no bias), q_temp_coef and q_temp_every (absent or
// every = 0: none), bias (on q, k, v), out_bias (on o; default: as bias), head_scale, sink, own_kv
// (booleans; own_kv false: the run order gives this layer another entry's cache and it
// has no key and value products), names (optional): q, k, v, o, bias (a suffix),
// head_scale, sink, q_norm, k_norm, score_bias, gate, conv (a suffix).
class SinkAttention : public Mixer {
public:
    SinkAttention(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        g_.nh = (int)s.get_int("num_heads");
        g_.nkv = (int)s.get_int("num_kv_heads");
        g_.hd = (int)s.get_int("head_dim");
        g_.vd = (int)s.get_int("v_head_dim", g_.hd);
        g_.window = (int)s.get_int("window", 0);
        g_.scale = s.has("scale") ? (float)s.get_double("scale") : (float)(1.0 / std::sqrt((double)g_.hd));
        bias_ = flag(s, "bias", false);
        out_bias_ = flag(s, "out_bias", bias_);
        head_scale_ = flag(s, "head_scale", false);
        sink_ = flag(s, "sink", false);
        own_kv_ = flag(s, "own_kv", true);
        g_.softcap = s.has("softcap") ? (float)s.get_double("softcap") : 0.0f;
        has_slopes_ = s.has("distance_slope_exponent");
        slope_exponent_ = has_slopes_ ? s.get_double("distance_slope_exponent") : 0.0;
        q_every_ = (int)s.get_int("q_temp_every", 0);
        q_coef_ = q_every_ > 0 ? (float)s.get_double("q_temp_coef") : 0.0f;
        if (g_.softcap < 0.0f || q_every_ < 0)
            config_error("sink_attention: softcap and q_temp_every must not be negative");
        if (hidden_ <= 0 || g_.nh <= 0 || g_.nkv <= 0) config_error("sink_attention: sizes must be positive");
        if (g_.nh % g_.nkv) config_error("sink_attention: num_heads must be a multiple of num_kv_heads");
        if (g_.hd <= 0 || g_.hd > 512 || g_.vd <= 0 || g_.vd > 512)
            config_error(fmt("sink_attention: head sizes %d and %d: the kernels take 1 to 512", g_.hd, g_.vd));
        if (g_.window < 0) config_error("sink_attention: window must not be negative");
        g_.keep_first = g_.window > 0 ? (int)s.get_int("keep_first", 0) : 0;
        if (g_.keep_first < 0) config_error("sink_attention: keep_first must not be negative");
        qk_norm_ = s.has("qk_norm_eps");
        qk_eps_ = qk_norm_ ? (float)s.get_double("qk_norm_eps") : 0.0f;
        score_bias_ = flag(s, "score_bias", false);
        if (score_bias_ && (sink_ || g_.softcap > 0.0f || has_slopes_ || head_scale_))
            config_error("sink_attention: weights that are sigmoids take no sink, cap, slopes or head factors");
        if (s.has("position")) {
            position_ = build_position(s.get_part("position"), dt, d);
            if (position_->rotary_dim() > g_.hd)
                config_error(fmt("sink_attention: rotary_dim %d is above the head size %d", position_->rotary_dim(),
                                 g_.hd));
        }
        gate_ = flag(s, "gate", false);
        conv_taps_ = (int)s.get_int("conv_taps", 0);
        if (conv_taps_ < 0) config_error("sink_attention: conv_taps must not be negative");
        unit_norm_ = s.has("qk_unit_norm_eps");
        if (unit_norm_) {
            if (qk_norm_) config_error("sink_attention: a q/k norm with weights and one without are not built together");
            qk_eps_ = (float)s.get_double("qk_unit_norm_eps");
        }
        if (conv_taps_ > 0 && (bias_ || !own_kv_))
            config_error("sink_attention: the convolutions over q, k and v take no bias and need keys and values of the layer's own");
        prepared_ = qk_norm_ || unit_norm_ || conv_taps_ > 0 || (position_ && position_->rotary_dim() > 0);
        if (prepared_ && q_every_ > 0)
            config_error("sink_attention: a query temperature together with a q/k norm or a rotation is not built");
        if (prepared_ && !own_kv_)
            config_error("sink_attention: a q/k norm or a rotation needs keys and values of the layer's own");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_qn_ = leaf("q_norm", "q_norm.weight");
        n_kn_ = leaf("k_norm", "k_norm.weight");
        n_sb_ = leaf("score_bias", "score_bias");
        n_q_ = leaf("q", "q_proj.weight");
        n_k_ = leaf("k", "k_proj.weight");
        n_v_ = leaf("v", "v_proj.weight");
        n_o_ = leaf("o", "o_proj.weight");
        n_bias_ = leaf("bias", ".bias");
        n_hs_ = leaf("head_scale", "head_scale");
        n_sink_ = leaf("sink", "sink");
        n_gate_ = leaf("gate", "g_proj.weight");
        n_conv_ = leaf("conv", ".conv");
    }

    void tensors(const std::string &p, TensorList &out) const override {
        long long qw = (long long)g_.nh * g_.hd, kw = (long long)g_.nkv * g_.hd, vw = (long long)g_.nkv * g_.vd;
        long long ow = (long long)g_.nh * g_.vd;
        auto mat = [&](const std::string &leaf, long long rows, long long cols, bool with_bias) {
            out.emplace_back(name(p, leaf), TensorSpec{{rows, cols}, MATRIX, false});
            if (with_bias) out.emplace_back(name(p, leaf + n_bias_), TensorSpec{{rows}, PARAM, false, 0.0f, 0.02f});
        };
        mat(n_q_, qw, hidden_, bias_);
        if (own_kv_) {
            mat(n_k_, kw, hidden_, bias_);
            mat(n_v_, vw, hidden_, bias_);
        }
        if (head_scale_) out.emplace_back(name(p, n_hs_), TensorSpec{{g_.nh}, PARAM, false, 1.0f, 0.1f});
        if (sink_) out.emplace_back(name(p, n_sink_), TensorSpec{{g_.nh}, PARAM, false, 0.0f, 0.5f});
        if (qk_norm_) {
            out.emplace_back(name(p, n_qn_), TensorSpec{{g_.hd}, PARAM, false, 1.0f, 0.1f});
            out.emplace_back(name(p, n_kn_), TensorSpec{{g_.hd}, PARAM, false, 1.0f, 0.1f});
        }
        if (score_bias_) out.emplace_back(name(p, n_sb_), TensorSpec{{g_.nh}, PARAM, false, -2.0f, 0.5f});
        if (gate_) out.emplace_back(name(p, n_gate_), TensorSpec{{ow, hidden_}, MATRIX, false});
        if (conv_taps_ > 0) {
            out.emplace_back(name(p, n_q_ + n_conv_), TensorSpec{{qw, conv_taps_}, PARAM, false, 0.25f, 0.25f});
            out.emplace_back(name(p, n_k_ + n_conv_), TensorSpec{{kw, conv_taps_}, PARAM, false, 0.25f, 0.25f});
            out.emplace_back(name(p, n_v_ + n_conv_), TensorSpec{{vw, conv_taps_}, PARAM, false, 0.25f, 0.25f});
        }
        mat(n_o_, hidden_, ow, out_bias_);
        if (position_) position_->tensors(name(p, "position"), out);
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> in = {take(t, name(p, n_q_))};
        std::vector<DevTensor> bs;
        if (bias_) bs.push_back(take(t, name(p, n_q_ + n_bias_)));
        if (own_kv_) {
            in.push_back(take(t, name(p, n_k_)));
            if (bias_) bs.push_back(take(t, name(p, n_k_ + n_bias_)));
            in.push_back(take(t, name(p, n_v_)));
            if (bias_) bs.push_back(take(t, name(p, n_v_ + n_bias_)));
        }
        if (gate_) {
            gate_col0_ = 0;
            for (auto &m : in) gate_col0_ += m.shape[0];
            in.push_back(take(t, name(p, n_gate_)));       // the gate reads what q, k and v read
        }
        w_in_ = fuse_rows(*dev, in);
        if (conv_taps_ > 0) {
            std::vector<DevTensor> cw = {take(t, name(p, n_q_ + n_conv_)), take(t, name(p, n_k_ + n_conv_)),
                                         take(t, name(p, n_v_ + n_conv_))};
            conv_w_ = fuse_rows(*dev, cw);
        }
        if (bias_) {
            // one bias vector over the fused product's columns
            for (auto &b : bs) b.shape = {b.numel(), 1};
            b_in_ = fuse_rows(*dev, bs);
        }
        if (head_scale_) temp_ = take(t, name(p, n_hs_));
        if (sink_) sinks_ = take(t, name(p, n_sink_));
        if (qk_norm_) {
            q_norm_ = take(t, name(p, n_qn_));
            k_norm_ = take(t, name(p, n_kn_));
        }
        if (score_bias_) {
            score_b_ = take(t, name(p, n_sb_));
            g_.score_bias = (const float *)score_b_.ptr;
        }
        if (position_) position_->load(name(p, "position"), t);
        w_o_ = take(t, name(p, n_o_));
        if (out_bias_) b_o_ = take(t, name(p, n_o_ + n_bias_));
        if (has_slopes_) {
            std::vector<float> sl((size_t)g_.nh);
            for (int a = 0; a < g_.nh; a++)
                sl[(size_t)a] = (float)std::pow(2.0, -slope_exponent_ * (double)(a + 1) / (double)g_.nh);
            slopes_ = dev->tensor(F32, {g_.nh});
            cuda_check(cudaMemcpy(slopes_.ptr, sl.data(), sl.size() * 4, cudaMemcpyHostToDevice),
                       "copying the heads' slopes");
            g_.slopes = (const float *)slopes_.ptr;
        }
        g_.head_scale = head_scale_ ? (const float *)temp_.ptr : nullptr;
        g_.sink = sink_ ? (const float *)sinks_.ptr : nullptr;
        if (head_scale_) {
            // one kernel takes the largest raw score before the factor: it needs factors > 0
            std::vector<float> host((size_t)g_.nh);
            cuda_check(cudaMemcpy(host.data(), temp_.ptr, host.size() * 4, cudaMemcpyDeviceToHost),
                       "reading the heads' factors");
            g_.head_scale_positive = true;
            for (float v : host) g_.head_scale_positive = g_.head_scale_positive && v > 0.0f;
        }
    }

    size_t weight_bytes() const override {
        return w_in_.bytes() + w_o_.bytes() + b_in_.bytes() + b_o_.bytes() + temp_.bytes() + sinks_.bytes() +
               q_norm_.bytes() + k_norm_.bytes() + score_b_.bytes() + conv_w_.bytes();
    }

    // the convolutions' last taps - 1 inputs: the products' sums of q, k and v
    long long conv_width() const { return (long long)g_.nh * g_.hd + (long long)g_.nkv * (g_.hd + g_.vd); }
    StateSpec state_spec() const override {
        return conv_taps_ > 1 ? StateSpec{{conv_taps_ - 1, conv_width()}, F32} : StateSpec();
    }
    bool strided_state() const override { return true; }

    KVSpec kv_spec() const override {
        return own_kv_ ? KVSpec{g_.nkv, g_.hd, g_.window, g_.vd, false, g_.keep_first} : KVSpec();
    }

    bool take_side_rows(DevTensor &m) override {
        if (!w_in_ || shared_ || m.shape.size() != 2 || m.shape[1] != hidden_ || side_cols_ > 0) return false;
        side_col0_ = w_in_.shape[0];
        side_cols_ = m.shape[0];
        std::vector<DevTensor> both = {w_in_, m};
        w_in_ = DevTensor();
        m = DevTensor();
        w_in_ = fuse_rows(*dev, both);
        return true;
    }

    void prepare(long long n_positions) override {
        chunk_ = ops::attention_chunk();
        if (position_) position_->prepare(n_positions);
    }
    bool supports(StepKind) const override { return true; }
    bool graph_safe() const override { return true; }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        if (!chunk_) chunk_ = ops::attention_chunk();
        if (position_ && ctx.max_pos >= position_->n_positions())
            fail(JB_LLM_EINVAL, fmt("position %lld is beyond the %lld positions the encoding was prepared "
                                    "for", ctx.max_pos, position_->n_positions()));
        if (!cache.kv.k || cache.kv_heads != g_.nkv || cache.head_dim != g_.hd || cache.v_head_dim != g_.vd)
            fail(JB_LLM_EINVAL, "sink_attention: the cache this layer was given does not hold keys and values "
                                "of its head count and sizes");
        if (own_kv_ != cache.kv.writes)
            fail(JB_LLM_EINVAL, own_kv_ ? "sink_attention: a layer with keys and values of its own was given "
                                          "another layer's cache"
                                        : "sink_attention: a layer without key and value products needs "
                                          "another layer's cache (cache_of in the run order)");
        long long n = ctx.n_rows;
        const float *b_in = bias_ ? (const float *)b_in_.ptr : nullptr;
        // a pair's shared first product holds this mixer's columns first; it is borrowed, not owned
        Stack own;
        if (!shared_) own = ops::linear(d, h, ctx.dtype, n, hidden_, w_in_);
        else if (!ctx.shared) fail(JB_LLM_EFAIL, "sink_attention: the shared first product is missing");
        Stack &qkv = shared_ ? const_cast<Stack &>(*ctx.shared) : own;
        int max_chunks = (int)(ctx.max_pos / chunk_ + 1);
        if (g_.window) max_chunks = std::min(max_chunks, (g_.window - 1) / chunk_ + 2);
        // the kept first positions' chunks come in front of the window's
        max_chunks += ops::attention_kept_chunks(g_.window, g_.keep_first);
        bool decode = ctx.kind == DECODE;
        if (prepared_) {
            // (the convolutions over time,) bias, per-head norms and the rotation in one pass over
            // the product's sums, K and V into the cache; then attention over the cache
            Stack conv;
            if (conv_taps_ > 0) conv = convolve(ctx, qkv, cache);
            int rot = position_ ? position_->rotary_dim() : 0;
            Buf q = ops::qkv_prepare_append(d, conv ? conv : qkv, b_in, qk_norm_ ? (const float *)q_norm_.ptr : nullptr,
                                            qk_norm_ ? (const float *)k_norm_.ptr : nullptr, qk_eps_,
                                            rot ? position_->cos() : nullptr, rot ? position_->sin() : nullptr,
                                            rot / 2, ctx.row_pos, ctx.row_seq, cache.kv, g_, ctx.dtype,
                                            rot && position_->pairs(), unit_norm_);
            conv = Stack();
            const int32_t *blocks = prefill_blocks(ctx, decode);
            Buf a = ops::attention(d, q.ptr, n, cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks, blocks,
                                   n_blocks_, decode);
            return finish(ctx, qkv, a);
        }
        if (decode && ctx.dtype == BF16 && q_every_ == 0 && !g_.keep_first && !score_bias_) {
            // one new token per sequence: the attention kernel makes q and the new key and
            // value from the product's sums and its bias itself, where it takes the sizes
            Buf a = ops::attention_decode_qkv(d, qkv, nullptr, nullptr, 0.0f, nullptr, nullptr, cache.kv, g_,
                                              ctx.row_pos, ctx.row_seq, max_chunks, b_in);
            if (a) return finish(ctx, qkv, a);
        }
        Buf q = ops::qkv_bias_append(d, qkv, b_in, ctx.row_pos, ctx.row_seq, cache.kv, g_, ctx.dtype, own_kv_,
                                     q_coef_, q_every_);
        const int32_t *blocks = prefill_blocks(ctx, decode);
        Buf a = ops::attention(d, q.ptr, n, cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks, blocks, n_blocks_,
                               decode);
        return finish(ctx, qkv, a);
    }

    // q, k and v through their convolutions over time, as one sum [n, q + k + v] in float32;
    // the state holds each sequence's last taps - 1 sums.
    Stack convolve(StepContext &ctx, const Stack &qkv, LayerCache &cache) {
        long long C = conv_width();
        long long stride = cache.state_stride > 0 ? cache.state_stride : (long long)(conv_taps_ - 1) * C;
        if (conv_taps_ > 1 && (!cache.state || cache.state_spec.bytes() < state_spec().bytes()))
            fail(JB_LLM_EINVAL, "sink_attention: the cache holds no state for the layer's convolutions");
        float *st = (float *)cache.state;
        Stack out;
        out.S = 1;
        out.n = ctx.n_rows;
        out.m = C;
        const float *w = (const float *)conv_w_.ptr;
        // rows that read sums of earlier steps which other rows of this step replace: two launches
        bool two = ctx.kind == EXTEND && conv_taps_ > 1;
        out.buf = ops::causal_conv(*ctx.dev, qkv, 0, C, w, nullptr, conv_taps_, st, stride, ctx.row_pos, ctx.row_seq,
                                   ctx.seq_slot, false, F32, true, !two);
        if (two)
            ops::causal_conv(*ctx.dev, qkv, 0, C, w, nullptr, conv_taps_, st, stride, ctx.row_pos, ctx.row_seq,
                             ctx.seq_slot, false, F32, false, true);
        return out;
    }

    // the heads' outputs times the gate's sigmoid (where there is one), then the output product
    Stack finish(StepContext &ctx, Stack &qkv, Buf &a) {
        if (gate_)
            a = ops::gate_rows(*ctx.dev, a.ptr, ctx.dtype, ctx.n_rows, (long long)g_.nh * g_.vd, qkv, gate_col0_);
        keep_side(ctx, qkv);
        return output(ctx, a);
    }

    // Runs of consecutive positions for the tensor-core prefill kernel, where it takes this
    // mixer (null otherwise); the same for every layer of the step with this grouping of
    // heads.  n_blocks_ gets their number.
    const int32_t *prefill_blocks(StepContext &ctx, bool decode) {
        n_blocks_ = 0;
        if (decode || ctx.dtype != BF16 || !ops::attention_tc_ok(g_.nh, g_.nkv, g_.hd) || g_.vd != g_.hd ||
            (head_scale_ && !g_.head_scale_positive) || ctx.seq_len.empty())
            return nullptr;
        int per = ops::attention_block_positions(g_.nh, g_.nkv);
        std::string key = "attention_blocks/" + std::to_string(per);
        auto it = ctx.extras.find(key);
        if (it == ctx.extras.end()) {
            StepContext::Extra e;
            e.buf = ops::attention_blocks(*ctx.dev, ctx.seq_row0.data(), ctx.seq_pos0.data(), ctx.seq_len.data(),
                                          ctx.n_seqs, per, &e.n);
            it = ctx.extras.emplace(key, std::move(e)).first;
        }
        n_blocks_ = it->second.n;
        return it->second.buf.as<int32_t>();
    }

    // the product goes to whoever gave the side rows, or back to the pool
    void keep_side(StepContext &ctx, Stack &qkv) {
        if (shared_) return;            // the product is the pair's
        if (side_cols_ > 0) {
            ctx.side = std::move(qkv);
            ctx.side_col0 = side_col0_;
        }
        qkv = Stack();
    }

    DevTensor *first_matrix() override { return w_in_ && !bias_ && side_cols_ == 0 ? &w_in_ : nullptr; }
    void share_first_product(long long col0) override {
        if (col0 != 0) fail(JB_LLM_EINVAL, "sink_attention: its columns must come first in a shared product");
        shared_ = true;
    }

    Stack output(StepContext &ctx, const Buf &a) {
        Stack out = ops::linear(*ctx.dev, a.ptr, ctx.dtype, ctx.n_rows, (long long)g_.nh * g_.vd, w_o_);
        out.bias = out_bias_ ? (const float *)b_o_.ptr : nullptr;
        return out;
    }

    Json info() const override {
        Json o = Json::object();
        o.set("own_kv", own_kv_);
        o.set("v_head_dim", g_.vd);
        return o;
    }

private:
    static bool flag(const PartSpec &s, const char *key, bool dflt) {
        return s.has(key) ? s.params.get(key).as_bool() : dflt;
    }
    long long hidden_;
    ops::AttnGeometry g_;
    bool bias_, out_bias_, head_scale_, sink_, own_kv_;
    bool qk_norm_ = false, score_bias_ = false;
    bool prepared_ = false;      // q and k are normed or rotated: qkv_prepare_append makes them
    bool gate_ = false, unit_norm_ = false;
    bool shared_ = false;        // the first product's rows went into a pair's shared first product
    int conv_taps_ = 0;
    long long gate_col0_ = 0;
    std::string n_gate_, n_conv_;
    DevTensor conv_w_;
    float qk_eps_ = 0.0f;
    std::unique_ptr<PositionEncoding> position_;
    DevTensor q_norm_, k_norm_, score_b_;
    std::string n_qn_, n_kn_, n_sb_;
    int n_blocks_ = 0;
    bool has_slopes_ = false;
    double slope_exponent_ = 0.0;
    float q_coef_ = 0.0f;
    int q_every_ = 0;
    std::string n_q_, n_k_, n_v_, n_o_, n_bias_, n_hs_, n_sink_;
    DevTensor w_in_, b_in_, w_o_, b_o_, temp_, sinks_, slopes_;
    long long side_col0_ = 0, side_cols_ = 0;
    int chunk_ = 0;
};

// Latent attention: keys and values of all heads come from one latent vector per
// position, and one rotated key part is shared by all heads.  With H heads, per head
// D plain and R rotated query/key values and Dv values, a latent of C values and a
// query latent of Cq:
//
//   cq = rms(Wdq h) wq;  q = Wuq cq, per head [D plain | R rotated]
//   z = Wdkv h;  c = rms(z[0:C]) wc;  kr = z[C:C+R]
//   the first rotary_dim values of q's rotated part and of kr turn pair by pair
//   (2i, 2i+1) with the position
//   s_ij = (q_plain_i . (Wuk c_j)_head + q_rot_i . kr_j) * scale,  j <= i;  softmax
//   out = Wo (concat_heads(sum_j p_ij (Wuv c_j)_head) * sigmoid(Wg h))     (the gate optional)
//
// The cache holds [c | kr] per position, once for all heads, and the values are read
// from the same rows (KVSpec::values_in_keys).  Keys and values per head are never
// formed: a head's query goes through its key matrix first (q_lat = Wuk_head^T q_plain),
// scores and weighted sums run over the latents, and the head's value matrix is
// applied to the weighted sum; the two per-head products are one product per head
// over rows gathered head by head (ops::linear_heads).
//
// A step of whole prompts in bfloat16 whose per-head sizes the tensor-core attention
// kernel takes (D + R = Dv = 64 or 128) forms keys and values per head after all,
// for that step alone, in pages of its own: [Wuk_head c | kr] and Wuv_head c are one
// product of the rows [c | kr] with a matrix made at load time (the heads' key and
// value matrices with an identity for the shared part).  The cache gets the latents
// as always, and decoding goes on from them.
//
// params: hidden_size, num_heads, head_dim (D), rot_dim (R), v_head_dim (Dv), kv_rank
// (C), q_rank (Cq), scale, eps, gate (default true), per_head_prompts (default true:
// false keeps prompts on the latents too), position (a part, kind rope_pairs), names
// (optional): dq, dq_norm, uq, dkv, dkv_norm, uk, uv, gate, o
class LatentAttention : public Mixer {
public:
    LatentAttention(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        H_ = (int)s.get_int("num_heads");
        D_ = s.get_int("head_dim");
        R_ = s.get_int("rot_dim");
        Dv_ = s.get_int("v_head_dim");
        C_ = s.get_int("kv_rank");
        Cq_ = s.get_int("q_rank");
        scale_ = (float)s.get_double("scale");
        eps_ = (float)s.get_double("eps");
        gate_ = s.has("gate") ? s.params.get("gate").as_bool() : true;
        per_head_prompts_ = s.has("per_head_prompts") ? s.params.get("per_head_prompts").as_bool() : true;
        if (hidden_ <= 0 || H_ <= 0 || D_ <= 0 || R_ < 0 || Dv_ <= 0 || C_ <= 0 || Cq_ <= 0)
            config_error("latent_attention: sizes must be positive");
        if (C_ + R_ > 512)
            config_error(fmt("latent_attention: kv_rank + rot_dim = %lld: the attention kernels take rows of "
                             "up to 512 values", C_ + R_));
        position_ = build_position(s.get_part("position"), dt, d);
        if (position_->rotary_dim() > R_ || position_->rotary_dim() % 2)
            config_error(fmt("latent_attention: %d rotated dimensions do not fit the rotated part of %lld",
                             position_->rotary_dim(), R_));
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_dq_ = leaf("dq", "q_down.weight");
        n_dqn_ = leaf("dq_norm", "q_down_norm.weight");
        n_uq_ = leaf("uq", "q_up.weight");
        n_dkv_ = leaf("dkv", "kv_down.weight");
        n_dkvn_ = leaf("dkv_norm", "kv_down_norm.weight");
        n_uk_ = leaf("uk", "k_up.weight");
        n_uv_ = leaf("uv", "v_up.weight");
        n_g_ = leaf("gate", "gate.weight");
        n_o_ = leaf("o", "o_proj.weight");
        g_.nh = H_;
        g_.nkv = 1;
        g_.hd = (int)(C_ + R_);
        g_.vd = (int)C_;
        g_.scale = scale_;
    }

    void tensors(const std::string &p, TensorList &out) const override {
        out.emplace_back(name(p, n_dq_), TensorSpec{{Cq_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_dqn_), TensorSpec{{Cq_}, PARAM, false, 1.0f, 0.1f});
        out.emplace_back(name(p, n_uq_), TensorSpec{{H_ * (D_ + R_), Cq_}, MATRIX, false});
        out.emplace_back(name(p, n_dkv_), TensorSpec{{C_ + R_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_dkvn_), TensorSpec{{C_}, PARAM, false, 1.0f, 0.1f});
        out.emplace_back(name(p, n_uk_), TensorSpec{{H_ * D_, C_}, MATRIX, false});
        out.emplace_back(name(p, n_uv_), TensorSpec{{H_ * Dv_, C_}, MATRIX, false});
        if (gate_) out.emplace_back(name(p, n_g_), TensorSpec{{H_ * Dv_, hidden_}, MATRIX, false});
        out.emplace_back(name(p, n_o_), TensorSpec{{hidden_, H_ * Dv_}, MATRIX, false});
        position_->tensors(name(p, "position"), out);
    }

    void load(const std::string &p, TensorMap &t) override {
        // the three matrices that read the mixer's input: one product
        std::vector<DevTensor> in = {take(t, name(p, n_dq_)), take(t, name(p, n_dkv_))};
        if (gate_) in.push_back(take(t, name(p, n_g_)));
        w_in_ = fuse_rows(*dev, in);
        wq_norm_ = take(t, name(p, n_dqn_));
        wc_norm_ = take(t, name(p, n_dkvn_));
        w_uq_ = take(t, name(p, n_uq_));
        {
            // a head's query goes through its key matrix: [D, C] per head, kept as [C, D]
            DevTensor uk = take(t, name(p, n_uk_));
            w_ukT_ = ops::transpose_heads(*dev, uk, H_);
        }
        w_uv_ = take(t, name(p, n_uv_));
        w_o_ = take(t, name(p, n_o_));
        position_->load(name(p, "position"), t);
        if (per_head_prompts_ && dtype == BF16 && D_ + R_ == Dv_ && ops::attention_tc_ok(H_, H_, (int)Dv_) &&
            w_uv_.dt == BF16 && w_ukT_.dt == BF16)
            make_expander(take_back_uk());
    }

    // [H D, C] once more out of its transposed form (load() has given the original back)
    DevTensor take_back_uk() {
        DevTensor t = w_ukT_;
        t.shape = {H_ * C_, D_};
        return ops::transpose_heads(*dev, t, H_);     // [H, C, D] -> [H, D, C]
    }

    // Rows [c | kr] times this matrix are, head by head, [Wuk_head c | kr], and after
    // all heads' keys the values Wuv c: [H (D + R) + H Dv, C + R].
    void make_expander(const DevTensor &uk) {
        size_t es = dtype_size(uk.dt);
        long long W = C_ + R_, hd = D_ + R_;
        w_expand_ = dev->tensor(uk.dt, {H_ * hd + H_ * Dv_, W}, true);
        std::vector<uint16_t> eye((size_t)(R_ * R_), 0);
        for (long long i = 0; i < R_; i++) eye[(size_t)(i * R_ + i)] = 0x3f80;      // 1.0 in bfloat16
        char *dst = (char *)w_expand_.ptr;
        for (int h = 0; h < H_; h++) {
            cuda_check(cudaMemcpy2D(dst + (size_t)(h * hd) * W * es, W * es, (const char *)uk.ptr + (size_t)h * D_ * C_ * es,
                                    C_ * es, C_ * es, D_, cudaMemcpyDeviceToDevice), "placing a head's key matrix");
            if (R_ > 0)
                cuda_check(cudaMemcpy2D(dst + ((size_t)(h * hd + D_) * W + C_) * es, W * es, eye.data(), R_ * es,
                                        R_ * es, R_, cudaMemcpyHostToDevice), "placing the shared part's identity");
        }
        cuda_check(cudaMemcpy2D(dst + (size_t)(H_ * hd) * W * es, W * es, w_uv_.ptr, C_ * es, C_ * es, H_ * Dv_,
                                cudaMemcpyDeviceToDevice), "placing the value matrices");
        dev->sync();
    }

    size_t weight_bytes() const override {
        // (the matrix a prompt step uses instead of uk and uv is not read by a decode step)
        return w_in_.bytes() + w_uq_.bytes() + w_ukT_.bytes() + w_uv_.bytes() + w_o_.bytes() +
               wq_norm_.bytes() + wc_norm_.bytes();
    }

    KVSpec kv_spec() const override { return KVSpec{1, (int)(C_ + R_), 0, (int)C_, true}; }

    void prepare(long long n_positions) override {
        position_->prepare(n_positions);
        chunk_ = ops::attention_chunk();
    }
    bool supports(StepKind) const override { return true; }
    bool graph_safe() const override { return true; }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        Device &d = *ctx.dev;
        int rot_half = position_->rotary_dim() / 2;
        if (rot_half > 0 && ctx.max_pos >= position_->n_positions())
            fail(JB_LLM_EINVAL, fmt("position %lld is beyond the %lld positions the encoding was prepared "
                                    "for", ctx.max_pos, position_->n_positions()));
        if (!cache.kv.k || !cache.kv.writes || cache.kv_heads != 1 || cache.head_dim != g_.hd ||
            cache.v_head_dim != g_.vd || cache.kv.v_ld != g_.hd)
            fail(JB_LLM_EINVAL, "latent_attention: the cache this layer was given does not hold its latents");
        if (!chunk_) chunk_ = ops::attention_chunk();
        long long n = ctx.n_rows;
        size_t esz = dtype_size(ctx.dtype);
        Stack P = ops::linear(d, h, ctx.dtype, n, hidden_, w_in_);
        if (w_expand_ && ctx.kind == PREFILL && ctx.dtype == BF16 && !ctx.captured && !ctx.seq_len.empty())
            return forward_per_head(ctx, P, cache, rot_half);
        Buf cq = ops::latent_down(d, P, 0, Cq_, (const float *)wq_norm_.ptr, Cq_, C_,
                                  (const float *)wc_norm_.ptr, R_, position_->cos(), position_->sin(), rot_half,
                                  ctx.row_pos, ctx.row_seq, cache.kv, eps_, ctx.dtype);
        Buf q_lat = d.pool.get((size_t)n * (size_t)H_ * (size_t)(C_ + R_) * esz);
        {
            Stack Q = ops::linear(d, cq.ptr, ctx.dtype, n, Cq_, w_uq_);
            Buf q_plain = ops::latent_q_split(d, Q, H_, D_, R_, C_, position_->cos(), position_->sin(), rot_half,
                                              ctx.row_pos, q_lat.ptr, ctx.dtype);
            ops::HeadStack A = ops::linear_heads(d, q_plain.ptr, ctx.dtype, H_, n, D_, w_ukT_);
            ops::latent_q_join(d, A, R_, q_lat.ptr, ctx.dtype);
        }
        int max_chunks = (int)(ctx.max_pos / chunk_ + 1);
        // the weighted sums of the latents, one head's rows together
        Buf o = ops::attention(d, q_lat.ptr, n, cache.kv, g_, ctx.row_pos, ctx.row_seq, max_chunks, nullptr, 0,
                               ctx.kind == DECODE, false, true);
        q_lat.reset();
        ops::HeadStack V = ops::linear_heads(d, o.ptr, ctx.dtype, H_, n, C_, w_uv_);
        Stack none;
        Buf a = ops::heads_gate(d, V, gate_ ? P : none, Cq_ + C_ + R_, ctx.dtype);
        return ops::linear(d, a.ptr, ctx.dtype, n, (long long)H_ * Dv_, w_o_);
    }

    // Whole prompts on the tensor cores: keys and values per head, for this step alone.
    Stack forward_per_head(StepContext &ctx, Stack &P, LayerCache &cache, int rot_half) {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        int hd = (int)(D_ + R_);
        Buf rows;
        Buf cq = ops::latent_down(d, P, 0, Cq_, (const float *)wq_norm_.ptr, Cq_, C_,
                                  (const float *)wc_norm_.ptr, R_, position_->cos(), position_->sin(), rot_half,
                                  ctx.row_pos, ctx.row_seq, cache.kv, eps_, ctx.dtype, &rows);
        // whole queries [n, H, D + R], the rotated part turned
        Buf q = d.pool.get((size_t)n * (size_t)H_ * (size_t)hd * 2);
        {
            Stack Q = ops::linear(d, cq.ptr, ctx.dtype, n, Cq_, w_uq_);
            ops::latent_q_split(d, Q, H_, D_, R_, D_, position_->cos(), position_->sin(), rot_half, ctx.row_pos,
                                q.ptr, ctx.dtype, false);
        }
        // pages of this step's own: every sequence starts at position 0 and gets the pages
        // it needs one after the other
        std::vector<int32_t> table;
        long long n_pages = 0, most = 0;
        for (int i = 0; i < ctx.n_seqs; i++) most = std::max(most, pages_for(ctx.seq_len[(size_t)i]));
        int stride = (int)((most + 7) / 8 * 8);
        table.assign((size_t)ctx.n_seqs * (size_t)stride, -1);
        for (int i = 0; i < ctx.n_seqs; i++)
            for (long long p = 0; p < pages_for(ctx.seq_len[(size_t)i]); p++)
                table[(size_t)i * (size_t)stride + (size_t)p] = (int32_t)n_pages++;
        Buf bt = d.pool.get(std::max<size_t>(table.size() * 4, 16));
        d.upload(bt.ptr, table.data(), table.size() * 4);
        size_t page_vals = (size_t)H_ * PAGE * (size_t)hd;
        Buf kp = d.pool.get((size_t)n_pages * page_vals * 2), vp = d.pool.get((size_t)n_pages * page_vals * 2);
        // slots past a sequence's end are never seen but are multiplied by weights of 0
        cuda_check(cudaMemsetAsync(kp.ptr, 0, kp.bytes, d.stream), "clearing a step's key pages");
        cuda_check(cudaMemsetAsync(vp.ptr, 0, vp.bytes, d.stream), "clearing a step's value pages");
        ops::AttnCache own;
        own.k = kp.ptr;
        own.v = vp.ptr;
        own.n_pages = n_pages;
        own.dt = BF16;
        own.block_table = bt.as<int32_t>();
        own.bt_stride = stride;
        {
            Stack kv = ops::linear(d, rows.ptr, ctx.dtype, n, C_ + R_, w_expand_);
            ops::kv_append(d, kv, ctx.row_pos, ctx.row_seq, own, H_, hd, hd);
        }
        ops::AttnGeometry g;
        g.nh = g.nkv = H_;
        g.hd = g.vd = hd;
        g.scale = scale_;
        int per = ops::attention_block_positions(g.nh, g.nkv);
        std::string key = "attention_blocks/" + std::to_string(per);
        auto it = ctx.extras.find(key);
        if (it == ctx.extras.end()) {
            StepContext::Extra e;
            e.buf = ops::attention_blocks(d, ctx.seq_row0.data(), ctx.seq_pos0.data(), ctx.seq_len.data(), ctx.n_seqs,
                                          per, &e.n);
            it = ctx.extras.emplace(key, std::move(e)).first;
        }
        int max_chunks = (int)(ctx.max_pos / chunk_ + 1);
        Buf o = ops::attention(d, q.ptr, n, own, g, ctx.row_pos, ctx.row_seq, max_chunks,
                               it->second.buf.as<int32_t>(), it->second.n, false);
        Buf a = gate_ ? ops::gate_rows(d, o.ptr, ctx.dtype, n, (long long)H_ * Dv_, P, Cq_ + C_ + R_) : std::move(o);
        return ops::linear(d, a.ptr, ctx.dtype, n, (long long)H_ * Dv_, w_o_);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("position", position_->info());
        o.set("position_kind", position_->spec.kind);
        o.set("gate", gate_);
        o.set("per_head_prompts", (bool)w_expand_);
        return o;
    }

private:
    long long hidden_, D_, R_, Dv_, C_, Cq_;
    int H_;
    float scale_, eps_;
    bool gate_;
    ops::AttnGeometry g_;
    std::unique_ptr<PositionEncoding> position_;
    std::string n_dq_, n_dqn_, n_uq_, n_dkv_, n_dkvn_, n_uk_, n_uv_, n_g_, n_o_;
    DevTensor w_in_, wq_norm_, wc_norm_, w_uq_, w_ukT_, w_uv_, w_o_, w_expand_;
    bool per_head_prompts_ = true;
    int chunk_ = 0;
};

}  // namespace

void register_builtin_mixers() {
    register_part("mixer", "latent_attention", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new LatentAttention(s, dt, d));
    });
    register_part("mixer", "sink_attention", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new SinkAttention(s, dt, d));
    });
    register_part("mixer", "gqa_attention", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new GQAAttention(s, dt, d));
    });
}

}  // namespace jb
