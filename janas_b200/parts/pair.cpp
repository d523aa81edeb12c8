// Two mixers side by side that read the same input, their results joined into one.
//
//   "sum":         out = left_scale * left(h) + right_scale * right(h)
//   "normed_mean": out = (rms(left(h)) wl + rms(right(h)) wr) / 2, each result normed over the
//                  model's width (eps inside the root) with a weight of its own
//
// Each side is any registered mixer.  At most one side may keep keys and values (the pair's
// cache group is that side's); the sides' fixed-size states lie one after the other in the
// pair's state row per slot, and each side is told the row's length (LayerCache::state_stride).
//
// Where both sides offer the matrix of their first product (Mixer::first_matrix), the two are
// one matrix and one product serves both sides (share_first_product false: each runs its own).
//
// params: hidden_size, left, right (parts), join ("sum" or "normed_mean"), left_scale and
// right_scale (for "sum"; default 1), eps (for "normed_mean"), share_first_product (default
// true), names (optional): left, right (the sides' prefixes below the mixer's), left_out,
// right_out (the weights of "normed_mean")
#include "part.h"

namespace jb {

namespace {

class PairMixer : public Mixer {
public:
    PairMixer(const PartSpec &s, DType dt, Device *d) : Mixer(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        if (hidden_ <= 0) config_error("pair: hidden_size must be positive");
        left_ = build_mixer(s.get_part("left"), dt, d);
        right_ = build_mixer(s.get_part("right"), dt, d);
        std::string join = s.params.get("join").is_string() ? s.params.get("join").as_string() : "sum";
        if (join != "sum" && join != "normed_mean") config_error("pair: join '" + join + "' is not sum or normed_mean");
        normed_ = join == "normed_mean";
        if (normed_) {
            eps_ = (float)s.get_double("eps");
            sl_ = sr_ = 0.5f;
        } else {
            sl_ = s.has("left_scale") ? (float)s.get_double("left_scale") : 1.0f;
            sr_ = s.has("right_scale") ? (float)s.get_double("right_scale") : 1.0f;
        }
        if (!left_->kv_spec().none() && !right_->kv_spec().none())
            config_error("pair: only one side may keep keys and values");
        for (Mixer *m : {left_.get(), right_.get()})
            if (!m->state_spec().none() && (!m->strided_state() || m->state_spec().dtype != F32))
                config_error("pair: a side's state must be float32 and its mixer must take the row's length");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_left_ = leaf("left", "left");
        n_right_ = leaf("right", "right");
        n_left_out_ = leaf("left_out", "left.out");
        n_right_out_ = leaf("right_out", "right.out");
        share_ = !s.has("share_first_product") || s.params.get("share_first_product").as_bool();
    }

    void tensors(const std::string &p, TensorList &out) const override {
        left_->tensors(name(p, n_left_), out);
        right_->tensors(name(p, n_right_), out);
        if (normed_) {
            out.emplace_back(name(p, n_left_out_), TensorSpec{{hidden_}, PARAM, false, 1.0f, 0.1f});
            out.emplace_back(name(p, n_right_out_), TensorSpec{{hidden_}, PARAM, false, 1.0f, 0.1f});
        }
    }

    void load(const std::string &p, TensorMap &t) override {
        left_->load(name(p, n_left_), t);
        right_->load(name(p, n_right_), t);
        if (normed_) {
            wl_ = take(t, name(p, n_left_out_));
            wr_ = take(t, name(p, n_right_out_));
        }
        // Both sides' first products read the same input: one product for both, the left side's
        // columns first, the right side's from a multiple of eight on (rows of zeros between).
        DevTensor *a = share_ ? left_->first_matrix() : nullptr, *b = share_ ? right_->first_matrix() : nullptr;
        if (a && b && a->shape.size() == 2 && b->shape.size() == 2 && a->shape[1] == hidden_ && b->shape[1] == hidden_) {
            long long rows = a->shape[0], col0 = (rows + 7) / 8 * 8;
            std::vector<DevTensor> both = {*a};
            if (col0 > rows) both.push_back(dev->tensor(a->dt, {col0 - rows, hidden_}, true));
            both.push_back(*b);
            long long total = col0 + b->shape[0];
            if (total % 8) both.push_back(dev->tensor(a->dt, {8 - total % 8, hidden_}, true));    // rows of sums four to a load
            *a = DevTensor();
            *b = DevTensor();
            w_first_ = fuse_rows(*dev, both);
            left_->share_first_product(0);
            right_->share_first_product(col0);
        }
    }

    size_t weight_bytes() const override {
        return left_->weight_bytes() + right_->weight_bytes() + wl_.bytes() + wr_.bytes() + w_first_.bytes();
    }

    KVSpec kv_spec() const override { return left_->kv_spec().none() ? right_->kv_spec() : left_->kv_spec(); }

    static long long floats(const StateSpec &sp) { return sp.none() ? 0 : (long long)(sp.bytes() / 4); }
    StateSpec state_spec() const override {
        long long total = floats(left_->state_spec()) + floats(right_->state_spec());
        return total ? StateSpec{{total}, F32} : StateSpec();
    }
    bool strided_state() const override { return true; }

    void prepare(long long n_positions) override {
        left_->prepare(n_positions);
        right_->prepare(n_positions);
    }
    bool supports(StepKind k) const override { return left_->supports(k) && right_->supports(k); }
    bool graph_safe() const override { return left_->graph_safe() && right_->graph_safe(); }

    Stack forward(StepContext &ctx, const void *h, LayerCache &cache) override {
        long long total = floats(state_spec());
        if (total && (!cache.state || (long long)(cache.state_spec.bytes() / 4) < total))
            fail(JB_LLM_EINVAL, "pair: the cache holds no state of the two sides' size for the layer");
        long long stride = cache.state_stride > 0 ? cache.state_stride : total;
        long long at = 0;
        Stack first;
        if (w_first_) {
            first = ops::linear(*ctx.dev, h, ctx.dtype, ctx.n_rows, hidden_, w_first_);
            ctx.shared = &first;
        }
        Stack result[2];
        Mixer *side[2] = {left_.get(), right_.get()};
        for (int i = 0; i < 2; i++) {
            LayerCache lc = cache;
            StateSpec sp = side[i]->state_spec();
            if (sp.none()) {
                lc.state = nullptr;
                lc.state_spec = StateSpec();
            } else {
                lc.state = (float *)cache.state + at;
                lc.state_spec = sp;
                lc.state_stride = stride;
                at += floats(sp);
            }
            if (side[i]->kv_spec().none()) lc.kv = ops::AttnCache();
            result[i] = side[i]->forward(ctx, h, lc);
            ops::resolve_bias(*ctx.dev, result[i]);
        }
        ctx.shared = nullptr;
        first = Stack();
        return ops::pair_combine(*ctx.dev, result[0], result[1], normed_ ? (const float *)wl_.ptr : nullptr,
                                 normed_ ? (const float *)wr_.ptr : nullptr, sl_, sr_, eps_,
                                 ctx.kind == DECODE && ctx.dtype == BF16);
    }

    Json info() const override {
        Json o = Json::object();
        o.set("left", left_->info());
        o.set("right", right_->info());
        return o;
    }

private:
    long long hidden_;
    std::unique_ptr<Mixer> left_, right_;
    bool normed_ = false;
    float sl_ = 1.0f, sr_ = 1.0f, eps_ = 0.0f;
    std::string n_left_, n_right_, n_left_out_, n_right_out_;
    DevTensor wl_, wr_;
    bool share_ = true;
    DevTensor w_first_;          // both sides' first matrices as one, where both offer theirs
};

}  // namespace

void register_pair_mixers() {
    register_part("mixer", "pair", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new PairMixer(s, dt, d));
    });
}

}  // namespace jb
