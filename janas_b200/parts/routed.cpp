// A routed feed-forward (mixture of experts): small feed-forwards of which every token
// uses a few, chosen by a router, with optional identity experts and a shared expert.
//
//   s = softmax(R h) over all E + I router outputs (E experts with matrices, then I
//       identity experts whose output is h itself), in float32
//   choice = s + correction;  the router outputs form `groups` equal groups of neighbours,
//       a group's score is its largest choice score, only the `group_keep` best groups'
//       outputs can be chosen, and the `top` largest choice scores among them are
//   weight_e = s_e * scale for a chosen e (not renormalized)
//   out = sum_{chosen e < E} weight_e Wd_e act(Wu_e h) + (sum_{chosen e >= E} weight_e) h
//         + Wd_shared act(Wu_shared h)
//
// All experts' up matrices, the shared expert's and the router's rows are ONE matrix, so
// one product over h gives every hidden value and the router's logits; the activation
// kernel multiplies expert e's values by the token's weight for e (0 where e was not
// chosen: those values are not even read), and one down product over [experts | shared]
// is the weighted sum.  Nothing is gathered, sorted or counted on the host: a step's
// launches do not depend on what the router chooses, so a decode step can be captured.
// The price is the products of the experts a token did not choose.
//
// The identity experts' term is not added here: it rides on the result as
// Stack::skip (h with one coefficient per row) and is taken by the kernel that ends the
// sublayer, or by ops::resolve_bias for any other consumer.
#include "part.h"

namespace jb {

namespace {

// params: hidden_size, experts, expert_ff, identity (default 0), top, groups (default 1),
// group_keep (default groups), scale (default 1), correction (default false: a vector
// added to the scores for the choice alone), shared_ff (default 0: no shared expert),
// activation ("relu2", "relu", "gelu_tanh", "silu"), gated (default false: an expert is
// Wd (act(Wg h) * (Wu h)) with a gate matrix of its own), score ("softmax", the default, or
// "sigmoid": each score the sigmoid of its own logit), group_best (default 1: a group's score
// is the sum of this many of its largest choice scores), names (optional): expert (a prefix,
// the expert's index follows), gate, up, down, router, correction, shared
class RoutedFFN : public FeedForward {
public:
    RoutedFFN(const PartSpec &s, DType dt, Device *d) : FeedForward(s, dt, d) {
        hidden_ = s.get_int("hidden_size");
        experts_ = s.get_int("experts");
        ff_ = s.get_int("expert_ff");
        identity_ = s.get_int("identity", 0);
        top_ = s.get_int("top");
        groups_ = s.get_int("groups", 1);
        keep_ = s.get_int("group_keep", groups_);
        scale_ = s.has("scale") ? (float)s.get_double("scale") : 1.0f;
        correction_ = s.has("correction") && s.params.get("correction").as_bool();
        shared_ff_ = s.get_int("shared_ff", 0);
        std::string act = s.params.get("activation").is_string() ? s.params.get("activation").as_string() : "";
        act_ = ops::activation_kind(act);
        if (act_ < 0) config_error("routed: activation '" + act + "' is not one of relu2, relu, gelu_tanh, silu");
        gated_ = s.has("gated") && s.params.get("gated").as_bool();
        std::string score = s.params.get("score").is_string() ? s.params.get("score").as_string() : "softmax";
        if (score != "softmax" && score != "sigmoid") config_error("routed: score '" + score + "' is not softmax or sigmoid");
        sigmoid_ = score == "sigmoid";
        group_best_ = s.get_int("group_best", 1);
        if (group_best_ < 1) config_error("routed: group_best must be positive");
        if (gated_ && s.get_int("shared_ff", 0) > 0) config_error("routed: experts with a gate and a shared expert together are not built");
        long long outs = experts_ + identity_;
        if (hidden_ <= 0 || experts_ < 0 || identity_ < 0 || outs <= 0 || (experts_ > 0 && ff_ <= 0) ||
            shared_ff_ < 0)
            config_error("routed: sizes must be positive");
        if (outs > 2048) config_error("routed: the router's kernel takes up to 2048 outputs");
        if (groups_ <= 0 || outs % groups_) config_error("routed: the router's outputs do not form equal groups");
        if (keep_ <= 0 || keep_ > groups_) config_error("routed: group_keep must be between 1 and groups");
        if (top_ <= 0 || top_ > keep_ * (outs / groups_))
            config_error("routed: top must be between 1 and the outputs of the kept groups");
        const Json &nm = s.params.get("names");
        auto leaf = [&](const char *key, const char *dflt) {
            return nm.is_object() && nm.get(key).is_string() ? nm.get(key).as_string() : std::string(dflt);
        };
        n_expert_ = leaf("expert", "experts.");
        n_up_ = leaf("up", "up_proj.weight");
        n_down_ = leaf("down", "down_proj.weight");
        n_router_ = leaf("router", "router.weight");
        n_corr_ = leaf("correction", "router.correction");
        n_shared_ = leaf("shared", "shared");
        n_gate_ = leaf("gate", "gate_proj.weight");
        // the columns of the first product: experts, shared expert, padding to a
        // multiple of 8 (so that every row of sums can be read four values at a time), router
        act_width_ = experts_ * ff_ + shared_ff_;
        up_width_ = gated_ ? 2 * experts_ * ff_ : act_width_;
        router_col0_ = (up_width_ + 7) / 8 * 8;
    }

    void tensors(const std::string &p, TensorList &out) const override {
        for (long long e = 0; e < experts_; e++) {
            std::string ep = name(p, n_expert_ + std::to_string(e));
            if (gated_) out.emplace_back(name(ep, n_gate_), TensorSpec{{ff_, hidden_}, MATRIX, false});
            out.emplace_back(name(ep, n_up_), TensorSpec{{ff_, hidden_}, MATRIX, false});
            out.emplace_back(name(ep, n_down_), TensorSpec{{hidden_, ff_}, MATRIX, false});
        }
        out.emplace_back(name(p, n_router_), TensorSpec{{experts_ + identity_, hidden_}, MATRIX, false});
        if (correction_)
            out.emplace_back(name(p, n_corr_), TensorSpec{{experts_ + identity_}, PARAM, false, 0.0f, 0.05f});
        if (shared_ff_ > 0) {
            std::string sp = name(p, n_shared_);
            out.emplace_back(name(sp, n_up_), TensorSpec{{shared_ff_, hidden_}, MATRIX, false});
            out.emplace_back(name(sp, n_down_), TensorSpec{{hidden_, shared_ff_}, MATRIX, false});
        }
    }

    void load(const std::string &p, TensorMap &t) override {
        std::vector<DevTensor> ups, downs;
        for (long long e = 0; e < experts_; e++) {
            std::string ep = name(p, n_expert_ + std::to_string(e));
            if (gated_) ups.push_back(take(t, name(ep, n_gate_)));      // per expert [gate | up]
            ups.push_back(take(t, name(ep, n_up_)));
            downs.push_back(take(t, name(ep, n_down_)));
        }
        if (shared_ff_ > 0) {
            std::string sp = name(p, n_shared_);
            ups.push_back(take(t, name(sp, n_up_)));
            downs.push_back(take(t, name(sp, n_down_)));
        }
        DevTensor router = take(t, name(p, n_router_));
        if (router_col0_ > up_width_) ups.push_back(dev->tensor(router.dt, {router_col0_ - up_width_, hidden_}, true));
        ups.push_back(router);
        w_up_ = fuse_rows(*dev, ups);
        if (!downs.empty()) w_down_ = fuse_cols(*dev, downs);
        if (correction_) corr_ = take(t, name(p, n_corr_));
    }

    size_t weight_bytes() const override { return w_up_.bytes() + w_down_.bytes() + corr_.bytes(); }

    Stack forward(StepContext &ctx, const void *h) override {
        Device &d = *ctx.dev;
        long long n = ctx.n_rows;
        Stack z = ops::linear(d, h, ctx.dtype, n, hidden_, w_up_);
        ops::RouteParams r;
        r.experts = (int)(experts_ + identity_);
        r.groups = (int)groups_;
        r.keep = (int)keep_;
        r.top = (int)top_;
        r.first_identity = (int)experts_;
        r.scale = scale_;
        r.correction = correction_ ? (const float *)corr_.ptr : nullptr;
        r.sigmoid_scores = sigmoid_;
        r.group_best = (int)group_best_;
        Buf skip_coef;
        Buf weights = ops::moe_route(d, z, router_col0_, r, identity_ > 0 ? &skip_coef : nullptr);
        Stack out;
        if (act_width_ > 0) {
            Buf act = gated_ ? ops::gated_weighted(d, z, weights.as<float>(), (int)(experts_ + identity_),
                                                   (int)experts_, ff_, act_, ctx.dtype)
                             : ops::activation_weighted(d, z, act_width_, weights.as<float>(),
                                                        (int)(experts_ + identity_), (int)experts_, ff_, act_,
                                                        ctx.dtype);
            z = Stack();
            out = ops::linear(d, act.ptr, ctx.dtype, n, act_width_, w_down_);
        } else {
            // identity experts alone: nothing but the skip term
            out.S = 1;
            out.n = n;
            out.m = hidden_;
            out.buf = d.pool.get((size_t)n * (size_t)hidden_ * 4);
            cuda_check(cudaMemsetAsync(out.buf.ptr, 0, out.buf.bytes, d.stream), "clearing a sum");
        }
        if (identity_ > 0) {
            out.skip = h;
            out.skip_dt = ctx.dtype;
            out.skip_coef = skip_coef.as<float>();
            out.skip_coef_ld = 1;
            out.skip_hold = std::move(skip_coef);
        }
        return out;
    }

    Json info() const override {
        Json o = Json::object();
        o.set("experts", experts_);
        o.set("identity", identity_);
        o.set("router_col0", router_col0_);
        return o;
    }

private:
    long long hidden_, experts_, ff_, identity_, top_, groups_, keep_, shared_ff_;
    long long act_width_ = 0, up_width_ = 0, router_col0_ = 0, group_best_ = 1;
    bool gated_ = false, sigmoid_ = false;
    std::string n_gate_;
    float scale_;
    bool correction_;
    int act_;
    std::string n_expert_, n_up_, n_down_, n_router_, n_corr_, n_shared_;
    DevTensor w_up_, w_down_, corr_;
};

}  // namespace

void register_routed_feed_forwards() {
    register_part("feed_forward", "routed", [](const PartSpec &s, DType dt, Device *d) {
        return std::unique_ptr<Part>(new RoutedFFN(s, dt, d));
    });
}

}  // namespace jb
