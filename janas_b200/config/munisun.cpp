// Typed configuration of the Munisun decoder, read from its config.json.
//
// The file names the design ("architecture": "Munisun"), the sizes (vocab, width), the
// constants (norm.eps, embedding.scale, token_side.dim) and a list of layers.  Each layer
// gives its mixer's type, the sizes of the mixer's two sides and its feed-forward, or null
// for none:
//
//   type "parallel":   mixer {left {heads, kv_heads, dim, vdim, scale, softcap, rot {base, dims,
//       scaling {factor, low, high, original}}}, right {heads, vdim, state, groups, conv,
//       norm_groups}, left_scale, right_scale}
//   type "parallel_2": mixer {left {heads, kv_heads, dim, vdim, scale, conv, rot {base, dims}},
//       right {heads, dim, vdim, decay [one number per head]}}
//   mlp {kind "dense", ff} or {kind "moe", expert {ff}, router {experts, top, groups {count, keep}}}
//
// What the design fixes is written here.  Every norm of the residual stream is an RMS norm
// whose stored weight lies around zero (the norm multiplies by 1 + w); a layer has a norm in
// front of and on the result of each sublayer; after the sublayers every layer adds an input
// of the token itself, from its own columns of a second table of vectors per token.  The
// two sides of a mixer read the same normed input.  "parallel": softmax attention with a
// weighted RMS norm per head on q and k before the rotation, a cap on the scores and a
// sigmoid gate on the joined heads, beside a Mamba-2 recurrence; the results are added with
// the two factors.  "parallel_2": softmax attention with a short convolution over time on
// q, k and v and an unweighted RMS norm per head on q and k after the rotation, beside a
// linear attention with a decay per head; each result is RMS-normed over the width with a
// weight of its own, and the mixer gives half their sum.  The rotation turns neighbours
// (2i, 2i + 1).  Experts and the dense feed-forward are SwiGLU; the router's scores are
// sigmoids, a correction joins them for the choice alone, a group's score is the sum of its
// two largest choice scores, and the chosen experts' scores weigh them as they are.
//
// Tensor names: embed, side.embed, final.norm, head; layer i below "l<i>": norm1, norm1b,
// norm2, norm2b, mix.left.{q, k, v, o, g, q.norm, k.norm, q.conv, k.conv, v.conv},
// mix.right.{in, conv, conv.b, dt_bias, A_log, D, norm, o} or mix.right.{q, k, v, g, o, norm},
// mix.left.out, mix.right.out, mlp.{gate, up, down} or mlp.{e<j>.gate, e<j>.up, e<j>.down,
// router, correction}, side.{gate, proj, norm}.
#include "munisun.h"

namespace jb {

namespace {

long long need_int(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number() || !v.whole())
        config_error("config.json: " + where + key + " must be a whole number, got " + v.dump());
    return v.as_int();
}

double need_num(const Json &d, const char *key, const std::string &where) {
    const Json &v = d.get(key);
    if (v.is_bool() || !v.is_number())
        config_error("config.json: " + where + key + " must be a number, got " + v.dump());
    return v.as_double();
}

long long opt_int(const Json &d, const char *key, const std::string &where, long long dflt) {
    return d.get(key).is_null() ? dflt : need_int(d, key, where);
}

const Json &need_obj(const Json &d, const char *key, const std::string &where) {
    if (!d.get(key).is_object()) config_error("config.json: " + where + key + " must be an object");
    return d.get(key);
}

MunisunConfig::Attention read_attention(const Json &m, const std::string &w) {
    MunisunConfig::Attention a;
    a.heads = need_int(m, "heads", w);
    a.kv_heads = opt_int(m, "kv_heads", w, a.heads);
    a.dim = need_int(m, "dim", w);
    a.vdim = opt_int(m, "vdim", w, a.dim);
    a.scale = need_num(m, "scale", w);
    if (!m.get("softcap").is_null()) a.softcap = need_num(m, "softcap", w);
    a.conv = opt_int(m, "conv", w, 0);
    if (!m.get("rot").is_null()) {
        const Json &r = need_obj(m, "rot", w);
        a.rot_dims = need_int(r, "dims", w + "rot.");
        a.rot_base = need_num(r, "base", w + "rot.");
        if (!r.get("scaling").is_null()) {
            const Json &sc = need_obj(r, "scaling", w + "rot.");
            a.rot_scaling = true;
            a.sc_factor = need_num(sc, "factor", w + "rot.scaling.");
            a.sc_low = need_num(sc, "low", w + "rot.scaling.");
            a.sc_high = need_num(sc, "high", w + "rot.scaling.");
            a.sc_original = need_num(sc, "original", w + "rot.scaling.");
        }
    }
    return a;
}

Json attention_json(const MunisunConfig::Attention &a) {
    Json m = Json::object();
    if (a.conv > 0) m.set("conv", a.conv);
    m.set("dim", a.dim);
    m.set("heads", a.heads);
    m.set("kv_heads", a.kv_heads);
    if (a.rot_dims > 0) {
        Json r = Json::object();
        r.set("base", a.rot_base);
        r.set("dims", a.rot_dims);
        if (a.rot_scaling) {
            Json sc = Json::object();
            sc.set("factor", a.sc_factor);
            sc.set("high", a.sc_high);
            sc.set("low", a.sc_low);
            sc.set("original", a.sc_original);
            r.set("scaling", sc);
        }
        m.set("rot", r);
    }
    m.set("scale", a.scale);
    if (a.softcap > 0) m.set("softcap", a.softcap);
    m.set("vdim", a.vdim);
    return m;
}

}  // namespace

MunisunConfig MunisunConfig::from_json(const Json &d) {
    MunisunConfig c;
    c.vocab = need_int(d, "vocab", "");
    c.width = need_int(d, "width", "");
    c.norm_eps = need_num(need_obj(d, "norm", ""), "eps", "norm.");
    if (!d.get("embedding").is_null() && !need_obj(d, "embedding", "").get("scale").is_null())
        c.embedding_scale = need_num(d.get("embedding"), "scale", "embedding.");
    if (!d.get("token_side").is_null()) c.side_dim = need_int(need_obj(d, "token_side", ""), "dim", "token_side.");
    const Json &ls = d.get("layers");
    if (!ls.is_array() || ls.size() == 0) config_error("config.json: layers must be a list of layers");
    for (size_t i = 0; i < ls.size(); i++) {
        const Json &l = ls[i];
        std::string where = fmt("layers[%zu].", i);
        if (!l.is_object() || !l.get("type").is_string() || !l.get("mixer").is_object())
            config_error("config.json: " + where + " needs a type and a mixer");
        Layer y;
        y.type = l.get("type").as_string();
        const Json &m = l.get("mixer");
        std::string mw = where + "mixer.";
        if (y.type != "parallel" && y.type != "parallel_2")
            config_error("config.json: " + where + "type '" + y.type +
                         "': this design's mixers are 'parallel' and 'parallel_2'");
        y.left = read_attention(need_obj(m, "left", mw), mw + "left.");
        const Json &r = need_obj(m, "right", mw);
        std::string rw = mw + "right.";
        if (y.type == "parallel") {
            y.ssm_heads = need_int(r, "heads", rw);
            y.ssm_vdim = need_int(r, "vdim", rw);
            y.ssm_state = need_int(r, "state", rw);
            y.ssm_groups = opt_int(r, "groups", rw, 1);
            y.ssm_conv = opt_int(r, "conv", rw, 1);
            y.ssm_norm_groups = opt_int(r, "norm_groups", rw, 1);
            if (!m.get("left_scale").is_null()) y.left_scale = need_num(m, "left_scale", mw);
            if (!m.get("right_scale").is_null()) y.right_scale = need_num(m, "right_scale", mw);
        } else {
            y.lin_heads = need_int(r, "heads", rw);
            y.lin_dim = need_int(r, "dim", rw);
            y.lin_vdim = opt_int(r, "vdim", rw, y.lin_dim);
            const Json &dc = r.get("decay");
            if (!dc.is_array()) config_error("config.json: " + rw + "decay must list one number per head");
            for (size_t k = 0; k < dc.size(); k++) {
                if (dc[k].is_bool() || !dc[k].is_number())
                    config_error("config.json: " + rw + "decay must list numbers");
                y.lin_decay.push_back(dc[k].as_double());
            }
        }
        const Json &f = l.get("mlp");
        if (!f.is_null()) {
            std::string fw = where + "mlp.";
            if (!f.is_object() || !f.get("kind").is_string())
                config_error("config.json: " + where + "mlp must be null or an object with a kind");
            y.has_mlp = true;
            y.mlp_kind = f.get("kind").as_string();
            if (y.mlp_kind == "dense") {
                y.ff = need_int(f, "ff", fw);
            } else if (y.mlp_kind == "moe") {
                const Json &ro = need_obj(f, "router", fw);
                y.experts = need_int(ro, "experts", fw + "router.");
                y.top = need_int(ro, "top", fw + "router.");
                if (!ro.get("groups").is_null()) {
                    const Json &g = need_obj(ro, "groups", fw + "router.");
                    y.groups = need_int(g, "count", fw + "router.groups.");
                    y.group_keep = opt_int(g, "keep", fw + "router.groups.", y.groups);
                }
                y.expert_ff = need_int(need_obj(f, "expert", fw), "ff", fw + "expert.");
            } else {
                config_error("config.json: " + fw + "kind '" + y.mlp_kind + "': this design's are 'dense' and 'moe'");
            }
        }
        c.layers.push_back(y);
    }
    c.validate();
    return c;
}

void MunisunConfig::validate() const {
    if (vocab <= 0 || width <= 0) config_error("config.json: vocab and width must be positive");
    if (layers.empty() || layers.size() > 100000) config_error("config.json: layers must not be empty");
    if (side_dim < 0) config_error("config.json: token_side.dim must be positive");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        std::string where = fmt("config.json: layers[%zu]: ", i);
        const Attention &a = y.left;
        if (a.heads <= 0 || a.dim <= 0 || a.vdim <= 0) config_error(where + "heads, dim and vdim must be positive");
        if (a.kv_heads <= 0 || a.heads % a.kv_heads) config_error(where + "heads must be a multiple of kv_heads");
        if (a.dim > 512 || a.vdim > 512) config_error(where + "the attention kernels take head sizes up to 512");
        if (a.rot_dims < 0 || a.rot_dims % 2 || a.rot_dims > a.dim)
            config_error(where + "rot.dims must be even and at most dim");
        if (a.rot_dims > 0 && a.rot_base <= 0) config_error(where + "rot.base must be positive");
        if (a.softcap < 0 || a.conv < 0) config_error(where + "softcap and conv must not be negative");
        if (y.type == "parallel") {
            if (y.ssm_heads <= 0 || y.ssm_vdim <= 0 || y.ssm_state <= 0 || y.ssm_groups <= 0 || y.ssm_conv <= 0 ||
                y.ssm_norm_groups <= 0)
                config_error(where + "the right side's sizes must be positive");
            if (y.ssm_heads % y.ssm_groups) config_error(where + "right.heads must be a multiple of right.groups");
            if ((y.ssm_heads * y.ssm_vdim) % y.ssm_norm_groups)
                config_error(where + "right.norm_groups must divide heads * vdim");
        } else {
            if (y.lin_heads <= 0 || y.lin_dim <= 0 || y.lin_vdim <= 0)
                config_error(where + "the right side's sizes must be positive");
            if ((long long)y.lin_decay.size() != y.lin_heads)
                config_error(where + "right.decay must list one number per head");
        }
        if (y.has_mlp && y.mlp_kind == "dense" && y.ff <= 0) config_error(where + "mlp.ff must be positive");
        if (y.has_mlp && y.mlp_kind == "moe") {
            if (y.experts <= 0 || y.expert_ff <= 0) config_error(where + "the router needs experts");
            if (y.groups <= 0 || y.experts % y.groups) config_error(where + "the experts do not form equal groups");
            if (y.group_keep <= 0 || y.group_keep > y.groups)
                config_error(where + "router.groups.keep must be between 1 and count");
            if (y.top <= 0 || y.top > y.group_keep * (y.experts / y.groups))
                config_error(where + "router.top must be between 1 and the experts of the kept groups");
        }
    }
}

Json MunisunConfig::to_json() const {
    Json d = Json::object();
    d.set("architecture", "Munisun");
    Json em = Json::object();
    em.set("scale", embedding_scale);
    d.set("embedding", em);
    Json ls = Json::array();
    for (auto &y : layers) {
        Json l = Json::object(), m = Json::object(), r = Json::object();
        m.set("left", attention_json(y.left));
        if (y.type == "parallel") {
            r.set("conv", y.ssm_conv);
            r.set("groups", y.ssm_groups);
            r.set("heads", y.ssm_heads);
            r.set("norm_groups", y.ssm_norm_groups);
            r.set("state", y.ssm_state);
            r.set("vdim", y.ssm_vdim);
            m.set("left_scale", y.left_scale);
            m.set("right_scale", y.right_scale);
        } else {
            Json dc = Json::array();
            for (double v : y.lin_decay) dc.push(Json(v));
            r.set("decay", dc);
            r.set("dim", y.lin_dim);
            r.set("heads", y.lin_heads);
            r.set("vdim", y.lin_vdim);
        }
        m.set("right", r);
        l.set("mixer", m);
        if (y.has_mlp && y.mlp_kind == "dense") {
            Json f = Json::object();
            f.set("ff", y.ff);
            f.set("kind", y.mlp_kind);
            l.set("mlp", f);
        } else if (y.has_mlp) {
            Json f = Json::object(), e = Json::object(), ro = Json::object(), g = Json::object();
            e.set("ff", y.expert_ff);
            f.set("expert", e);
            f.set("kind", y.mlp_kind);
            ro.set("experts", y.experts);
            g.set("count", y.groups);
            g.set("keep", y.group_keep);
            ro.set("groups", g);
            ro.set("top", y.top);
            f.set("router", ro);
            l.set("mlp", f);
        } else {
            l.set("mlp", Json());
        }
        l.set("type", y.type);
        ls.push(l);
    }
    d.set("layers", ls);
    Json n = Json::object();
    n.set("eps", norm_eps);
    d.set("norm", n);
    if (side_dim > 0) {
        Json ts = Json::object();
        ts.set("dim", side_dim);
        d.set("token_side", ts);
    }
    d.set("vocab", vocab);
    d.set("width", width);
    return d;
}

ModelSpec MunisunConfig::to_model_spec() const {
    // every norm of the residual stream: an RMS norm over the width whose weight, named as
    // the norm itself, is stored around zero
    PartSpec norm{"rmsnorm", Json::object()};
    norm.params.set("size", width);
    norm.params.set("eps", norm_eps);
    norm.params.set("one_plus", true);
    {
        Json nm = Json::object();
        nm.set("weight", "");
        norm.params.set("names", nm);
    }
    // the design gives no limit on positions: the cache's size is the limit
    const long long positions = 1ll << 30;
    ModelSpec s;
    s.architecture = "Munisun";
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = positions;
    s.embedding_name = "embed";
    s.embedding_scale = embedding_scale;
    s.head_name = "head";
    s.tie_embeddings = false;
    s.final_norm_name = "final.norm";
    s.final_norm = norm;
    if (side_dim > 0) {
        s.token_table_name = "side.embed";
        s.token_table_width = side_dim * (long long)layers.size();
    }
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        const Attention &a = y.left;
        bool parallel = y.type == "parallel";
        PartSpec left{"sink_attention", Json::object()};
        left.params.set("hidden_size", width);
        left.params.set("num_heads", a.heads);
        left.params.set("num_kv_heads", a.kv_heads);
        left.params.set("head_dim", a.dim);
        left.params.set("v_head_dim", a.vdim);
        left.params.set("scale", a.scale);
        left.params.set("bias", false);
        if (a.softcap > 0) left.params.set("softcap", a.softcap);
        if (parallel) {
            left.params.set("qk_norm_eps", norm_eps);
            left.params.set("gate", true);
        } else {
            left.params.set("qk_unit_norm_eps", norm_eps);
        }
        if (a.conv > 0) left.params.set("conv_taps", a.conv);
        if (a.rot_dims > 0) {
            PartSpec pos{"rope_pairs", Json::object()};
            pos.params.set("rotary_dim", a.rot_dims);
            pos.params.set("theta", a.rot_base);
            pos.params.set("max_positions", positions);
            if (a.rot_scaling) {
                Json sc = Json::object();
                sc.set("factor", a.sc_factor);
                sc.set("low", a.sc_low);
                sc.set("high", a.sc_high);
                sc.set("original", a.sc_original);
                pos.params.set("scaling", sc);
            }
            left.params.set("position", pos.to_json());
        }
        {
            Json nm = Json::object();
            nm.set("q", "q");
            nm.set("k", "k");
            nm.set("v", "v");
            nm.set("o", "o");
            nm.set("gate", "g");
            nm.set("q_norm", "q.norm");
            nm.set("k_norm", "k.norm");
            nm.set("conv", ".conv");
            left.params.set("names", nm);
        }
        PartSpec right;
        if (parallel) {
            right.kind = "mamba2";
            right.params.set("hidden_size", width);
            right.params.set("heads", y.ssm_heads);
            right.params.set("head_dim", y.ssm_vdim);
            right.params.set("state", y.ssm_state);
            right.params.set("groups", y.ssm_groups);
            right.params.set("conv_taps", y.ssm_conv);
            right.params.set("norm_groups", y.ssm_norm_groups);
            right.params.set("eps", norm_eps);
            Json nm = Json::object();
            nm.set("in", "in");
            nm.set("conv", "conv");
            nm.set("conv_bias", "conv.b");
            nm.set("dt_bias", "dt_bias");
            nm.set("a_log", "A_log");
            nm.set("d", "D");
            nm.set("norm", "norm");
            nm.set("o", "o");
            right.params.set("names", nm);
        } else {
            right.kind = "decay_attention";
            right.params.set("hidden_size", width);
            right.params.set("heads", y.lin_heads);
            right.params.set("head_dim", y.lin_dim);
            right.params.set("v_head_dim", y.lin_vdim);
            Json dc = Json::array();
            for (double v : y.lin_decay) dc.push(Json(v));
            right.params.set("decay", dc);
            right.params.set("eps", norm_eps);
            Json nm = Json::object();
            nm.set("q", "q");
            nm.set("k", "k");
            nm.set("v", "v");
            nm.set("g", "g");
            nm.set("o", "o");
            nm.set("norm", "norm");
            right.params.set("names", nm);
        }
        PartSpec mixer{"pair", Json::object()};
        mixer.params.set("hidden_size", width);
        mixer.params.set("left", left.to_json());
        mixer.params.set("right", right.to_json());
        if (parallel) {
            mixer.params.set("join", "sum");
            mixer.params.set("left_scale", y.left_scale);
            mixer.params.set("right_scale", y.right_scale);
        } else {
            mixer.params.set("join", "normed_mean");
            mixer.params.set("eps", norm_eps);
        }
        {
            Json nm = Json::object();
            nm.set("left", "left");
            nm.set("right", "right");
            nm.set("left_out", "left.out");
            nm.set("right_out", "right.out");
            mixer.params.set("names", nm);
        }
        LayerSpec l;
        l.block = "sandwich";
        l.prefix = fmt("l%zu", i);
        l.mixer = mixer;
        l.mixer_name = "mix";
        l.mixer_norm = norm;
        l.mixer_norm_name = "norm1";
        l.post_mixer_norm = norm;
        l.post_mixer_norm_name = "norm1b";
        l.block_params.set("hidden_size", width);
        if (side_dim > 0) {
            Json ts = Json::object(), nm = Json::object();
            ts.set("dim", side_dim);
            ts.set("col0", side_dim * (long long)i);
            ts.set("eps", norm_eps);
            nm.set("gate", "side.gate");
            nm.set("proj", "side.proj");
            nm.set("norm", "side.norm");
            ts.set("names", nm);
            l.block_params.set("token_side", ts);
        }
        if (y.has_mlp) {
            PartSpec ffn;
            if (y.mlp_kind == "dense") {
                ffn.kind = "swiglu";
                ffn.params.set("hidden_size", width);
                ffn.params.set("intermediate_size", y.ff);
                Json nm = Json::object();
                nm.set("gate", "gate");
                nm.set("up", "up");
                nm.set("down", "down");
                ffn.params.set("names", nm);
            } else {
                ffn.kind = "routed";
                ffn.params.set("hidden_size", width);
                ffn.params.set("experts", y.experts);
                ffn.params.set("expert_ff", y.expert_ff);
                ffn.params.set("top", y.top);
                ffn.params.set("groups", y.groups);
                ffn.params.set("group_keep", y.group_keep);
                ffn.params.set("group_best", 2);
                ffn.params.set("score", "sigmoid");
                ffn.params.set("correction", true);
                ffn.params.set("gated", true);
                ffn.params.set("activation", "silu");
                Json nm = Json::object();
                nm.set("expert", "e");
                nm.set("gate", "gate");
                nm.set("up", "up");
                nm.set("down", "down");
                nm.set("router", "router");
                nm.set("correction", "correction");
                ffn.params.set("names", nm);
            }
            l.feed_forward = ffn;
            l.ffn_name = "mlp";
            l.ffn_norm = norm;
            l.ffn_norm_name = "norm2";
            l.post_ffn_norm = norm;
            l.post_ffn_norm_name = "norm2b";
        }
        s.layers.push_back(l);
    }
    for (size_t i = 0; i < layers.size(); i++) {
        RunEntry r;
        r.layer = (int)i;
        s.run_order.push_back(r);
    }
    s.validate();
    return s;
}

void register_munisun() {
    register_architecture("Munisun", "munisun", [](const Json &d) {
        return std::unique_ptr<ArchConfig>(new MunisunConfig(MunisunConfig::from_json(d)));
    });
}

}  // namespace jb
