// Typed configuration of the Kefesun decoder, read from its config.json.
//
// The file names the design ("architecture": "Kefesun"), the sizes (vocab, width), the
// constants (norm.eps, embedding.scale, canon.taps) and a list of layers.  Each layer
// gives its mixer's type and sizes and its feed-forward, or null for none:
//
//   type "attention": heads, kv_heads, dim, vdim, scale, and optionally mask {size,
//       keep_first} (a sliding window with first positions that stay visible) and
//       rot {base, dims} (a rotation of the first dims values of each head)
//   type "mingru": width
//   mlp {kind "moe", expert {ff}, router {experts, top, identity, scale, groups {count,
//       keep}}, shared {ff} or null}
//
// What the design fixes is written here.  The embedding rows are multiplied by
// embedding.scale and the head is the embedding table itself, without the factor.  A
// layer has no norm in front of a sublayer: each sublayer reads the residual stream
// through a short causal convolution (x + conv(x), canon.taps taps) and its result goes
// through a layer norm with a weight and no bias before it is added.  The attention
// mixer has biases on q, k and v (none on o), an RMS norm per head on q and k with the
// layer's eps, rotates value i of a head with value i + dims / 2, and weighs a visible
// key by sigmoid(score + a learned number per head), without a softmax.  The minGRU's z
// and x have biases, g and o have none.  The experts' activation is the square of relu;
// a correction vector is added to the router's scores for the choice alone.
//
// Tensor names: embed, final.norm; layer i below "l<i>": norm1, norm2, canon1, canon2,
// mix.{q, q.b, k, k.b, v, v.b, q.norm, k.norm, pb, o} or mix.{z, z.b, x, x.b, g, o},
// mlp.{e<j>.up, e<j>.down, router, correction, shared.up, shared.down}.
#include "kefesun.h"

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

}  // namespace

KefesunConfig KefesunConfig::from_json(const Json &d) {
    KefesunConfig c;
    c.vocab = need_int(d, "vocab", "");
    c.width = need_int(d, "width", "");
    if (!d.get("norm").is_object()) config_error("config.json: norm must be an object with eps");
    c.norm_eps = need_num(d.get("norm"), "eps", "norm.");
    if (!d.get("embedding").is_null()) {
        if (!d.get("embedding").is_object()) config_error("config.json: embedding must be an object with scale");
        if (!d.get("embedding").get("scale").is_null())
            c.embedding_scale = need_num(d.get("embedding"), "scale", "embedding.");
    }
    if (!d.get("canon").is_null()) {
        if (!d.get("canon").is_object()) config_error("config.json: canon must be an object with taps");
        c.taps = need_int(d.get("canon"), "taps", "canon.");
        if (c.taps < 1) config_error("config.json: canon.taps must be positive");
    }
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
        if (y.type == "attention") {
            y.heads = need_int(m, "heads", mw);
            y.kv_heads = opt_int(m, "kv_heads", mw, y.heads);
            y.dim = need_int(m, "dim", mw);
            y.vdim = opt_int(m, "vdim", mw, y.dim);
            y.scale = need_num(m, "scale", mw);
            if (!m.get("mask").is_null()) {
                if (!m.get("mask").is_object())
                    config_error("config.json: " + mw + "mask must be an object with size");
                y.window = need_int(m.get("mask"), "size", mw + "mask.");
                if (y.window <= 0) config_error("config.json: " + mw + "mask.size must be positive");
                y.keep_first = opt_int(m.get("mask"), "keep_first", mw + "mask.", 0);
            }
            if (!m.get("rot").is_null()) {
                if (!m.get("rot").is_object())
                    config_error("config.json: " + mw + "rot must be an object with base and dims");
                y.rot_dims = need_int(m.get("rot"), "dims", mw + "rot.");
                y.rot_base = need_num(m.get("rot"), "base", mw + "rot.");
            }
        } else if (y.type == "mingru") {
            y.gru_width = need_int(m, "width", mw);
        } else {
            config_error("config.json: " + where + "type '" + y.type +
                         "': this design's mixers are 'attention' and 'mingru'");
        }
        const Json &f = l.get("mlp");
        if (!f.is_null()) {
            std::string fw = where + "mlp.";
            if (!f.is_object() || !f.get("kind").is_string())
                config_error("config.json: " + where + "mlp must be null or an object with a kind");
            y.has_mlp = true;
            y.mlp_kind = f.get("kind").as_string();
            if (y.mlp_kind != "moe")
                config_error("config.json: " + fw + "kind '" + y.mlp_kind + "': this design's is 'moe'");
            const Json &r = f.get("router");
            if (!r.is_object()) config_error("config.json: " + fw + "router must be an object");
            y.experts = need_int(r, "experts", fw + "router.");
            y.top = need_int(r, "top", fw + "router.");
            y.identity = opt_int(r, "identity", fw + "router.", 0);
            y.router_scale = r.get("scale").is_null() ? 1.0 : need_num(r, "scale", fw + "router.");
            if (!r.get("groups").is_null()) {
                if (!r.get("groups").is_object())
                    config_error("config.json: " + fw + "router.groups must be an object with count and keep");
                y.groups = need_int(r.get("groups"), "count", fw + "router.groups.");
                y.group_keep = opt_int(r.get("groups"), "keep", fw + "router.groups.", y.groups);
            }
            if (y.experts > 0) {
                if (!f.get("expert").is_object()) config_error("config.json: " + fw + "expert must be an object with ff");
                y.expert_ff = need_int(f.get("expert"), "ff", fw + "expert.");
            }
            if (!f.get("shared").is_null()) {
                if (!f.get("shared").is_object()) config_error("config.json: " + fw + "shared must be null or an object with ff");
                y.shared_ff = need_int(f.get("shared"), "ff", fw + "shared.");
            }
        }
        c.layers.push_back(y);
    }
    c.validate();
    return c;
}

void KefesunConfig::validate() const {
    if (vocab <= 0 || width <= 0) config_error("config.json: vocab and width must be positive");
    if (layers.empty() || layers.size() > 100000) config_error("config.json: layers must not be empty");
    if (taps < 0) config_error("config.json: canon.taps must be positive");
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        std::string where = fmt("config.json: layers[%zu]: ", i);
        if (y.type == "attention") {
            if (y.heads <= 0 || y.dim <= 0 || y.vdim <= 0) config_error(where + "heads, dim and vdim must be positive");
            if (y.kv_heads <= 0 || y.heads % y.kv_heads) config_error(where + "heads must be a multiple of kv_heads");
            if (y.dim > 512 || y.vdim > 512) config_error(where + "the attention kernels take head sizes up to 512");
            if (y.rot_dims < 0 || y.rot_dims % 2 || y.rot_dims > y.dim)
                config_error(where + "rot.dims must be even and at most dim");
            if (y.rot_dims > 0 && y.rot_base <= 0) config_error(where + "rot.base must be positive");
            if (y.keep_first < 0) config_error(where + "mask.keep_first must not be negative");
        } else {
            if (y.gru_width <= 0) config_error(where + "mixer.width must be positive");
        }
        if (y.has_mlp) {
            long long outs = y.experts + y.identity;
            if (y.experts < 0 || y.identity < 0 || outs <= 0) config_error(where + "the router needs experts");
            if (y.experts > 0 && y.expert_ff <= 0) config_error(where + "mlp.expert.ff must be positive");
            if (y.groups <= 0 || outs % y.groups) config_error(where + "the router's outputs do not form equal groups");
            if (y.group_keep <= 0 || y.group_keep > y.groups)
                config_error(where + "router.groups.keep must be between 1 and count");
            if (y.top <= 0 || y.top > y.group_keep * (outs / y.groups))
                config_error(where + "router.top must be between 1 and the outputs of the kept groups");
            if (y.shared_ff < 0) config_error(where + "mlp.shared.ff must be positive");
        }
    }
}

Json KefesunConfig::to_json() const {
    Json d = Json::object();
    d.set("architecture", "Kefesun");
    if (taps > 0) {
        Json c = Json::object();
        c.set("taps", taps);
        d.set("canon", c);
    } else {
        d.set("canon", Json());
    }
    Json em = Json::object();
    em.set("scale", embedding_scale);
    d.set("embedding", em);
    Json ls = Json::array();
    for (auto &y : layers) {
        Json l = Json::object(), m = Json::object();
        if (y.type == "attention") {
            m.set("dim", y.dim);
            m.set("heads", y.heads);
            m.set("kv_heads", y.kv_heads);
            if (y.window > 0) {
                Json w = Json::object();
                w.set("keep_first", y.keep_first);
                w.set("size", y.window);
                m.set("mask", w);
            } else {
                m.set("mask", Json());
            }
            if (y.rot_dims > 0) {
                Json r = Json::object();
                r.set("base", y.rot_base);
                r.set("dims", y.rot_dims);
                m.set("rot", r);
            } else {
                m.set("rot", Json());
            }
            m.set("scale", y.scale);
            m.set("vdim", y.vdim);
        } else {
            m.set("width", y.gru_width);
        }
        l.set("mixer", m);
        if (y.has_mlp) {
            Json f = Json::object(), e = Json::object(), r = Json::object(), g = Json::object();
            e.set("ff", y.expert_ff);
            f.set("expert", e);
            f.set("kind", y.mlp_kind);
            r.set("experts", y.experts);
            g.set("count", y.groups);
            g.set("keep", y.group_keep);
            r.set("groups", g);
            r.set("identity", y.identity);
            r.set("scale", y.router_scale);
            r.set("top", y.top);
            f.set("router", r);
            if (y.shared_ff > 0) {
                Json sh = Json::object();
                sh.set("ff", y.shared_ff);
                f.set("shared", sh);
            } else {
                f.set("shared", Json());
            }
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
    d.set("vocab", vocab);
    d.set("width", width);
    return d;
}

ModelSpec KefesunConfig::to_model_spec() const {
    // every norm of the residual stream: a layer norm over the width with a weight, named
    // as the norm itself, and no bias
    PartSpec norm{"layernorm", Json::object()};
    norm.params.set("size", width);
    norm.params.set("eps", norm_eps);
    {
        Json nm = Json::object();
        nm.set("weight", "");
        nm.set("bias", Json());
        norm.params.set("names", nm);
    }
    // the design gives no limit on positions: the cache's size is the limit
    const long long positions = 1ll << 30;
    ModelSpec s;
    s.architecture = "Kefesun";
    s.hidden_size = width;
    s.vocab_size = vocab;
    s.max_positions = positions;
    s.embedding_name = "embed";
    s.embedding_scale = embedding_scale;
    s.head_name = "head";           // no such tensor: the head is the embedding table
    s.tie_embeddings = true;
    s.final_norm_name = "final.norm";
    s.final_norm = norm;
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        PartSpec mixer;
        if (y.type == "attention") {
            mixer.kind = "sink_attention";
            mixer.params.set("hidden_size", width);
            mixer.params.set("num_heads", y.heads);
            mixer.params.set("num_kv_heads", y.kv_heads);
            mixer.params.set("head_dim", y.dim);
            mixer.params.set("v_head_dim", y.vdim);
            mixer.params.set("scale", y.scale);
            mixer.params.set("window", y.window);
            mixer.params.set("keep_first", y.window > 0 ? y.keep_first : 0);
            mixer.params.set("qk_norm_eps", norm_eps);
            mixer.params.set("score_bias", true);
            mixer.params.set("bias", true);
            mixer.params.set("out_bias", false);
            mixer.params.set("head_scale", false);
            mixer.params.set("sink", false);
            mixer.params.set("own_kv", true);
            if (y.rot_dims > 0) {
                PartSpec pos{"rope_neox", Json::object()};
                pos.params.set("rotary_dim", y.rot_dims);
                pos.params.set("theta", y.rot_base);
                pos.params.set("max_positions", positions);
                mixer.params.set("position", pos.to_json());
            }
            Json nm = Json::object();
            nm.set("q", "q");
            nm.set("k", "k");
            nm.set("v", "v");
            nm.set("o", "o");
            nm.set("bias", ".b");
            nm.set("q_norm", "q.norm");
            nm.set("k_norm", "k.norm");
            nm.set("score_bias", "pb");
            mixer.params.set("names", nm);
        } else {
            mixer.kind = "mingru";
            mixer.params.set("hidden_size", width);
            mixer.params.set("width", y.gru_width);
            mixer.params.set("bias", true);
            Json nm = Json::object();
            nm.set("z", "z");
            nm.set("x", "x");
            nm.set("g", "g");
            nm.set("o", "o");
            nm.set("bias", ".b");
            mixer.params.set("names", nm);
        }
        LayerSpec l;
        l.block = "result_norm";
        l.prefix = fmt("l%zu", i);
        l.mixer = mixer;
        l.mixer_name = "mix";
        l.post_mixer_norm = norm;
        l.post_mixer_norm_name = "norm1";
        l.block_params.set("hidden_size", width);
        l.block_params.set("conv_taps", taps);
        l.block_params.set("mixer_conv", "canon1");
        l.block_params.set("ffn_conv", "canon2");
        if (y.has_mlp) {
            PartSpec ffn{"routed", Json::object()};
            ffn.params.set("hidden_size", width);
            ffn.params.set("experts", y.experts);
            ffn.params.set("expert_ff", y.expert_ff);
            ffn.params.set("identity", y.identity);
            ffn.params.set("top", y.top);
            ffn.params.set("groups", y.groups);
            ffn.params.set("group_keep", y.group_keep);
            ffn.params.set("scale", y.router_scale);
            ffn.params.set("correction", true);
            ffn.params.set("shared_ff", y.shared_ff);
            ffn.params.set("activation", "relu2");
            Json nm = Json::object();
            nm.set("expert", "e");
            nm.set("up", "up");
            nm.set("down", "down");
            nm.set("router", "router");
            nm.set("correction", "correction");
            nm.set("shared", "shared");
            ffn.params.set("names", nm);
            l.feed_forward = ffn;
            l.ffn_name = "mlp";
            l.post_ffn_norm = norm;
            l.post_ffn_norm_name = "norm2";
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

void register_kefesun() {
    register_architecture("Kefesun", "kefesun", [](const Json &d) {
        return std::unique_ptr<ArchConfig>(new KefesunConfig(KefesunConfig::from_json(d)));
    });
}

}  // namespace jb
