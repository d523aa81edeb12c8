// Architecture-neutral description of a decoder: what the engine builds from.
//
// A typed architecture configuration (Qwen3Config) is turned into a ModelSpec.
// The spec is plain data: for every layer it names the mixer, the feed-forward,
// the norms and the block arrangement together with their constants, and
// run_order lists which layers run in which order.  The engine, the cache and
// the weight loader read only this spec, never the architecture's own
// configuration, so that a second architecture adds a configuration class and a
// to_model_spec and nothing else.
//
// The reference keeps the same information in a table row per architecture and
// per-layer fields (struct janas_arch src/llm/arch.h:21-62, struct layer
// src/llm/model_impl.h:36-106); layers that read another layer's keys and values
// are src/llm/model_load.c:1047-1056.
//
// A spec is also JSON (to_json / from_json): that is how a model that is not a
// registered architecture (a test's toy model) reaches the library.
#pragma once

#include <string>
#include <vector>

#include "../core/error.h"
#include "../core/json.h"

namespace jb {

// A configuration that cannot be built: a missing key, a wrong value.  The
// C interface reports it as JB_LLM_EOPEN (an unsupported architecture: EMODEL).
[[noreturn]] void config_error(const std::string &m, int code = JB_LLM_EOPEN);

// One part of a layer: its registered kind and its constants (a JSON object;
// a value may itself be a part, written {"kind": ..., "params": {...}}).
struct PartSpec {
    std::string kind;
    Json params = Json::object();

    bool has(const std::string &k) const { return params.has(k) && !params.get(k).is_null(); }
    long long get_int(const std::string &k) const;            // config_error when absent or not whole
    long long get_int(const std::string &k, long long dflt) const;
    double get_double(const std::string &k) const;
    PartSpec get_part(const std::string &k) const;

    Json to_json() const;
    static PartSpec from_json(const Json &j);
};

// One layer: how its parts are arranged and where its tensors are found.
// prefix is the layer's tensor-name prefix in the checkpoint; the four *_name
// fields are the sub-prefixes of its parts below it.
//
// A part whose kind is empty is absent: a layer may have no feed-forward (then it
// needs no ffn_norm either), an arrangement whose sublayers read the residual stream
// itself has no mixer_norm, and only some block arrangements have norms on the
// sublayers' results (post_mixer_norm, post_ffn_norm).  block_params are the
// arrangement's own constants and the names of tensors it owns (gates on the
// residual branches, for instance); they are found below `prefix` too.
struct LayerSpec {
    std::string block;
    PartSpec mixer, feed_forward, mixer_norm, ffn_norm;
    PartSpec post_mixer_norm, post_ffn_norm;
    Json block_params = Json::object();
    std::string prefix;
    std::string mixer_name = "self_attn";
    std::string ffn_name = "mlp";
    std::string mixer_norm_name = "input_layernorm";
    std::string ffn_norm_name = "post_attention_layernorm";
    std::string post_mixer_norm_name = "post_mixer_norm";
    std::string post_ffn_norm_name = "post_ffn_norm";
};

// One entry of the run order: run `layer` (its weights).  A layer may be named
// by several entries; every entry is a place of its own in the cache.  With
// cache_of >= 0 (the index of an earlier entry) the entry's mixer writes nothing
// and reads that entry's cache.
//
// add_embedding: before this entry runs, the embedding output (the residual stream
// as it was before the first entry) is added to the residual stream once more: the
// start of a repeated pass over layers that have run already.
struct RunEntry {
    int layer = 0;
    int cache_of = -1;
    bool add_embedding = false;
};

struct ModelSpec {
    std::string architecture;
    long long hidden_size = 0, vocab_size = 0, max_positions = 0;
    std::vector<LayerSpec> layers;
    std::vector<RunEntry> run_order;
    PartSpec final_norm;
    // a norm on the embedding rows before the first layer (kind "": none)
    PartSpec embedding_norm;
    std::string embedding_norm_name = "model.embed_norm";
    bool tie_embeddings = false;
    // a table [max_positions, hidden] of learned position vectors added to the
    // embedding rows ("" for none), and a factor on the logits
    std::string position_table_name;
    double logit_scale = 1.0;
    // a factor on the embedding rows as they enter the residual stream (a tied head reads
    // the table without it)
    double embedding_scale = 1.0;
    // a second table [vocab, token_table_width] of vectors per token ("" for none), which
    // the layers' blocks read by columns (a per-layer input of the token itself)
    std::string token_table_name;
    long long token_table_width = 0;
    std::string embedding_name = "model.embed_tokens.weight";
    std::string final_norm_name = "model.norm";
    std::string head_name = "lm_head.weight";

    void validate() const;          // config_error
    Json to_json() const;
    static ModelSpec from_json(const Json &j);
};

}  // namespace jb
