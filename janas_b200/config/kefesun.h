// The Kefesun decoder's typed configuration (see kefesun.cpp).
#pragma once

#include <string>
#include <vector>

#include "registry.h"

namespace jb {

struct KefesunConfig : ArchConfig {
    struct Layer {
        std::string type;                 // which mixer: "attention" or "mingru"
        // attention
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        double scale = 0;
        long long window = 0;             // mask.size; 0: every earlier position is seen
        long long keep_first = 0;         // mask.keep_first: first positions seen beside the window
        long long rot_dims = 0;           // 0: no rotation
        double rot_base = 0;
        // mingru
        long long gru_width = 0;
        // feed-forward
        bool has_mlp = false;
        std::string mlp_kind;             // "moe"
        long long experts = 0, expert_ff = 0, identity = 0, top = 0;
        long long groups = 1, group_keep = 1;
        double router_scale = 1.0;
        long long shared_ff = 0;          // 0: no shared expert
    };
    long long vocab = 0, width = 0;
    double norm_eps = 0, embedding_scale = 1.0;
    long long taps = 0;                   // canon.taps; 0: the sublayers read the residual stream as it is
    std::vector<Layer> layers;

    static KefesunConfig from_json(const Json &config_json);
    void validate() const;

    std::string architecture() const override { return "Kefesun"; }
    Json to_json() const override;
    ModelSpec to_model_spec() const override;
};

void register_kefesun();

}  // namespace jb
