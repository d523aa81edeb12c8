// The Munisun decoder's typed configuration (see munisun.cpp).
#pragma once

#include <string>
#include <vector>

#include "registry.h"

namespace jb {

struct MunisunConfig : ArchConfig {
    // the softmax attention side of a mixer
    struct Attention {
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        double scale = 0;
        long long rot_dims = 0;           // 0: no rotation
        double rot_base = 0;
        bool rot_scaling = false;         // rot.scaling {factor, low, high, original}
        double sc_factor = 0, sc_low = 0, sc_high = 0, sc_original = 0;
        double softcap = 0;               // 0: none
        long long conv = 0;               // taps of the convolutions over q, k and v; 0: none
    };
    struct Layer {
        std::string type;                 // which mixer: "parallel" or "parallel_2"
        Attention left;
        // "parallel": the state-space side and the two factors
        long long ssm_heads = 0, ssm_vdim = 0, ssm_state = 0, ssm_groups = 1, ssm_conv = 1, ssm_norm_groups = 1;
        double left_scale = 1.0, right_scale = 1.0;
        // "parallel_2": the linear attention side
        long long lin_heads = 0, lin_dim = 0, lin_vdim = 0;
        std::vector<double> lin_decay;
        // feed-forward
        bool has_mlp = false;
        std::string mlp_kind;             // "dense" or "moe"
        long long ff = 0;                 // dense
        long long experts = 0, expert_ff = 0, top = 0, groups = 1, group_keep = 1;
    };
    long long vocab = 0, width = 0;
    double norm_eps = 0, embedding_scale = 1.0;
    long long side_dim = 0;               // token_side.dim; 0: no per-layer token input
    std::vector<Layer> layers;

    static MunisunConfig from_json(const Json &config_json);
    void validate() const;

    std::string architecture() const override { return "Munisun"; }
    Json to_json() const override;
    ModelSpec to_model_spec() const override;
};

void register_munisun();

}  // namespace jb
