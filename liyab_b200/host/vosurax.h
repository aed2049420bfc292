// Vosurax: a decoder of pre-norm blocks whose mixers keep a memory.  A block's mixer is either a retention (a matrix
// memory per head with a fixed decay and rotated queries and keys) or two mixers side by side on the same input, attention
// in chunks with normalised queries and keys and an output gate beside a gated matrix memory, each branch's output over
// its own root mean square and the two halved.  The feed-forward is dense (GELU), a mixture of small gated experts with a
// shared one, or absent.  A stretch of blocks may run several times over the same weights, every pass with caches and
// memories of its own and a learned vector added to the stream before it.  Norm gains are stored around zero.  No
// position table; the head is a matrix of its own.
//
// config.json: {"architecture": "Vosurax", "vocab", "width", "norm": {"eps"}, "loop": {"start", "stop", "times"} or absent,
// "layers": [{"type": "retention", "mixer": {"heads", "dim", "vdim", "decay": [..], "rot": {"base", "dims"}}, "mlp": ..} |
// {"type": "parallel", "mixer": {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"}}, "right": {"heads",
// "dim", "vdim", "gate_cap"}}, "mlp": ..}], "mlp": {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"}, "router":
// {"experts", "top"}, "shared": {"ff"} or absent} | null}.
// Tensors: embed, head, final.norm, loop.step, and per layer l<i>.norm1, l<i>.norm2, l<i>.mix.*, l<i>.mlp.*.
#pragma once

#include <optional>

#include "arch.h"

namespace liyab {

struct VosuraxConfig final : public ArchitectureConfig {
    struct Layer {
        bool parallel = false;
        // retention, or the right branch of a parallel mixer
        int64_t heads = 0, dim = 0, vdim = 0, rot_dims = 0;
        double rot_base = 10000.0, gate_cap = 0.0;
        std::vector<double> decay;
        // the left branch of a parallel mixer
        int64_t a_heads = 0, a_kv_heads = 0, a_dim = 0, a_vdim = 0, a_chunk = 0;
        double a_scale = 1.0;
        // feed-forward: ff > 0 dense; experts > 0 routed; neither: none
        int64_t ff = 0, experts = 0, top = 0, expert_ff = 0, shared_ff = 0;
    };
    int64_t vocab = 0, width = 0;
    double norm_eps = 1e-6;
    int64_t loop_start = 0, loop_stop = 0, loop_times = 0;            // times 0: no stretch runs twice
    int64_t max_positions = int64_t{1} << 17;                         // the design has no limit of its own; the engine's tables need one
    std::vector<Layer> layers;
    Json raw;

    static std::unique_ptr<VosuraxConfig> parse(const Json& raw);
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
    CheckpointMap checkpoint_map() const override;
    std::vector<std::string> ignored_tensors() const override;
};

}  // namespace liyab
