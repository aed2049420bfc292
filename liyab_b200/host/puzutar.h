// Puzutar: a decoder of parallel blocks.  Every block normalises the stream once (RMS norm in groups) and feeds
// both its mixer (after a token shift) and its dense xIELU feed-forward from that; a gated per-token side input
// follows.  The mixer is attention over latent rows with a sliding window; a block may read the latent rows of an
// earlier block instead of making its own.  No position table: positions act through the rotation inside the mixer.
// The head is tied to the embedding.
//
// config.json: {"architecture": "Puzutar", "vocab", "width", "norm": {"eps", "groups"}, "token_side": {"dim"} or absent,
// "layers": [{"type": "latent_attention", "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale",
// "mask": {"size"}, "rot": {"base", "dims"}, "kv_from"?}, "mlp": {"kind": "dense", "ff"} or null}, ...]}.
// Tensors: embed, side.embed, final.norm, and per layer l<i>.norm1, l<i>.shift, l<i>.mix.{q, dkv, dkv.norm, uk, uv, o},
// l<i>.mlp.{up, up.b, down, down.b, act}, l<i>.side.{gate, proj, norm}.
#pragma once

#include <optional>

#include "arch.h"

namespace liyab {

struct PuzutarConfig final : public ArchitectureConfig {
    struct Layer {
        int64_t heads = 0, dim = 0, rot_dim = 0, vdim = 0, kv_rank = 0, window = 0, rot_dims = 0;
        double scale = 1.0, rot_base = 10000.0;
        std::optional<int64_t> kv_from;
        int64_t ff = 0;                 // 0: the block has no feed-forward
    };
    int64_t vocab = 0, width = 0, norm_groups = 1, side_dim = 0;      // side_dim 0: no per-token side input
    double norm_eps = 1e-6;
    int64_t max_positions = int64_t{1} << 17;                         // the design has no limit of its own; the engine's tables need one
    std::vector<Layer> layers;
    Json raw;

    static std::unique_ptr<PuzutarConfig> parse(const Json& raw);
    Json to_json() const override { return raw; }
    ModelSpec model_spec() const override;
    CheckpointMap checkpoint_map() const override;
};

}  // namespace liyab
