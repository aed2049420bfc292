#include "puzutar.h"

#include <cmath>

namespace liyab {
namespace {

int64_t int_in(const Json& obj, const char* key, const std::string& where, int64_t lo, int64_t hi = int64_t{1} << 30) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_int() || v->as_int() < lo || v->as_int() > hi)
        throw invalid_model("missing or invalid {}{} in config.json (got {}, need an integer in [{}, {}])", where, key, v == nullptr ? "nothing" : v->dump(), lo, hi);
    return v->as_int();
}

double number_in(const Json& obj, const char* key, const std::string& where) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_number() || !std::isfinite(v->as_number()))
        throw invalid_model("missing or invalid {}{} in config.json (got {}, need a finite number)", where, key, v == nullptr ? "nothing" : v->dump());
    return v->as_number();
}

const Json& object_in(const Json& obj, const char* key, const std::string& where) {
    const Json* v = obj.find(key);
    if (v == nullptr || !v->is_object()) throw invalid_model("missing or invalid {}{} in config.json (need an object)", where, key);
    return *v;
}

}  // namespace

std::unique_ptr<PuzutarConfig> PuzutarConfig::parse(const Json& raw) {
    auto c = std::make_unique<PuzutarConfig>();
    c->raw = raw;
    c->vocab = int_in(raw, "vocab", "", 1);
    c->width = int_in(raw, "width", "", 1);
    const Json& norm = object_in(raw, "norm", "");
    c->norm_eps = number_in(norm, "eps", "norm.");
    c->norm_groups = norm.contains("groups") ? int_in(norm, "groups", "norm.", 1) : 1;
    if (c->norm_eps < 0 || c->width % c->norm_groups != 0)
        throw invalid_model("invalid norm in config.json: width {} does not split into {} groups, or eps {} is negative", c->width, c->norm_groups, c->norm_eps);
    if (const Json* side = raw.find("token_side"); side != nullptr && !side->is_null()) c->side_dim = int_in(*side, "dim", "token_side.", 1);
    if (const Json* p = raw.find("max_positions"); p != nullptr && !p->is_null()) c->max_positions = int_in(raw, "max_positions", "", 1);
    const Json* layers = raw.find("layers");
    if (layers == nullptr || !layers->is_array() || layers->size() == 0) throw invalid_model("missing or invalid layers in config.json (need a list of layers)");
    for (size_t i = 0; i < layers->size(); ++i) {
        const Json& lj = (*layers)[i];
        const std::string where = std::format("layers[{}].", i);
        if (!lj.is_object()) throw invalid_model("invalid {} in config.json (need an object)", where);
        const std::string type = lj.get_string("type", "");
        if (type != "latent_attention") throw unsupported("{}type '{}' is not supported; supported: latent_attention", where, type);
        const Json& m = object_in(lj, "mixer", where);
        const std::string mw = where + "mixer.";
        Layer l;
        l.heads = int_in(m, "heads", mw, 1, 65535);
        l.dim = int_in(m, "dim", mw, 0);
        l.rot_dim = int_in(m, "rot_dim", mw, 0);
        l.vdim = int_in(m, "vdim", mw, 1);
        l.kv_rank = int_in(m, "kv_rank", mw, 1);
        l.scale = number_in(m, "scale", mw);
        if (const Json* mask = m.find("mask"); mask != nullptr && !mask->is_null()) l.window = int_in(*mask, "size", mw + "mask.", 1);
        l.rot_dims = l.rot_dim;
        if (const Json* rot = m.find("rot"); rot != nullptr && !rot->is_null()) {
            l.rot_base = number_in(*rot, "base", mw + "rot.");
            if (rot->contains("dims")) l.rot_dims = int_in(*rot, "dims", mw + "rot.", 0);
        } else if (l.rot_dim > 0) {
            throw invalid_model("missing {}rot in config.json (the rotated part needs its base)", mw);
        }
        if (l.rot_dims > l.rot_dim || l.rot_dims % 2 != 0 || l.rot_base <= 0)
            throw invalid_model("invalid {}rot in config.json: {} of {} values to rotate, base {}", mw, l.rot_dims, l.rot_dim, l.rot_base);
        if (l.dim + l.rot_dim == 0) throw invalid_model("invalid {}dim and rot_dim in config.json: queries have no values", mw);
        if (const Json* from = m.find("kv_from"); from != nullptr && !from->is_null()) {
            const int64_t j = int_in(m, "kv_from", mw, 0, static_cast<int64_t>(i) - 1);
            const Layer& src = c->layers[static_cast<size_t>(j)];
            if (src.kv_from) throw invalid_model("invalid {}kv_from in config.json: layer {} has no latent of its own", mw, j);
            if (src.kv_rank != l.kv_rank || src.rot_dim != l.rot_dim || src.rot_dims != l.rot_dims || src.rot_base != l.rot_base)
                throw invalid_model("invalid {}kv_from in config.json: layer {} differs in kv_rank, rot_dim or rotation", mw, j);
            l.kv_from = j;
        }
        if (const Json* mlp = lj.find("mlp"); mlp != nullptr && !mlp->is_null()) {
            const std::string kind = mlp->get_string("kind", "");
            if (kind != "dense") throw unsupported("{}mlp.kind '{}' is not supported; supported: dense", where, kind);
            l.ff = int_in(*mlp, "ff", where + "mlp.", 1);
        }
        c->layers.push_back(l);
    }
    return c;
}

ModelSpec PuzutarConfig::model_spec() const {
    ModelSpec m;
    m.architecture = "puzutar";
    m.embedding = {vocab, width, 1.0};
    m.position = {"none", Json::object().set("max_positions", max_positions)};
    const PartSpec norm{"rms_norm", Json::object().set("size", width).set("groups", norm_groups).set("eps", norm_eps)};
    for (size_t i = 0; i < layers.size(); ++i) {
        const Layer& c = layers[i];
        LayerSpec l;
        l.arrangement = "parallel";
        l.slots.push_back({"norm", Role::Norm, norm});
        l.slots.push_back({"shift", Role::Shift, {"lerp_previous", Json::object().set("size", width)}});
        l.slots.push_back({"mixer", Role::Mixer,
                           {"latent_attention", Json::object().set("hidden", width).set("n_head", c.heads).set("dim", c.dim).set("rot_dim", c.rot_dim)
                                                    .set("rot_dims", c.rot_dims).set("rot_base", c.rot_base).set("vdim", c.vdim).set("kv_rank", c.kv_rank)
                                                    .set("window", c.window).set("scale", c.scale).set("eps", norm_eps).set("own_latent", !c.kv_from.has_value())}});
        if (c.ff > 0)
            l.slots.push_back({"feed_forward", Role::FeedForward,
                               {"dense", Json::object().set("hidden", width).set("inner", c.ff).set("activation", "xielu").set("bias", true)}});
        if (side_dim > 0)
            l.slots.push_back({"token_input", Role::TokenInput,
                               {"gated_side", Json::object().set("hidden", width).set("dim", side_dim).set("vocab", vocab).set("eps", norm_eps)}});
        m.layers.push_back(std::move(l));
        m.run_order.push_back({static_cast<int>(i), static_cast<int>(c.kv_from.value_or(static_cast<int64_t>(i)))});
    }
    m.final_norm = norm;
    m.head = {vocab, width, true, false, 1.0, 0.0};
    m.max_positions = max_positions;
    return m;
}

CheckpointMap PuzutarConfig::checkpoint_map() const {
    using K = ParamKind;
    const int64_t L = static_cast<int64_t>(layers.size());
    CheckpointMap m;
    m.push_back({"embedding.weight", CheckpointTensor::one("embed", {vocab, width}, K::Table)});
    m.push_back({"final_norm.weight", CheckpointTensor::one("final.norm", {width}, K::Vector, "none", 1.0, 0.1)});
    for (int64_t i = 0; i < L; ++i) {
        const Layer& c = layers[static_cast<size_t>(i)];
        const std::string p = std::format("layers.{}.", i), f = std::format("l{}.", i);
        const int64_t q_rows = c.heads * (c.dim + c.rot_dim), d_rows = c.kv_rank + c.rot_dim;
        m.push_back({p + "norm.weight", CheckpointTensor::one(f + "norm1", {width}, K::Vector, "none", 1.0, 0.1)});
        m.push_back({p + "shift.weight", CheckpointTensor::one(f + "shift", {width}, K::Vector, "none", 0.5, 0.2)});
        CheckpointTensor proj = CheckpointTensor::one(f + "mix.q", {q_rows, width});
        if (!c.kv_from) {
            // Queries and the row behind the latent come from one product: [q | dkv] joined along the output features.
            proj.sources.push_back({f + "mix.dkv", {d_rows, width}});
            proj.concat_axis = 0;
            m.push_back({p + "mixer.latent_norm.weight", CheckpointTensor::one(f + "mix.dkv.norm", {c.kv_rank}, K::Vector, "none", 1.0, 0.1)});
        }
        m.push_back({p + "mixer.proj.weight", proj});
        m.push_back({p + "mixer.uk.weight", CheckpointTensor::one(f + "mix.uk", {c.heads * c.dim, c.kv_rank}, K::Matrix, "none", 0.0, 0.05)});
        m.push_back({p + "mixer.uv.weight", CheckpointTensor::one(f + "mix.uv", {c.heads * c.vdim, c.kv_rank}, K::Matrix, "none", 0.0, 0.05)});
        m.push_back({p + "mixer.out.weight", CheckpointTensor::one(f + "mix.o", {width, c.heads * c.vdim})});
        if (c.ff > 0) {
            m.push_back({p + "feed_forward.up.weight", CheckpointTensor::one(f + "mlp.up", {c.ff, width})});
            m.push_back({p + "feed_forward.up.bias", CheckpointTensor::one(f + "mlp.up.b", {c.ff}, K::Vector)});
            m.push_back({p + "feed_forward.down.weight", CheckpointTensor::one(f + "mlp.down", {width, c.ff})});
            m.push_back({p + "feed_forward.down.bias", CheckpointTensor::one(f + "mlp.down.b", {width}, K::Vector)});
            m.push_back({p + "feed_forward.act", CheckpointTensor::one(f + "mlp.act", {2}, K::Vector, "none", 0.5, 0.2)});
        }
        if (side_dim > 0) {
            // Every block's slice of the one side table becomes a table of its own.
            CheckpointTensor table = CheckpointTensor::one("side.embed", {vocab, L * side_dim}, K::Table, "none", 0.0, 0.5);
            table.slice_axis = 1;
            table.slice_begin = i * side_dim;
            table.slice_end = (i + 1) * side_dim;
            m.push_back({p + "token_input.table", table});
            m.push_back({p + "token_input.gate.weight", CheckpointTensor::one(f + "side.gate", {side_dim, width})});
            m.push_back({p + "token_input.proj.weight", CheckpointTensor::one(f + "side.proj", {width, side_dim}, K::Matrix, "none", 0.0, 0.1)});
            m.push_back({p + "token_input.norm.weight", CheckpointTensor::one(f + "side.norm", {width}, K::Vector, "none", 0.1, 0.02)});
        }
    }
    return m;
}

void register_puzutar() {
    register_architecture({"puzutar", {"Puzutar", "PuzutarForCausalLM"}, [](const Json& raw) -> std::unique_ptr<ArchitectureConfig> {
                               return PuzutarConfig::parse(raw);
                           }});
}

}  // namespace liyab
