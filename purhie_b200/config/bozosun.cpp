// The Bozosun design: a decoder of layers that each pair a mixer (grouped-query attention or a selective state-space
// mixer) with a gated feed-forward (one, a routed mixture of them, or none), every part between a layer norm in
// front and a layer norm behind, the normed output added with a factor.
//
// config.json keys, all read here and nowhere else:
//   architecture ("Bozosun"), vocab, width, residual_mult, norm.eps, embedding.scale,
//   layers[i].type ("attention" | "mamba1"), layers[i].mixer, layers[i].mlp (null: the layer has no feed-forward);
//   an attention mixer: heads, kv_heads, dim, vdim, scale, v_mix, rot {base, dims, scaling {factor, original, fast,
//     slow} or null};
//   a mamba1 mixer: inner, state, dt_rank, conv;
//   mlp.kind "dense": ff, limit;  mlp.kind "moe": expert {ff, limit}, router {experts, top};
//   max_position (optional): the longest sequence the rotary table is made for.
// Tensor names: embed, head, final.norm(.b), and per layer i: l<i>.norm1 / norm1b / norm2 / norm2b (each with .b),
// l<i>.mix.{q, k, v, o, vmix} or l<i>.mix.{in, conv, conv.b, x, dt, dt.b, A_log, D, o}, l<i>.mlp.{gate, up, down} or
// l<i>.mlp.{router, router.b, e<j>.gate, e<j>.up, e<j>.down}.
//
// What the design fixes and the code therefore states: the gate of every feed-forward is g' sigmoid(1.702 g') (u' + 1)
// with g' = min(g, limit) and u' = clamp(u, -limit, limit); rotary pairs are interleaved (2i, 2i + 1); attention sees
// every earlier position; the values of every layer with v_mix but the first such layer are blended with that first
// layer's values of the same token by the layer's scalar `vmix`.
#include "config.h"

namespace qe {

namespace {
constexpr double kGateAlpha = 1.702, kUpShift = 1.0;
constexpr long long kDefaultMaxPosition = 65536;

Json names(std::initializer_list<std::pair<const char*, std::string>> list) {
    Json n = Json::object();
    for (const auto& kv : list) n.set(kv.first, kv.second);
    return n;
}
const Json& object_at(const Json& d, const std::string& key, const std::string& where) {
    const Json* v = d.find(key);
    if (!v || !v->is_object()) throw ConfigError("config.json: " + where + "'" + key + "' must be an object");
    return *v;
}
}  // namespace

class BozosunConfig : public ModelConfig {
public:
    Json source;                        // config.json as read (checked)
    long long vocab = 0, width = 0, max_position = kDefaultMaxPosition;
    double residual_mult = 1.0, eps = 0.0, embedding_scale = 1.0;

    static std::unique_ptr<ModelConfig> read(const Json& d) {
        std::unique_ptr<BozosunConfig> c(new BozosunConfig());
        c->architecture = "Bozosun";
        c->source = d;
        c->vocab = take_int(d, "vocab");
        c->width = take_int(d, "width");
        c->residual_mult = take_float(d, "residual_mult", 1.0);
        c->eps = take_float(object_at(d, "norm", ""), "eps");
        c->embedding_scale = has_value(d, "embedding") ? take_float(object_at(d, "embedding", ""), "scale", 1.0) : 1.0;
        c->max_position = take_int(d, "max_position", kDefaultMaxPosition, 1);
        const Json* layers = d.find("layers");
        if (!layers || !layers->is_array() || layers->size() == 0) throw ConfigError("config.json: 'layers' must be a non-empty list");
        long long mix_heads = -1, mix_vdim = -1;
        for (size_t i = 0; i < layers->size(); i++) {
            const Json& l = (*layers)[i];
            const std::string where = "layers[" + std::to_string(i) + "].";
            if (!l.is_object()) throw ConfigError("config.json: " + where + " must be an object");
            const std::string type = l.get_string("type", "");
            const Json& m = object_at(l, "mixer", where);
            if (type == "attention") {
                const long long heads = take_int(m, "heads"), kv = take_int(m, "kv_heads"), dim = take_int(m, "dim"), vdim = take_int(m, "vdim");
                take_float(m, "scale");
                if (heads % kv) throw ConfigError("config.json: " + where + "mixer: " + std::to_string(heads) + " heads are not a multiple of " + std::to_string(kv) + " kv_heads");
                if (has_value(m, "rot")) {
                    const Json& rot = object_at(m, "rot", where + "mixer.");
                    const long long dims = take_int(rot, "dims", 2);
                    if (dims % 2 || dims > dim) throw ConfigError("config.json: " + where + "mixer.rot.dims must be even and at most dim");
                    if (!(take_float(rot, "base") > 1.0)) throw ConfigError("config.json: " + where + "mixer.rot.base must be above 1");
                    if (has_value(rot, "scaling")) {
                        const Json& sc = object_at(rot, "scaling", where + "mixer.rot.");
                        for (const char* key : {"factor", "original", "fast", "slow"})
                            if (!(take_float(sc, key) > 0)) throw ConfigError("config.json: " + where + "mixer.rot.scaling." + key + " must be positive");
                    }
                }
                if (take_bool(m, "v_mix", false)) {
                    if (mix_heads >= 0 && (mix_heads != kv || mix_vdim != vdim))
                        throw ConfigError("config.json: " + where + "mixer: layers with v_mix must agree in kv_heads and vdim");
                    mix_heads = kv; mix_vdim = vdim;
                }
            } else if (type == "mamba1") {
                take_int(m, "inner"); take_int(m, "state"); take_int(m, "dt_rank"); take_int(m, "conv");
            } else {
                throw ConfigError("config.json: " + where + "type '" + type + "' is not known (attention, mamba1)");
            }
            if (has_value(l, "mlp")) {
                const Json& f = object_at(l, "mlp", where);
                const std::string kind = f.get_string("kind", "");
                if (kind == "dense") {
                    take_int(f, "ff");
                    if (!(take_float(f, "limit") > 0)) throw ConfigError("config.json: " + where + "mlp.limit must be positive");
                } else if (kind == "moe") {
                    const Json& e = object_at(f, "expert", where + "mlp.");
                    const Json& r = object_at(f, "router", where + "mlp.");
                    take_int(e, "ff");
                    if (!(take_float(e, "limit") > 0)) throw ConfigError("config.json: " + where + "mlp.expert.limit must be positive");
                    if (take_int(r, "top") > take_int(r, "experts")) throw ConfigError("config.json: " + where + "mlp.router.top exceeds experts");
                } else {
                    throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not known (dense, moe)");
                }
            }
        }
        return std::unique_ptr<ModelConfig>(c.release());
    }

    Json to_json() const override {
        Json d = source;
        d.set("architecture", "Bozosun");
        return d;
    }

    ModelSpec build_spec() const override {
        auto norm = [&](const std::string& name) {
            Json p = Json::object();
            p.set("size", width);
            p.set("eps", eps);
            p.set("names", names({{"weight", name}, {"bias", name + ".b"}}));
            return PartSpec("layernorm", p);
        };
        auto gate = [&](double limit) {
            Json a = Json::object();
            a.set("kind", "clamped_swish");
            a.set("alpha", kGateAlpha);
            a.set("limit", limit);
            a.set("shift", kUpShift);
            return a;
        };
        ModelSpec spec;
        spec.hidden_size = width;
        spec.vocab_size = vocab;
        spec.max_position = max_position;
        const Json& layers = source.at("layers");
        bool mixing_started = false;
        for (size_t i = 0; i < layers.size(); i++) {
            const Json& l = layers[i];
            const Json& m = l.at("mixer");
            const std::string p = "l" + std::to_string(i) + ".";
            LayerSpec layer;
            layer.arrangement = "sandwich_norm";
            layer.params.set("residual_factor", residual_mult);
            layer.parts.push_back({"mixer_norm", norm(p + "norm1")});
            if (l.at("type").as_string() == "attention") {
                Json a = Json::object();
                a.set("hidden_size", width);
                a.set("num_heads", m.at("heads"));
                a.set("num_kv_heads", m.at("kv_heads"));
                a.set("head_dim", m.at("dim"));
                a.set("value_dim", m.at("vdim"));
                a.set("qk_norm_eps", Json());
                a.set("bias", false);
                a.set("window", Json());
                a.set("scale", m.at("scale"));
                Json n = names({{"q_proj", p + "mix.q"}, {"k_proj", p + "mix.k"}, {"v_proj", p + "mix.v"}, {"o_proj", p + "mix.o"}});
                if (take_bool(m, "v_mix", false)) {
                    a.set("value_mix", mixing_started ? "blend" : "first");
                    n.set("value_mix_factor", p + "mix.vmix");
                    mixing_started = true;
                }
                if (has_value(m, "rot")) {
                    const Json& rot = m.at("rot");
                    Json pos = Json::object();
                    pos.set("theta", rot.at("base"));
                    pos.set("n_rot", rot.at("dims"));
                    pos.set("max_position", max_position);
                    pos.set("pairing", "interleaved");
                    if (has_value(rot, "scaling")) {
                        Json sc = rot.at("scaling");
                        sc.set("kind", "yarn");
                        pos.set("scaling", sc);
                    }
                    a.set("position", PartSpec("rope_neox", pos).to_json());
                } else {
                    a.set("position", Json());
                }
                a.set("names", n);
                layer.parts.push_back({"mixer", PartSpec("attention", a)});
            } else {
                Json s = Json::object();
                s.set("hidden_size", width);
                s.set("inner", m.at("inner"));
                s.set("state", m.at("state"));
                s.set("dt_rank", m.at("dt_rank"));
                s.set("conv", m.at("conv"));
                s.set("names", names({{"in_proj", p + "mix.in"}, {"conv_weight", p + "mix.conv"}, {"conv_bias", p + "mix.conv.b"},
                                      {"x_proj", p + "mix.x"}, {"dt_proj", p + "mix.dt"}, {"dt_bias", p + "mix.dt.b"},
                                      {"a_log", p + "mix.A_log"}, {"d", p + "mix.D"}, {"out_proj", p + "mix.o"}}));
                layer.parts.push_back({"mixer", PartSpec("mamba1", s)});
            }
            layer.parts.push_back({"mixer_post_norm", norm(p + "norm1b")});
            if (has_value(l, "mlp")) {
                const Json& f = l.at("mlp");
                layer.parts.push_back({"feed_forward_norm", norm(p + "norm2")});
                if (f.at("kind").as_string() == "dense") {
                    Json g = Json::object();
                    g.set("hidden_size", width);
                    g.set("intermediate_size", f.at("ff"));
                    g.set("activation", gate(f.at("limit").as_double()));
                    g.set("names", names({{"gate_proj", p + "mlp.gate"}, {"up_proj", p + "mlp.up"}, {"down_proj", p + "mlp.down"}}));
                    layer.parts.push_back({"feed_forward", PartSpec("swiglu", g)});
                } else {
                    const long long experts = f.at("router").at("experts").as_int();
                    Json g = Json::object();
                    g.set("hidden_size", width);
                    g.set("intermediate_size", f.at("expert").at("ff"));
                    g.set("experts", experts);
                    g.set("top", f.at("router").at("top"));
                    g.set("activation", gate(f.at("expert").at("limit").as_double()));
                    g.set("names", names({{"router", p + "mlp.router"}, {"router_bias", p + "mlp.router.b"}}));
                    Json list = Json::array();
                    for (long long e = 0; e < experts; e++) {
                        const std::string ep = p + "mlp.e" + std::to_string(e) + ".";
                        list.push(names({{"gate_proj", ep + "gate"}, {"up_proj", ep + "up"}, {"down_proj", ep + "down"}}));
                    }
                    g.set("expert_names", list);
                    layer.parts.push_back({"feed_forward", PartSpec("routed_glu", g)});
                }
                layer.parts.push_back({"feed_forward_post_norm", norm(p + "norm2b")});
            }
            spec.layers.push_back(std::move(layer));
            spec.schedule.push_back(LayerCall{(int)i, -1});
        }
        Json e = Json::object();
        e.set("vocab_size", vocab);
        e.set("hidden_size", width);
        e.set("scale", embedding_scale);
        e.set("names", names({{"weight", "embed"}}));
        spec.embedding = PartSpec("embedding", e);
        Json h = Json::object();
        h.set("hidden_size", width);
        h.set("vocab_size", vocab);
        h.set("names", names({{"weight", "head"}}));
        spec.head = PartSpec("lm_head", h);
        spec.final_norm = norm("final.norm");
        spec.validate();
        return spec;
    }
};

void register_bozosun_architecture() { register_architecture("Bozosun", BozosunConfig::read); }

}  // namespace qe
