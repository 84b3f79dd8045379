// The Sizizen design: a decoder whose layers norm what a part gives instead of what it reads, whose mixer is two
// mixers side by side (softmax attention under a block mask, and gated linear attention), and whose feed-forward is
// a gated unit or a mixture of ungated experts with a shared one.
//
//     x <- x + LN(mixer(x));  x <- x + LN(ff(x))          LN: layer norm with a weight and no bias
//     mixer(h) = (rms(left(h); w_l) + rms(right(h); w_r)) / 2
//
// config.json keys, all read here and nowhere else:
//   architecture ("Sizizen"), vocab, width, norm.eps, layers[i].type ("parallel"), layers[i].mixer {left, right},
//   layers[i].mlp (null: the layer has no feed-forward);
//   mixer.left: heads, kv_heads, dim, vdim, scale, rot {base, dims}, mask {size};
//   mixer.right: heads, dim, vdim, tau, rank (optional: the inner size of the decay's two products; without it the
//     stored matrices give it, and only a folder can be loaded);
//   mlp.kind "dense": ff;  mlp.kind "moe": expert {ff}, router {experts, top, groups {count, keep}}, shared {ff};
//   max_position (optional): the longest sequence the rotary table is made for.
// Tensor names: embed, head, final.norm, and per layer i: l<i>.norm1, l<i>.norm2,
// l<i>.mix.left.{q, q.b, k, k.b, v, v.b, q.norm, k.norm, o, out}, l<i>.mix.right.{q, k, v, g, o, norm, a1, a2, a2.b, out},
// l<i>.mlp.{gate, up, down} or l<i>.mlp.{router, correction, e<j>.up, e<j>.down, shared.up, shared.down}.
//
// What the design fixes and the code therefore states: the left mixer's q, k and v have biases, q and k are
// RMS-normed per head before the rotation, rotary pairs are (i, i + dims/2); the two sides are averaged (factor 1/2);
// the dense unit's gate is silu; experts and the shared expert are W_down relu(W_up h)^2; router scores are
// sigmoids, the choice adds the correction, the weights do not and are not renormalised; a group ranks by its two
// largest choice scores.
#include "config.h"

namespace qe {

namespace {
constexpr long long kDefaultMaxPosition = 65536;
constexpr double kSideFactor = 0.5;
const char* const kExpertActivation = "relu2";

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

class SizizenConfig : public ModelConfig {
public:
    Json source;                        // config.json as read (checked)
    long long vocab = 0, width = 0, max_position = kDefaultMaxPosition;
    double eps = 0.0;

    static std::unique_ptr<ModelConfig> read(const Json& d) {
        std::unique_ptr<SizizenConfig> c(new SizizenConfig());
        c->architecture = "Sizizen";
        c->source = d;
        c->vocab = take_int(d, "vocab");
        c->width = take_int(d, "width");
        c->eps = take_float(object_at(d, "norm", ""), "eps");
        c->max_position = take_int(d, "max_position", kDefaultMaxPosition, 1);
        const Json* layers = d.find("layers");
        if (!layers || !layers->is_array() || layers->size() == 0) throw ConfigError("config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < layers->size(); i++) {
            const Json& l = (*layers)[i];
            const std::string where = "layers[" + std::to_string(i) + "].";
            if (!l.is_object()) throw ConfigError("config.json: " + where + " must be an object");
            const std::string type = l.get_string("type", "");
            if (type != "parallel") throw ConfigError("config.json: " + where + "type '" + type + "' is not known (parallel)");
            const Json& m = object_at(l, "mixer", where);
            const Json& left = object_at(m, "left", where + "mixer.");
            const Json& right = object_at(m, "right", where + "mixer.");
            const long long heads = take_int(left, "heads"), kv = take_int(left, "kv_heads"), dim = take_int(left, "dim");
            take_int(left, "vdim");
            take_float(left, "scale");
            if (heads % kv)
                throw ConfigError("config.json: " + where + "mixer.left: " + std::to_string(heads) + " heads are not a multiple of " + std::to_string(kv) + " kv_heads");
            const Json& rot = object_at(left, "rot", where + "mixer.left.");
            const long long dims = take_int(rot, "dims", 0);          // 0: no dimension is rotated
            if (dims % 2 || dims > dim) throw ConfigError("config.json: " + where + "mixer.left.rot.dims must be even and at most dim");
            if (!(take_float(rot, "base") > 0)) throw ConfigError("config.json: " + where + "mixer.left.rot.base must be positive");
            take_int(object_at(left, "mask", where + "mixer.left."), "size");
            take_int(right, "heads"); take_int(right, "dim"); take_int(right, "vdim");
            take_int(right, "rank", 1, 1);
            if (!(take_float(right, "tau") > 0)) throw ConfigError("config.json: " + where + "mixer.right.tau must be positive");
            if (has_value(l, "mlp")) {
                const Json& f = object_at(l, "mlp", where);
                const std::string kind = f.get_string("kind", "");
                if (kind == "dense") {
                    take_int(f, "ff");
                } else if (kind == "moe") {
                    take_int(object_at(f, "expert", where + "mlp."), "ff");
                    const Json& r = object_at(f, "router", where + "mlp.");
                    const long long experts = take_int(r, "experts"), top = take_int(r, "top");
                    long long count = 1, keep = 1;
                    if (has_value(r, "groups")) {
                        const Json& g = object_at(r, "groups", where + "mlp.router.");
                        count = take_int(g, "count");
                        keep = take_int(g, "keep");
                    }
                    if (top > experts || experts % count || keep > count || keep * (experts / count) < top)
                        throw ConfigError("config.json: " + where + "mlp.router: top " + std::to_string(top) + " of " + std::to_string(experts) +
                                          " experts in " + std::to_string(keep) + " of " + std::to_string(count) + " groups cannot be chosen");
                    if (has_value(f, "shared")) take_int(object_at(f, "shared", where + "mlp."), "ff");
                } else {
                    throw ConfigError("config.json: " + where + "mlp.kind '" + kind + "' is not known (dense, moe)");
                }
            }
        }
        return std::unique_ptr<ModelConfig>(c.release());
    }

    Json to_json() const override {
        Json d = source;
        d.set("architecture", "Sizizen");
        return d;
    }

    ModelSpec build_spec() const override {
        auto norm = [&](const std::string& name) {
            Json p = Json::object();
            p.set("size", width);
            p.set("eps", eps);
            p.set("names", names({{"weight", name}}));
            return PartSpec("layernorm", p);
        };
        auto none = [&]() {
            Json p = Json::object();
            p.set("size", width);
            return PartSpec("none", p);
        };
        auto plain_mlp = [&](long long ff, const std::string& prefix) {
            Json g = Json::object();
            g.set("hidden_size", width);
            g.set("intermediate_size", ff);
            g.set("activation", kExpertActivation);
            g.set("names", names({{"up_proj", prefix + "up"}, {"down_proj", prefix + "down"}}));
            return PartSpec("mlp", g);
        };
        ModelSpec spec;
        spec.hidden_size = width;
        spec.vocab_size = vocab;
        spec.max_position = max_position;
        const Json& layers = source.at("layers");
        for (size_t i = 0; i < layers.size(); i++) {
            const Json& l = layers[i];
            const Json& left = l.at("mixer").at("left");
            const Json& right = l.at("mixer").at("right");
            const std::string p = "l" + std::to_string(i) + ".";
            LayerSpec layer;
            layer.arrangement = "sandwich_norm";
            layer.params.set("residual_factor", 1.0);
            layer.parts.push_back({"mixer_norm", none()});

            Json a = Json::object();
            a.set("hidden_size", width);
            a.set("num_heads", left.at("heads"));
            a.set("num_kv_heads", left.at("kv_heads"));
            a.set("head_dim", left.at("dim"));
            a.set("value_dim", left.at("vdim"));
            a.set("qk_norm_eps", eps);
            a.set("bias", true);
            a.set("window", Json());
            a.set("chunk", left.at("mask").at("size"));
            a.set("scale", left.at("scale"));
            if (left.at("rot").at("dims").as_int() > 0) {
                Json pos = Json::object();
                pos.set("theta", left.at("rot").at("base"));
                pos.set("n_rot", left.at("rot").at("dims"));
                pos.set("max_position", max_position);
                pos.set("pairing", "half");
                a.set("position", PartSpec("rope_neox", pos).to_json());
            } else {
                a.set("position", Json());
            }
            const std::string lp = p + "mix.left.";
            a.set("names", names({{"q_proj", lp + "q"}, {"k_proj", lp + "k"}, {"v_proj", lp + "v"}, {"o_proj", lp + "o"},
                                  {"q_bias", lp + "q.b"}, {"k_bias", lp + "k.b"}, {"v_bias", lp + "v.b"},
                                  {"q_norm", lp + "q.norm"}, {"k_norm", lp + "k.norm"}}));

            Json r = Json::object();
            r.set("hidden_size", width);
            r.set("num_heads", right.at("heads"));
            r.set("head_dim", right.at("dim"));
            r.set("value_dim", right.at("vdim"));
            r.set("tau", right.at("tau"));
            r.set("norm_eps", eps);
            const std::string rp = p + "mix.right.";
            r.set("decay_rank", has_value(right, "rank") ? right.at("rank") : Json());
            r.set("names", names({{"q_proj", rp + "q"}, {"k_proj", rp + "k"}, {"v_proj", rp + "v"}, {"g_proj", rp + "g"}, {"o_proj", rp + "o"},
                                  {"norm", rp + "norm"}, {"decay_down", rp + "a1"}, {"decay_up", rp + "a2"}, {"decay_bias", rp + "a2.b"}}));

            Json both = Json::object();
            both.set("hidden_size", width);
            both.set("eps", eps);
            both.set("factor", kSideFactor);
            both.set("left", PartSpec("attention", a).to_json());
            both.set("right", PartSpec("gated_linear_attention", r).to_json());
            both.set("names", names({{"left_norm", p + "mix.left.out"}, {"right_norm", p + "mix.right.out"}}));
            layer.parts.push_back({"mixer", PartSpec("side_by_side", both)});
            layer.parts.push_back({"mixer_post_norm", norm(p + "norm1")});

            if (has_value(l, "mlp")) {
                const Json& f = l.at("mlp");
                layer.parts.push_back({"feed_forward_norm", none()});
                if (f.at("kind").as_string() == "dense") {
                    Json g = Json::object();
                    g.set("hidden_size", width);
                    g.set("intermediate_size", f.at("ff"));
                    g.set("names", names({{"gate_proj", p + "mlp.gate"}, {"up_proj", p + "mlp.up"}, {"down_proj", p + "mlp.down"}}));
                    layer.parts.push_back({"feed_forward", PartSpec("swiglu", g)});
                } else {
                    const Json& router = f.at("router");
                    const long long experts = router.at("experts").as_int();
                    Json g = Json::object();
                    g.set("hidden_size", width);
                    g.set("intermediate_size", f.at("expert").at("ff"));
                    g.set("experts", experts);
                    g.set("top", router.at("top"));
                    g.set("gated", false);
                    g.set("activation", kExpertActivation);
                    Json scoring = Json::object();
                    scoring.set("kind", "sigmoid");
                    scoring.set("groups", has_value(router, "groups") ? router.at("groups").at("count") : Json(1));
                    scoring.set("keep", has_value(router, "groups") ? router.at("groups").at("keep") : Json(1));
                    g.set("scoring", scoring);
                    g.set("names", names({{"router", p + "mlp.router"}, {"correction", p + "mlp.correction"}}));
                    Json list = Json::array();
                    for (long long e = 0; e < experts; e++) {
                        const std::string ep = p + "mlp.e" + std::to_string(e) + ".";
                        list.push(names({{"up_proj", ep + "up"}, {"down_proj", ep + "down"}}));
                    }
                    g.set("expert_names", list);
                    if (has_value(f, "shared")) g.set("shared", plain_mlp(f.at("shared").at("ff").as_int(), p + "mlp.shared.").to_json());
                    layer.parts.push_back({"feed_forward", PartSpec("routed_glu", g)});
                }
                layer.parts.push_back({"feed_forward_post_norm", norm(p + "norm2")});
            }
            spec.layers.push_back(std::move(layer));
            spec.schedule.push_back(LayerCall{(int)i, -1});
        }
        Json e = Json::object();
        e.set("vocab_size", vocab);
        e.set("hidden_size", width);
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

void register_sizizen_architecture() { register_architecture("Sizizen", SizizenConfig::read); }

}  // namespace qe
