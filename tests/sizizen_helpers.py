"""Small Sizizen configurations and model folders with weights the tests choose themselves."""
import numpy as np

from bozosun_helpers import bf16_round, make_folder, tokens, write_safetensors  # noqa: F401  (re-exported)


def left(heads, kv_heads, dim, vdim, rot_dims, mask, base=10000.0, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"base": base, "dims": rot_dims},
            "mask": {"size": mask}, "scale": scale if scale is not None else dim ** -0.5}


def right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(ff, experts, top, groups, keep, shared):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top, "groups": {"count": groups, "keep": keep}},
            "shared": {"ff": shared}}


def config(width, vocab, layers, eps=1e-5):
    return {"architecture": "Sizizen", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "layers": [{"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp} for l, r, mlp in layers]}


# Configurations that differ in every size: groups of 1, 2 and 3 query heads per key head; values narrower than, as wide
# as and wider than keys on both sides; rotation over a whole head, part of one, a single pair; masks of 1, 5, 12, 16
# (a page) and longer than any prompt here, different from layer to layer; decays with tau 1 and 16; ranks 3 to 8;
# routers with and without real groups, top 1 and top = all kept experts; layers without a feed-forward.
CONFIG_A = config(48, 80, [
    (left(4, 2, 16, 8, 8, 12, scale=0.3), right(2, 8, 16, 4.0, 6), dense(64)),
    (left(3, 3, 8, 24, 8, 5, base=500.0), right(3, 24, 8, 1.0, 4), moe(16, 6, 2, 3, 2, 24)),
    (left(6, 2, 8, 8, 2, 1000), right(1, 16, 32, 16.0, 3), None),
    (left(2, 1, 24, 16, 12, 16, base=1e6, scale=0.15), right(4, 8, 8, 2.0, 8), moe(8, 8, 3, 1, 1, 8)),
], eps=1e-6)

CONFIG_B = config(40, 70, [
    (left(2, 2, 20, 12, 4, 1), right(5, 4, 12, 8.0, 5), moe(24, 4, 1, 4, 2, 16)),
    (left(5, 1, 8, 16, 6, 33, base=77.0, scale=0.5), right(2, 40, 4, 3.0, 7), dense(56)),
    (left(1, 1, 32, 40, 32, 9), right(2, 12, 20, 1.5, 2), moe(12, 9, 6, 3, 2, 40)),
], eps=1e-3)

# wider layers, stored in bfloat16: keys of 64 and 128 with values as wide or not, a state of 64 x 128 per head
CONFIG_C = config(128, 200, [
    (left(4, 2, 64, 64, 32, 48, base=5e5), right(2, 64, 128, 16.0, 16), dense(256)),
    (left(2, 1, 128, 128, 64, 100, base=5e5), right(4, 32, 32, 8.0, 8), moe(64, 8, 2, 4, 2, 128)),
    (left(4, 4, 32, 16, 32, 64), right(2, 128, 64, 4.0, 24), moe(32, 4, 2, 2, 1, 64)),
], eps=1e-6)


def draw_weights(cfg, seed, std=0.3):
    """Weights for every tensor the framework says the configuration reads: matrices N(0, 3 std / sqrt(fan_in)) so that
    activations stay of order one, norm weights around 1, biases small but not negligible, decay biases spread so that
    some channels forget within a few tokens and others keep for hundreds, corrections of the size of a score."""
    from purhie_b200.weights import expected_tensors
    rng = np.random.default_rng(seed)
    out = {}
    for name, spec in expected_tensors(cfg).items():
        shape = tuple(spec.shape)
        if name.endswith("a2.b"):
            a = rng.uniform(-2.0, 6.0, shape)
        elif name.endswith("correction"):
            a = rng.normal(0.0, 0.4, shape)
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.2, shape)
        elif spec.init == "scale":
            a = rng.uniform(0.5, 1.5, shape)
        elif len(shape) == 2:
            a = rng.normal(0.0, std * 3.0 / np.sqrt(shape[1]), shape)
        else:
            a = rng.normal(0.0, std, shape)
        out[name] = bf16_round(a.astype(np.float32))          # representable in either storage
    # The right mixer's first tokens give o = v (k . q), and the head norm behind it keeps only the sign of k . q: with q
    # and k drawn independently that product is a difference of like terms whose sign a bfloat16 rounding can turn.  Real
    # models do not live there; q is drawn near k so that a token's own term is positive and leads.
    for name in list(out):
        if name.endswith("mix.right.q"):
            k = out[name[:-1] + "k"]
            out[name] = bf16_round((k + 0.5 * out[name]).astype(np.float32))
    return out


def steady_choice(cfg, weights, seed=0):
    """The same weights with corrections that decide which experts are chosen, a different set in every layer: the chosen
    `top` lie inside `keep` groups and 20 above all others, so that a rounding of the router's input cannot change the
    set, while the weights (the scores without the correction) still follow the token."""
    rng = np.random.default_rng(seed)
    out = dict(weights)
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        r = mlp["router"]
        experts, top, groups, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
        per = experts // groups
        kept = rng.permutation(groups)[:keep]
        pool = np.concatenate([np.arange(g * per, (g + 1) * per) for g in kept])
        chosen = rng.permutation(pool)[:top]
        corr = np.full(experts, -10.0, dtype=np.float32)
        corr[chosen] = 10.0 + 2.0 * np.arange(top, dtype=np.float32)
        out[f"l{i}.mlp.correction"] = bf16_round(corr)
    return out
