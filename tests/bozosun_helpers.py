"""Small Bozosun configurations and model folders with weights the tests choose themselves."""
import json
import os
import struct

import numpy as np


def rot(dims, base=10000.0, scaling=None):
    return {"base": base, "dims": dims, "scaling": scaling}


def attention(heads, kv_heads, dim, vdim, rot_, v_mix=False, scale=None):
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": rot_,
                                           "scale": scale if scale is not None else dim ** -0.5, "v_mix": v_mix}}


def mamba(inner, state, dt_rank, conv):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, limit, experts, top):
    return {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "top": top}}


def config(width, vocab, layers, mult=0.5, eps=1e-5, embed_scale=4.0):
    out = []
    for mixer, mlp in layers:
        layer = dict(mixer)
        layer["mlp"] = mlp
        out.append(layer)
    return {"architecture": "Bozosun", "vocab": vocab, "width": width, "residual_mult": mult, "norm": {"eps": eps},
            "embedding": {"scale": embed_scale}, "layers": out}


YARN = {"factor": 8.0, "original": 64, "fast": 16.0, "slow": 2.0}

# Three configurations that differ in every size: kv groups of 1, 2 and 3 query heads, values as wide as keys and
# narrower and wider, rotation over a whole head and over part of one, with and without scaling, state mixers first
# and last, one and several chosen experts, layers without a feed-forward, value mixing that starts late.
CONFIG_A = config(48, 96, [
    (attention(4, 2, 16, 8, rot(16, 1e4, YARN), v_mix=True), dense(80, 1.25)),
    (mamba(64, 8, 5, 3), moe(24, 0.75, 5, 2)),
    (attention(4, 2, 16, 8, rot(16, 1e4, YARN), v_mix=True), moe(24, 0.75, 5, 2)),
    (mamba(64, 8, 5, 3), dense(80, 1.25)),
], mult=0.4, eps=1e-6, embed_scale=8.0)

CONFIG_B = config(40, 70, [
    (mamba(56, 20, 3, 5), None),
    (attention(6, 2, 24, 24, rot(12, 5e5, None)), moe(16, 2.0, 3, 1)),
    (attention(6, 2, 24, 40, rot(24, 5e5, None), v_mix=True, scale=0.3), dense(72, 0.5)),
    (attention(3, 1, 32, 40, None, v_mix=False), None),
    (attention(6, 2, 24, 40, rot(8, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}), v_mix=True), moe(16, 2.0, 7, 7)),
    (attention(2, 2, 8, 40, rot(8, 100.0, None), v_mix=True), dense(24, 3.0)),
], mult=1.0, eps=1e-3, embed_scale=1.0)

# head size 64 with values as wide: what the tensor-core attention kernels take in bfloat16
CONFIG_C = config(128, 200, [
    (attention(4, 2, 64, 64, rot(64, 5e5, {"factor": 3.0, "original": 128, "fast": 24.0, "slow": 1.5})), dense(256, 1.75)),
    (mamba(256, 16, 8, 4), moe(64, 0.9, 8, 2)),
    (attention(4, 2, 64, 64, rot(32, 5e5, None)), moe(64, 0.9, 8, 2)),
], mult=0.35, eps=1e-6, embed_scale=11.0)


# heads of 128 rotated over their whole width, values as wide, mixing: what the vector rotary kernels and the tcgen05
# prompt attention take
CONFIG_D = config(64, 50, [
    (attention(2, 1, 128, 128, rot(128, 1e5, {"factor": 6.0, "original": 1024, "fast": 20.0, "slow": 2.0}), v_mix=True), dense(48, 2.0)),
    (attention(2, 1, 128, 128, rot(128, 1e5, {"factor": 6.0, "original": 1024, "fast": 20.0, "slow": 2.0}), v_mix=True), None),
], mult=0.7, eps=1e-5, embed_scale=3.0)


def to_bf16_bytes(a):
    """Round float32 to bfloat16 (nearest even) and return the bytes."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    r = ((u >> 16) & 1) + 0x7FFF
    return ((u + r) >> 16).astype("<u2").tobytes()


def bf16_round(a):
    u = np.frombuffer(to_bf16_bytes(a), dtype="<u2").astype(np.uint32) << 16
    return u.view(np.float32).reshape(np.shape(a))


def write_safetensors(path, tensors, dtype="F32"):
    """{name: float array} -> a safetensors file (8-byte header length, JSON header, data)."""
    header, blobs, at = {}, [], 0
    for name, a in tensors.items():
        a = np.asarray(a, dtype=np.float32)
        raw = a.astype("<f4").tobytes() if dtype == "F32" else to_bf16_bytes(a)
        header[name] = {"dtype": dtype, "shape": list(a.shape), "data_offsets": [at, at + len(raw)]}
        blobs.append(raw)
        at += len(raw)
    text = json.dumps(header).encode()
    text += b" " * (-len(text) % 8)
    with open(path, "wb") as f:
        f.write(struct.pack("<Q", len(text)))
        f.write(text)
        for b in blobs:
            f.write(b)


def draw_weights(cfg, seed, std=0.3):
    """Weights for every tensor the framework says the configuration reads: matrices N(0, std / sqrt(fan_in)) scaled
    up so that activations stay of order one through the norms, norm weights around 1, biases and the rest small but
    not negligible, the mixing factors well inside (0, 1)."""
    from purhie_b200.weights import expected_tensors
    rng = np.random.default_rng(seed)
    out = {}
    for name, spec in expected_tensors(cfg).items():
        shape = tuple(spec.shape)
        if name.endswith("vmix"):
            a = rng.uniform(0.2, 0.8, shape)
        elif name.endswith("A_log"):
            a = rng.uniform(-1.5, 1.0, shape)
        elif name.endswith("dt.b"):
            a = rng.uniform(-3.0, 0.5, shape)
        elif name.endswith(".b"):
            a = rng.normal(0.0, 0.2, shape)
        elif spec.init == "scale":
            a = rng.uniform(0.5, 1.5, shape)
        elif name.endswith("mix.conv"):
            a = rng.normal(0.0, 0.5, shape)
        elif len(shape) == 2:
            a = rng.normal(0.0, std * 3.0 / np.sqrt(shape[1]), shape)
        else:
            a = rng.normal(0.0, std, shape)
        out[name] = bf16_round(a.astype(np.float32))          # representable in either storage
    return out


def steady_routing(cfg, weights, seed=0):
    """The same weights with router biases that decide which experts are chosen, a different set in every layer: the
    chosen `top` lie 60 above the rest and within 1 of each other, so that their weights still follow the token while a
    rounding of the router's input cannot change the set (what a reduced-precision run needs to be comparable at all)."""
    rng = np.random.default_rng(seed)
    out = dict(weights)
    for i, layer in enumerate(cfg["layers"]):
        mlp = layer.get("mlp")
        if not mlp or mlp["kind"] != "moe":
            continue
        experts, top = mlp["router"]["experts"], mlp["router"]["top"]
        bias = np.full(experts, -30.0, dtype=np.float32)
        chosen = rng.permutation(experts)[:top]
        bias[chosen] = 30.0 + rng.uniform(0.0, 1.0, top).astype(np.float32)
        out[f"l{i}.mlp.router.b"] = bf16_round(bias)
    return out


def make_folder(folder, cfg, weights, dtype="F32"):
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights, dtype)
    return str(folder)


def tokens(n, vocab, seed):
    return np.random.default_rng(seed).integers(0, vocab, n).tolist()
