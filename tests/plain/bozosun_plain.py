"""A plain, slow Bozosun forward pass: one whole sequence from position 0, no cache, one function per mechanism.

It shares no code with ``purhie_b200``: it reads ``config.json`` with ``json`` and the weight file by its byte
layout, and states every equation directly.  Everything runs in float64.

The design in short (names of config.json in quotes):

* x0 = embed[token] * "embedding.scale".
* A layer: x <- x + m * LN1b(mixer(LN1(x))), then, if it has a feed-forward, x <- x + m * LN2b(ff(LN2(x))), with
  m = "residual_mult" and LN the layer norm with weight and bias, (x - mean) / sqrt(var + eps) * w + b.
* Mixer "attention": grouped-query attention with a score scale of its own, rotary angles on the first "rot.dims"
  dimensions of each head in interleaved pairs (2i, 2i+1), frequencies blended between f_i and f_i / factor
  (a linear ramp between two pair indices found from "fast" and "slow" turns over the "original" length), cosines and
  sines stretched by 0.1 ln(factor) + 1; values of width "vdim"; in layers with "v_mix", except the first of them,
  v <- (1 - lambda) v + lambda v_first.
* Mixer "mamba1": in-projection to [x | z], a causal depthwise convolution with bias and silu on x, a selective scan
  whose step dt = softplus(W_dt dt_low + b), decay exp(dt A) with A = -exp(A_log), input dt x B, read-out C plus
  D x, a gate silu(z), and the out-projection.
* Feed-forward: g = min(Wg h, L), u = clamp(Wu h, -L, L), y = g sigmoid(1.702 g) (u + 1), out = Wd y; either one such
  layer ("dense") or "experts" of them of which each token takes the "top" by router logit, weighted by the softmax
  over the chosen logits.
* logits = head LN_final(x).
"""
import json
import math
import os
import struct

import numpy as np


# ---- files ---------------------------------------------------------------------------------------------------------
def read_safetensors(path):
    """{name: float64 array (int tables stay int)} from a file laid out as: 8-byte little-endian header length, the
    JSON header (name -> dtype, shape, data_offsets), the data."""
    with open(path, "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = data[lo:hi]
        kind = meta["dtype"]
        if kind == "BF16":
            a = np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16
            a = a.view(np.float32).astype(np.float64)
        elif kind == "F32":
            a = np.frombuffer(raw, dtype="<f4").astype(np.float64)
        elif kind == "I32":
            a = np.frombuffer(raw, dtype="<i4").copy()
        else:
            raise ValueError(f"{name}: dtype {kind}")
        out[name] = a.reshape(meta["shape"])
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small functions -----------------------------------------------------------------------------------------------
def layer_norm(x, w, b, eps):
    mu = x.mean(axis=-1, keepdims=True)
    var = ((x - mu) ** 2).mean(axis=-1, keepdims=True)
    return (x - mu) / np.sqrt(var + eps) * w + b


def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def softplus(x):
    return np.log1p(np.exp(-np.abs(x))) + np.maximum(x, 0.0)


def linear(x, w):
    """Weights are stored [out, in]."""
    return x @ w.T


# ---- rotary angles ---------------------------------------------------------------------------------------------------
def rotary_frequencies(rot):
    """Per pair i < dims/2: the frequency after the blend, and the stretch of cosines and sines."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    i = np.arange(half, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = sc["factor"], sc["original"]

    def pair_of(turns):                     # the (fractional) pair whose wavelength makes `turns` turns over `original`
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(pair_of(sc["fast"])), 0)
    hi = min(math.ceil(pair_of(sc["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(v, positions, rot):
    """v [T, H, D]: pairs (2i, 2i+1) of the first rot.dims dimensions turn by position * frequency_i."""
    f, stretch = rotary_frequencies(rot)
    dims = rot["dims"]
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * stretch)[:, None, :], (np.sin(ang) * stretch)[:, None, :]
    out = v.copy()
    a, b = v[..., 0:dims:2], v[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# ---- mixers -------------------------------------------------------------------------------------------------------------
def causal_attention(q, k, v, scale):
    """q [T, H, D], k [T, G, D], v [T, G, Dv]; query head h reads kv head h // (H // G); position i sees j <= i."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = np.where(mask, s, -np.inf)
        s = s - s.max(axis=-1, keepdims=True)
        p = np.exp(s)
        p = p / p.sum(axis=-1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def attention_mixer(h, w, pre, m, shared):
    """shared['v_first']: the values of the first layer with v_mix, for the later ones."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = linear(h, w[pre + "q"]).reshape(T, H, D)
    k = linear(h, w[pre + "k"]).reshape(T, G, D)
    v = linear(h, w[pre + "v"]).reshape(T, G, Dv)
    pos = np.arange(T)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    if m.get("v_mix"):
        if "v_first" not in shared:
            shared["v_first"] = v
        else:
            lam = float(w[pre + "vmix"])
            v = (1.0 - lam) * v + lam * shared["v_first"]
    o = causal_attention(q, k, v, m["scale"])
    return linear(o.reshape(T, H * Dv), w[pre + "o"])


def causal_conv(x, taps, bias):
    """x [T, C], taps [C, K]: y[t] = bias + sum_j taps[:, j] * x[t - (K - 1) + j], zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    y = np.tile(bias, (T, 1)).astype(np.float64)
    for j in range(K):
        y += padded[j:j + T] * taps[:, j]
    return y


def selective_scan(x, dt, A, B, C, D):
    """x, dt [T, C]; A [C, N]; B, C [T, N]; D [C].  S <- exp(dt A) S + dt x B; y = S C + D x, from S = 0."""
    T, Cn = x.shape
    S = np.zeros_like(A)
    y = np.zeros((T, Cn))
    for t in range(T):
        S = np.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + D * x[t]
    return y


def mamba1_mixer(h, w, pre, m):
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    xz = linear(h, w[pre + "in"])
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, w[pre + "conv"], w[pre + "conv.b"]))
    low = linear(x, w[pre + "x"])
    dt_low, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:R + 2 * N]
    dt = softplus(linear(dt_low, w[pre + "dt"]) + w[pre + "dt.b"])
    y = selective_scan(x, dt, -np.exp(w[pre + "A_log"]), B, C, w[pre + "D"])
    return linear(y * silu(z), w[pre + "o"])


# ---- feed-forward ----------------------------------------------------------------------------------------------------------
def gated_unit(h, gate, up, down, limit):
    g = np.minimum(linear(h, gate), limit)
    u = np.clip(linear(h, up), -limit, limit)
    return linear(g * sigmoid(1.702 * g) * (u + 1.0), down)


def dense_ff(h, w, pre, mlp):
    return gated_unit(h, w[pre + "gate"], w[pre + "up"], w[pre + "down"], mlp["limit"])


def router_choice(h, router, bias, top):
    """Indices [T, top] of the largest logits (ties: the lower index) and the softmax over those logits alone."""
    z = linear(h, router) + bias
    idx = np.argsort(-z, axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(z, idx, axis=-1)
    e = np.exp(chosen - chosen.max(axis=-1, keepdims=True))
    return idx, e / e.sum(axis=-1, keepdims=True)


def moe_ff(h, w, pre, mlp):
    idx, weight = router_choice(h, w[pre + "router"], w[pre + "router.b"], mlp["router"]["top"])
    out = np.zeros((h.shape[0], w[pre + "e0.down"].shape[0]))
    for t in range(h.shape[0]):
        for j, e in enumerate(idx[t]):
            p = f"{pre}e{e}."
            out[t] += weight[t, j] * gated_unit(h[t:t + 1], w[p + "gate"], w[p + "up"], w[p + "down"], mlp["expert"]["limit"])[0]
    return out


# ---- the model -------------------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from position 0.  layers_out (a list) receives the residual after each layer."""
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    x = w["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    shared = {}

    def ln(name, v):
        return layer_norm(v, w[name], w[name + ".b"], eps)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = ln(p + "norm1", x)
        if layer["type"] == "attention":
            y = attention_mixer(h, w, p + "mix.", layer["mixer"], shared)
        elif layer["type"] == "mamba1":
            y = mamba1_mixer(h, w, p + "mix.", layer["mixer"])
        else:
            raise ValueError(layer["type"])
        x = x + mult * ln(p + "norm1b", y)
        mlp = layer.get("mlp")
        if mlp:
            h = ln(p + "norm2", x)
            y = dense_ff(h, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_ff(h, w, p + "mlp.", mlp)
            x = x + mult * ln(p + "norm2b", y)
        if layers_out is not None:
            layers_out.append(x.copy())
    return linear(ln("final.norm", x), w["head"])
