"""A plain, slow Sizizen forward pass: one whole sequence from position 0, no cache, one function per mechanism.

It shares no code with ``purhie_b200``: it reads ``config.json`` with ``json`` and the weight file by its byte
layout, and states every equation directly.  Everything runs in float64.

The design in short (names of config.json in quotes):

* x0 = embed[token].
* A layer norms what a part gives, not what it reads: x <- x + LN1(mixer(x)), then, if the layer has a feed-forward,
  x <- x + LN2(ff(x)), LN(a) = (a - mean a) / sqrt(var a + eps) * w (no bias), eps = "norm.eps".
* The mixer "parallel" runs two mixers on the same input and returns (RMS(left; w_l) + RMS(right; w_r)) / 2 with
  RMS(a; w) = a / sqrt(mean a^2 + eps) * w over the model width.
  - left: grouped-query softmax attention with biases on q, k, v, an RMS norm per head on q and k (one weight for
    all heads), a rotation of the first "rot.dims" dimensions of each head (dimension i with i + dims/2, angle
    p * base^(-2i/dims)), the score scale "scale", values "vdim" wide, and a mask of blocks: position i sees j <= i
    with floor(i / "mask.size") = floor(j / "mask.size").
  - right: gated linear attention: per head a matrix S (dim x vdim), S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t,
    a_t = sigmoid(W_a2 W_a1 h + b)^(1/"tau") per key channel, q scaled by dim^(-1/2); o is RMS-normed per head,
    gated by silu(W_g h) and projected.
* Feed-forward "dense": W_down (silu(W_gate h) * W_up h).  "moe": experts W_down relu(W_up h)^2; scores sigmoid(W_r
  h); the choice adds "correction" to the scores, keeps the "groups.keep" groups of neighbouring experts whose two
  largest choice scores add up highest, and takes the "top" largest choice scores among those; the chosen experts'
  outputs are weighted with their scores (without the correction, not renormalised); a shared expert of the same
  form is added for every token.
* logits = head LN_final(x).
"""
import json
import math
import os
import struct

import numpy as np


# ---- files ---------------------------------------------------------------------------------------------------------
def read_safetensors(path):
    """{name: float64 array (int tables stay int)}: 8-byte little-endian header length, the JSON header (name ->
    dtype, shape, data_offsets), the data."""
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
            a = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
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
def sigmoid(x):
    return 1.0 / (1.0 + np.exp(-x))


def silu(x):
    return x * sigmoid(x)


def layer_norm(a, w, eps):
    mu = a.mean(axis=-1, keepdims=True)
    var = ((a - mu) ** 2).mean(axis=-1, keepdims=True)
    return (a - mu) / np.sqrt(var + eps) * w


def rms_norm(a, w, eps):
    return a / np.sqrt((a * a).mean(axis=-1, keepdims=True) + eps) * w


# ---- the left mixer ------------------------------------------------------------------------------------------------
def rotate(x, positions, base, dims):
    """x [T, heads, dim]: dimension i < dims/2 turns together with dimension i + dims/2 by positions * base^(-2i/dims)."""
    half = dims // 2
    out = x.copy()
    for i in range(half):
        angle = positions * base ** (-2.0 * i / dims)
        c, s = np.cos(angle)[:, None], np.sin(angle)[:, None]
        u, v = x[:, :, i], x[:, :, i + half]
        out[:, :, i] = u * c - v * s
        out[:, :, i + half] = v * c + u * s
    return out


def block_mask(T, size):
    """visible[i, j]: j <= i and both in the same block of `size` positions counted from 0."""
    i = np.arange(T)[:, None]
    j = np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def softmax_attention(q, k, v, scale, visible):
    """q [T, H, D], k [T, G, D], v [T, G, DV] -> [T, H, DV]; query head h reads key/value head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        s = q[:, h] @ k[:, g].T * scale
        s = np.where(visible, s, -np.inf)
        p = np.exp(s - s.max(axis=1, keepdims=True))
        p /= p.sum(axis=1, keepdims=True)
        out[:, h] = p @ v[:, g]
    return out


def left_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T + w[pre + "q.b"]).reshape(T, H, D)
    k = (h @ w[pre + "k"].T + w[pre + "k.b"]).reshape(T, G, D)
    v = (h @ w[pre + "v"].T + w[pre + "v.b"]).reshape(T, G, DV)
    q = rms_norm(q, w[pre + "q.norm"], eps)
    k = rms_norm(k, w[pre + "k.norm"], eps)
    pos = np.arange(T, dtype=np.float64)
    q = rotate(q, pos, m["rot"]["base"], m["rot"]["dims"])
    k = rotate(k, pos, m["rot"]["base"], m["rot"]["dims"])
    o = softmax_attention(q, k, v, m["scale"], block_mask(T, m["mask"]["size"]))
    return o.reshape(T, H * DV) @ w[pre + "o"].T


# ---- the right mixer -----------------------------------------------------------------------------------------------
def decayed_outer_recurrence(q, k, v, a):
    """Per head: S_t = diag(a_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.  q, k, a [T, H, D]; v [T, H, DV]."""
    T, H, D = q.shape
    DV = v.shape[2]
    o = np.zeros((T, H, DV))
    S = np.zeros((H, D, DV))
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hdv,hd->hv", S, q[t])
    return o


def right_mixer(h, w, pre, m, eps):
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[pre + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[pre + "k"].T).reshape(T, H, D)
    v = (h @ w[pre + "v"].T).reshape(T, H, DV)
    z = (h @ w[pre + "a1"].T) @ w[pre + "a2"].T + w[pre + "a2.b"]
    a = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, D)
    o = decayed_outer_recurrence(q, k, v, a)
    o = rms_norm(o, w[pre + "norm"], eps).reshape(T, H * DV)
    return (o * silu(h @ w[pre + "g"].T)) @ w[pre + "o"].T


def parallel_mixer(h, w, pre, m, eps):
    left = left_mixer(h, w, pre + "left.", m["left"], eps)
    right = right_mixer(h, w, pre + "right.", m["right"], eps)
    return 0.5 * (rms_norm(left, w[pre + "left.out"], eps) + rms_norm(right, w[pre + "right.out"], eps))


# ---- feed-forwards -------------------------------------------------------------------------------------------------
def dense_ff(h, w, pre):
    return (silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def squared_relu_expert(h, w, pre):
    return np.maximum(h @ w[pre + "up"].T, 0.0) ** 2 @ w[pre + "down"].T


def choose_experts(scores, correction, top, groups, keep):
    """One token.  Returns the chosen experts in descending order of their choice scores."""
    choice = scores + correction
    E = len(choice)
    per = E // groups
    group_score = [np.sort(choice[g * per:(g + 1) * per])[-2:].sum() for g in range(groups)]
    kept = sorted(range(groups), key=lambda g: (-group_score[g], g))[:keep]
    allowed = np.full(E, -np.inf)
    for g in kept:
        allowed[g * per:(g + 1) * per] = choice[g * per:(g + 1) * per]
    return sorted(range(E), key=lambda e: (-allowed[e], e))[:top]


def moe_ff(h, w, pre, f):
    r = f["router"]
    scores = sigmoid(h @ w[pre + "router"].T)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e in choose_experts(scores[t], w[pre + "correction"], r["top"], r["groups"]["count"], r["groups"]["keep"]):
            out[t] += scores[t, e] * squared_relu_expert(h[t:t + 1], w, f"{pre}e{e}.")[0]
    return out + squared_relu_expert(h, w, pre + "shared.")


# ---- the model -----------------------------------------------------------------------------------------------------
def forward(cfg, w, tokens, layer_outputs=None):
    """logits [T, vocab] for one sequence from position 0; layer_outputs (a list) receives x after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{i}."
        if layer["type"] != "parallel":
            raise ValueError(f"layer {i}: type {layer['type']}")
        x = x + layer_norm(parallel_mixer(x, w, pre + "mix.", layer["mixer"], eps), w[pre + "norm1"], eps)
        f = layer.get("mlp")
        if f is not None:
            y = dense_ff(x, w, pre + "mlp.") if f["kind"] == "dense" else moe_ff(x, w, pre + "mlp.", f)
            x = x + layer_norm(y, w[pre + "norm2"], eps)
        if layer_outputs is not None:
            layer_outputs.append(x.copy())
    return layer_norm(x, w["final.norm"], eps) @ w["head"].T
