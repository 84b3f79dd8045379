"""The Bozosun design in the engine against the plain implementation (GPU): every mechanism alone, whole prompts, cuts
down to two tokens, decoding, unequal batches, pages and state slots used again, keys far away and at page borders,
other sizes than any real model's, and greedy generation through the entry point and the scheduler."""
import copy
import json
import os

import numpy as np
import pytest

from plain import bozosun_plain as P
from bozosun_helpers import (CONFIG_A, CONFIG_B, CONFIG_C, CONFIG_D, YARN, attention, bf16_round, config, dense, draw_weights, make_folder,
                             mamba, moe, rot, steady_routing, tokens)

pytestmark = pytest.mark.gpu

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


class Models:
    """Per configuration and dtype: (folder, config, weights for the plain implementation).  The float32 runs read
    weights stored in 32 bits with routers left free; the bfloat16 runs read the same values stored as bfloat16 (which
    is what puts the tensor-core products to work) with routers whose choice a rounding cannot change."""

    def __init__(self, factory):
        self.items = {}
        for i, (name, cfg) in enumerate(CONFIGS.items()):
            w = draw_weights(cfg, 100 + i)
            self.items[name, "float32"] = (make_folder(factory.mktemp(f"bz_{name}_f32"), cfg, w, "F32"), cfg, f64(w))
            ws = steady_routing(cfg, w, i)
            self.items[name, "bfloat16"] = (make_folder(factory.mktemp(f"bz_{name}_bf16"), cfg, ws, "BF16"), cfg, f64(ws))

    def __getitem__(self, key):
        return self.items[key if isinstance(key, tuple) else (key, "float32")]


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    return Models(tmp_path_factory)


def engine_for(folder, dtype, **kw):
    from purhie_b200.engine import Engine
    opts = dict(page_size=8, max_tokens=512, max_requests=4, poison_cache=True)
    opts.update(kw)
    return Engine.from_folder(folder, dtype=dtype, **opts)


def close(got, ref, tol):
    got, ref = np.asarray(got, dtype=np.float64), np.asarray(ref, dtype=np.float64)
    assert got.shape == ref.shape
    assert np.isfinite(got).all()
    err = np.abs(got - ref).max() / max(np.abs(ref).max(), 1e-30)
    assert err < tol, f"relative error {err:.3e} (allowed {tol:.1e})"


def run_cut(engine, rid, toks, cuts):
    """Feed ``toks`` in portions of the given sizes (the last portion takes what is left); all logits."""
    from purhie_b200.engine import StepEntry
    engine.add_request(rid)
    rows, at = [], 0
    for n in list(cuts) + [len(toks)]:
        n = min(n, len(toks) - at)
        if n <= 0:
            break
        rows.append(engine.step([StepEntry(rid, toks[at:at + n], list(range(n)))]))
        at += n
    engine.release(rid)
    return np.concatenate(rows)


# ---- whole models ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_prompts_cuts_and_decoding_agree_with_the_plain_implementation(models, name, dtype):
    folder, cfg, w = models[name, dtype]
    eng = engine_for(folder, dtype)
    toks = tokens(75, cfg["vocab"], 7)
    ref = P.forward(cfg, w, toks)
    whole = run_cut(eng, "whole", toks, [])
    close(whole, ref, TOL[dtype])
    # one token (the first of a sequence alone), then two, then portions of changing size, single tokens between them
    cut = run_cut(eng, "cut", toks, [1, 2, 2, 5, 1, 1, 16, 3, 17, 2, 1])
    close(cut, ref, TOL[dtype])
    # a prompt, then token by token: every decode step replays a graph
    tail = run_cut(eng, "tail", toks, [30] + [1] * 45)
    close(tail, ref, TOL[dtype])
    if dtype == "float32":                      # the 32-bit kernels add in one order however the tokens arrive
        assert np.abs(cut - whole).max() <= 1e-5 * np.abs(ref).max()
        assert np.abs(tail - whole).max() <= 1e-5 * np.abs(ref).max()
    eng.check_cache()
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(models, name, dtype):
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models[name, dtype]
    # room for two requests' states and about 100 tokens: five requests must take turns, pages come back poisoned
    eng = engine_for(folder, dtype, max_tokens=104, max_requests=2)
    lengths = [41, 9, 1, 56, 23]
    reqs = {f"r{i}": tokens(n, cfg["vocab"], 20 + i) for i, n in enumerate(lengths)}
    refs = {r: P.forward(cfg, w, t) for r, t in reqs.items()}
    at = {r: 0 for r in reqs}
    got = {r: [] for r in reqs}
    waiting, live, step = list(reqs), [], 0
    portions = [2, 7, 1, 1, 13, 2, 1, 5, 1, 1, 1, 9]
    while waiting or live:
        while waiting and len(live) < 2:
            r = waiting.pop(0)
            eng.add_request(r)
            live.append(r)
        entries = []
        for j, r in enumerate(live):
            n = min(portions[(step + 3 * j) % len(portions)], len(reqs[r]) - at[r])
            entries.append(StepEntry(r, reqs[r][at[r]:at[r] + n], list(range(n))))
        out = eng.step(entries)
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.request_id].append(out[row:row + n])
            row += n
            at[e.request_id] += n
        for r in list(live):
            if at[r] == len(reqs[r]):
                eng.release(r)
                live.remove(r)
        step += 1
        eng.check_cache()
    for r in reqs:
        close(np.concatenate(got[r]), refs[r], TOL[dtype])
    eng.close()


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("A", "bfloat16"), ("C", "bfloat16"), ("C", "float32")])
def test_a_prompt_of_many_pairs_goes_through_the_tiled_expert_products(models, name, dtype):
    """Past a few hundred (token, choice) pairs the experts' products change kernels: row tiles by expert on the CUDA
    cores in float32, slices per expert through the tensor-core product in bfloat16."""
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models[name, dtype]
    eng = engine_for(folder, dtype, max_tokens=1024)
    toks = tokens(330, cfg["vocab"], 11)
    ref = P.forward(cfg, w, toks)
    close(run_cut(eng, "whole", toks, []), ref, TOL[dtype])
    # the same tokens as a long portion beside another request's decode row and a two-token portion
    eng.add_request("a"); eng.add_request("b"); eng.add_request("c")
    eng.step([StepEntry("b", toks[:5], []), StepEntry("c", toks[:9], [])])
    out = eng.step([StepEntry("b", toks[5:6], [0]), StepEntry("a", toks[:300], list(range(300))), StepEntry("c", toks[9:11], [0, 1])])
    close(out[1:301], ref[:300], TOL[dtype])
    close(out[:1], ref[5:6], TOL[dtype])
    close(out[301:], ref[9:11], TOL[dtype])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_heads_of_128_go_through_the_vector_rotary_kernels(tmp_path, dtype):
    """Interleaved pairs and the value blend in the kernels that hold four or eight dimensions of a head per lane: a
    short prompt with decoding (the few-token kernel), and a prompt long enough for the many-token one."""
    w = draw_weights(CONFIG_D, 5)
    folder = make_folder(tmp_path, CONFIG_D, w, "F32" if dtype == "float32" else "BF16")
    eng = engine_for(folder, dtype, page_size=16, max_tokens=4608)
    toks = tokens(70, CONFIG_D["vocab"], 2)
    close(run_cut(eng, "short", toks, [40] + [1] * 20), P.forward(CONFIG_D, f64(w), toks), TOL[dtype])
    toks = tokens(4200, CONFIG_D["vocab"], 3)
    ref = P.forward(CONFIG_D, f64(w), toks)
    got = run_cut(eng, "long", toks, [4100, 2, 1])
    close(got, ref, TOL[dtype])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_model_of_state_space_layers_alone_keeps_no_pages(tmp_path, dtype):
    """No attention anywhere: the cache manager has state slots and not one page group; a convolution of one tap
    keeps no inputs; a layer's feed-forward may be missing."""
    cfg = config(24, 40, [(mamba(40, 8, 4, 1), dense(32, 1.0)), (mamba(32, 16, 8, 2), None), (mamba(40, 8, 4, 6), moe(8, 1.5, 4, 2))],
                 mult=0.6, eps=1e-4, embed_scale=2.0)
    w = draw_weights(cfg, 17)
    if dtype == "bfloat16":
        w = steady_routing(cfg, w, 1)
    folder = make_folder(tmp_path, cfg, w, "F32" if dtype == "float32" else "BF16")
    eng = engine_for(folder, dtype, max_requests=2)
    assert eng.info()["total_pages"] == []
    toks = tokens(210, cfg["vocab"], 6)
    ref = P.forward(cfg, f64(w), toks)
    close(run_cut(eng, "whole", toks, []), ref, TOL[dtype])
    close(run_cut(eng, "cut", toks, [3, 1, 2, 195, 1, 1]), ref, TOL[dtype])
    eng.close()


def test_long_decoding_keeps_its_state(models):
    folder, cfg, w = models["A"]
    eng = engine_for(folder, "float32", max_tokens=256)
    toks = tokens(230, cfg["vocab"], 3)
    ref = P.forward(cfg, w, toks)
    got = run_cut(eng, "long", toks, [2] + [1] * 228)
    close(got, ref, TOL["float32"])
    eng.close()


def test_greedy_generation_through_the_entry_point_and_the_scheduler(models):
    from purhie_b200.api import load_model
    from purhie_b200.sampling import SamplerParams
    folder, cfg, w = models["A"]
    model = load_model(folder, dtype="float32")
    model.kv_cache_init(256, max_sequences=3, page_size=8, max_batch_tokens=24, prefill_chunk=11)
    prompts = [tokens(n, cfg["vocab"], 60 + i) for i, n in enumerate((1, 14, 37))]

    def plain_greedy(prompt, n):
        toks = list(prompt)
        for _ in range(n):
            toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
        return toks[len(prompt):]
    expected = [plain_greedy(p, 10) for p in prompts]
    for p, exp in zip(prompts, expected):
        assert model.generate_ex(p, 10, SamplerParams.greedy()) == exp
    assert model.generate(prompts, max_new_tokens=10) == expected        # chunked prompts beside decoding requests
    model.free()


def test_the_command_line_generates_from_a_folder_of_this_design(models):
    import subprocess
    import sys
    from helpers import ROOT
    folder, cfg, w = models["A"]
    prompt = tokens(12, cfg["vocab"], 8)
    toks = list(prompt)
    for _ in range(5):
        toks.append(int(P.forward(cfg, w, toks)[-1].argmax()))
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "qwen_demo"), folder, ",".join(map(str, prompt)), "5", "--dtype", "float32",
                        "--ctx", "64"], capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert [int(x) for x in lines[2:7]] == toks[12:]


def test_trace_replay_reads_a_folder_of_this_design(models, tmp_path):
    from helpers import TraceRun
    folder, cfg, w = models["B"]
    toks = tokens(40, cfg["vocab"], 5)
    ref = P.forward(cfg, w, toks)
    run = TraceRun(folder, "float32", tmp_path, 128)
    run.vocab = cfg["vocab"]
    a = run.step(0, [("x", toks[:17], [0, 16])])
    b = run.step(1, [("x", toks[17:19], [1]), ("y", toks[:3], [2])])
    c = run.step(2, [("x", toks[19:], [20])], end=["x", "y"])
    run.close()
    close(np.concatenate([a.numpy(), b.numpy()[:1], c.numpy()]), ref[[0, 16, 18, 39]], TOL["float32"])
    close(b.numpy()[1:], ref[[2]], TOL["float32"])


# ---- keys far away, at page borders, the first tokens -------------------------------------------------------------------
def spiked_model(tmp_path, key_at, length):
    """One attention layer whose last token's query matches the key of token ``key_at`` alone, through dimensions that
    are not rotated, and whose values copy a coordinate that only that token has: if the key is missed (a page's edge,
    a table one entry short, the first tokens) the output loses that coordinate and the logits move by much."""
    width, vocab = 32, 24
    cfg = config(width, vocab, [(attention(2, 1, 16, 8, rot(8, 1e4, None), scale=1.0), None)], mult=1.0, eps=1e-5, embed_scale=1.0)
    w = draw_weights(cfg, 9)
    toks = [1 + (i % 5) for i in range(length)]
    toks[key_at] = 20                    # a token no other position has
    toks[-1] = 21
    embed = np.zeros((vocab, width), dtype=np.float32)
    rng = np.random.default_rng(4)
    embed[:, :8] = rng.normal(0, 1.0, (vocab, 8))
    embed[20, 8], embed[20, 9] = 6.0, -4.0          # the marked token: a key coordinate and a value coordinate
    embed[21, 10] = 6.0                             # the asking token
    w["embed"] = embed
    # the norm in front passes coordinates through (weight 1, bias 0) up to the row's own scale
    w["l0.norm1"], w["l0.norm1.b"] = np.ones(width, np.float32), np.zeros(width, np.float32)
    q = np.zeros((32, width), np.float32)
    k = np.zeros((16, width), np.float32)
    v = np.zeros((8, width), np.float32)
    for h in range(2):
        q[h * 16 + 12, 10] = 2.0                    # unrotated dimension 12 of each head asks
    k[12, 8] = 2.0                                  # ... and only the marked token's key answers there
    v[0, 9] = 1.0
    v[1:, :8] = rng.normal(0, 0.3, (7, 8))
    w["l0.mix.q"], w["l0.mix.k"], w["l0.mix.v"] = q, k, v
    w = {n: bf16_round(a) for n, a in w.items()}
    return make_folder(tmp_path, cfg, w), cfg, f64(w), toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key_at,length", [(0, 300), (0, 2), (7, 200), (8, 200), (15, 18), (16, 18), (143, 400), (1, 9)])
def test_one_key_far_back_or_at_a_page_border_decides_the_last_token(tmp_path, key_at, length, dtype):
    from purhie_b200.engine import StepEntry
    folder, cfg, w, toks = spiked_model(tmp_path, key_at, length)
    ref = P.forward(cfg, w, toks)[-1:]
    # the marked key carries the answer: without it the logits differ by far more than any tolerance here
    without = list(toks)
    without[key_at] = 2
    assert np.abs(P.forward(cfg, w, without)[-1:] - ref).max() > 0.2 * np.abs(ref).max()
    eng = engine_for(folder, dtype, page_size=8, max_tokens=1024)
    for rid, cuts in (("prompt", []), ("decoded", [length - 1]), ("cut", [max(key_at, 1), 2])):
        got = run_cut(eng, rid, toks, cuts)[-1:]
        close(got, ref, TOL[dtype])
    eng.close()


# ---- the mechanisms alone ----------------------------------------------------------------------------------------------
def part_of(cfg, layer, name):
    from purhie_b200.config import ModelConfig
    spec = ModelConfig.from_dict(cfg).model_spec()
    part = spec["layers"][layer]["parts"][name] if layer is not None else spec[name]
    return part["kind"], part["params"]


def test_layer_norm_with_bias_and_the_scaled_embedding(models):
    from purhie_b200.parts import PartProbe
    folder, cfg, w = models["B"]
    rng = np.random.default_rng(0)
    x = rng.normal(0.5, 2.0, (9, cfg["width"])).astype(np.float32)
    add = rng.normal(0.0, 1.0, (9, cfg["width"])).astype(np.float32)
    p = PartProbe("norm", *part_of(cfg, 2, "feed_forward_norm"))
    p.bind_folder(folder)
    summed, normed = p.norm(x, add)
    close(summed, x.astype(np.float64) + add, 1e-6)
    close(normed, P.layer_norm(x.astype(np.float64) + add, w["l2.norm2"], w["l2.norm2.b"], cfg["norm"]["eps"]), 1e-5)
    a = models["A"]
    e = PartProbe("embedding", *part_of(a[1], None, "embedding"))
    e.bind_folder(a[0])
    ids = [0, 5, 95, 5]
    close(e.embedding(ids, a[1]["width"]), a[2]["embed"][ids] * a[1]["embedding"]["scale"], 1e-7)


@pytest.mark.parametrize("rot_", [rot(16, 1e4, YARN), rot(10, 5e5, None), rot(8, 100.0, {"factor": 2.0, "original": 16, "fast": 4.0, "slow": 1.0}),
                                  rot(32, 1e6, {"factor": 32.0, "original": 4096, "fast": 32.0, "slow": 1.0})])
def test_rotation_table_with_and_without_scaling(rot_):
    from purhie_b200.parts import PartProbe
    params = {"theta": rot_["base"], "n_rot": rot_["dims"], "max_position": 700, "pairing": "interleaved"}
    if rot_["scaling"]:
        params["scaling"] = dict(rot_["scaling"], kind="yarn")
    p = PartProbe("position", "rope_neox", params)
    p.bind_random(0)
    table = p.position_table()
    f, stretch = P.rotary_frequencies(rot_)
    ang = np.arange(700)[:, None] * f[None, :]
    close(table, np.concatenate([np.cos(ang), np.sin(ang)], axis=1) * stretch, 2e-6)
    if rot_["scaling"]:
        plain_f = rot_["base"] ** (-2.0 * np.arange(rot_["dims"] // 2) / rot_["dims"])
        assert not np.allclose(f, plain_f)              # the scaling changes something at these sizes


def test_state_space_mixer_alone_cut_batched_and_in_a_slot_used_again(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 1), ("B", 0)):
        folder, cfg, w = models[name]
        m = cfg["layers"][layer]["mixer"]
        rng = np.random.default_rng(layer)
        xs = {r: rng.normal(0, 1.0, (n, cfg["width"])).astype(np.float32) for r, n in ((1, 33), (2, 6), (3, 1), (4, 19))}
        ref = {r: P.mamba1_mixer(x.astype(np.float64), w, f"l{layer}.mix.", m) for r, x in xs.items()}
        p = PartProbe("mixer", *part_of(cfg, layer, "mixer"))
        p.bind_folder(folder)
        p.mixer_cache(8, 16, 2)                                  # two state slots
        p.add_request(1)
        close(p.mixer_step([(1, 33)], xs[1]), ref[1], 1e-4)     # whole
        p.release(1)
        p.add_request(2)                                         # the slot of request 1, zeroed
        p.add_request(3)
        out = p.mixer_step([(2, 2), (3, 1)], np.concatenate([xs[2][:2], xs[3]]))      # shorter than the convolution
        out2 = p.mixer_step([(2, 1)], xs[2][2:3])
        out3 = p.mixer_step([(2, 3)], xs[2][3:])
        close(np.concatenate([out[:2], out2, out3]), ref[2], 1e-4)
        close(out[2:], ref[3], 1e-4)
        p.release(3)
        p.add_request(4)
        a = p.mixer_step([(4, 7)], xs[4][:7])
        b = np.concatenate([p.mixer_step([(4, 1)], xs[4][i:i + 1]) for i in range(7, 19)])
        close(np.concatenate([a, b]), ref[4], 1e-4)


def test_gated_units_dense_and_routed_with_the_clamps_at_work(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("B", 2), ("A", 1), ("B", 1), ("B", 4)):
        folder, cfg, w = models[name]
        mlp = cfg["layers"][layer]["mlp"]
        rng = np.random.default_rng(layer)
        x = rng.normal(0, 3.0, (21, cfg["width"])).astype(np.float32)      # large enough to reach every clamp
        h = x.astype(np.float64)
        pre = f"l{layer}.mlp."
        limit = mlp["limit"] if mlp["kind"] == "dense" else mlp["expert"]["limit"]
        gate_name = pre + ("gate" if mlp["kind"] == "dense" else "e0.gate")
        g = P.linear(h, w[gate_name])
        assert (g > limit).any() and (g < -limit).any()                    # clamped above, free below
        ref = P.dense_ff(h, w, pre, mlp) if mlp["kind"] == "dense" else P.moe_ff(h, w, pre, mlp)
        p = PartProbe("feed_forward", *part_of(cfg, layer, "feed_forward"))
        p.bind_folder(folder)
        close(p.feed_forward(x), ref, 1e-4)
        close(p.feed_forward(x[:1]), ref[:1], 1e-4)                        # one row alone chooses the same experts


def test_attention_alone_with_values_wider_and_narrower_than_keys(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("B", 1), ("B", 3), ("C", 2)):
        folder, cfg, w = models[name]
        m = cfg["layers"][layer]["mixer"]
        x = np.random.default_rng(layer).normal(0, 1.0, (45, cfg["width"])).astype(np.float32)
        ref = P.attention_mixer(x.astype(np.float64), w, f"l{layer}.mix.", dict(m, v_mix=False), {})
        p = PartProbe("mixer", *part_of(cfg, layer, "mixer"))
        p.bind_folder(folder)
        p.mixer_cache(8, 16, 2)
        p.add_request(1)
        got = np.concatenate([p.mixer_step([(1, 9)], x[:9]), p.mixer_step([(1, 1)], x[9:10]), p.mixer_step([(1, 35)], x[10:])])
        close(got, ref, 1e-4)


def test_value_mixing_changes_the_later_layers_only(models):
    """The same model with the mixing factors at zero differs; the first mixing layer's factor is never read."""
    folder, cfg, w = models["A"]
    toks = tokens(20, cfg["vocab"], 1)
    ref = P.forward(cfg, w, toks)
    w0 = dict(w)
    w0["l2.mix.vmix"] = np.zeros(())
    assert np.abs(P.forward(cfg, w0, toks) - ref).max() > 1e-3 * np.abs(ref).max()
    from purhie_b200.config import ModelConfig
    from purhie_b200.weights import expected_tensors
    names = expected_tensors(ModelConfig.from_dict(cfg))
    assert "l2.mix.vmix" in names and "l0.mix.vmix" not in names
