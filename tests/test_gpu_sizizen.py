"""The Sizizen design in the engine against the plain implementation (GPU): every mechanism alone, whole prompts, cuts
down to two tokens, decoding, unequal batches, pages and state slots used again, keys far away, at page borders and
either side of a mask block's edge, other sizes than any real model's, and greedy generation through the entry point
and the scheduler."""
import os

import numpy as np
import pytest

from plain import sizizen_plain as P
from sizizen_helpers import (CONFIG_A, CONFIG_B, CONFIG_C, bf16_round, config, dense, draw_weights, left, make_folder, moe, right,
                             steady_choice, tokens)

pytestmark = pytest.mark.gpu

CONFIGS = {"A": CONFIG_A, "B": CONFIG_B, "C": CONFIG_C}
TOL = {"float32": 2e-4, "bfloat16": 6e-2}


def f64(w):
    return {k: np.asarray(v, dtype=np.float64) for k, v in w.items()}


class Models:
    """Per configuration and dtype: (folder, config, weights for the plain implementation).  The float32 runs read
    weights stored in 32 bits with routers left free; the bfloat16 runs read the same values stored as bfloat16 with
    corrections that fix which experts are chosen (a rounding of the router's input must not change the set)."""

    def __init__(self, factory):
        self.items = {}
        for i, (name, cfg) in enumerate(CONFIGS.items()):
            w = draw_weights(cfg, 300 + i)
            self.items[name, "float32"] = (make_folder(factory.mktemp(f"sz_{name}_f32"), cfg, w, "F32"), cfg, f64(w))
            ws = steady_choice(cfg, w, i)
            self.items[name, "bfloat16"] = (make_folder(factory.mktemp(f"sz_{name}_bf16"), cfg, ws, "BF16"), cfg, f64(ws))

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


def part_of(cfg, layer, name):
    from purhie_b200.config import ModelConfig
    spec = ModelConfig.from_dict(cfg).model_spec()
    part = spec["layers"][layer]["parts"][name] if layer is not None else spec[name]
    return part["kind"], part["params"]


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


def test_every_layer_agrees_with_the_plain_implementation(models):
    """The residual stream after each layer, so that a fault shows where it starts."""
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models["A"]
    toks = tokens(40, cfg["vocab"], 3)
    ref = []
    P.forward(cfg, w, toks, ref)
    eng = engine_for(folder, "float32")
    got = {}
    eng.set_layer_dump(lambda entry, x: got.__setitem__(entry, np.array(x)))
    eng.add_request("x")
    eng.step([StepEntry("x", toks, [len(toks) - 1])])
    assert sorted(got) == list(range(len(cfg["layers"])))
    for i, r in enumerate(ref):
        close(got[i], r, 1e-4)
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


@pytest.mark.parametrize("name,dtype", [("A", "float32"), ("C", "bfloat16"), ("C", "float32")])
def test_a_long_prompt_alone_and_beside_a_decode_row_and_a_two_token_portion(models, name, dtype):
    """330 tokens: many blocks of the mask, hundreds of steps of the recurrence, and enough (token, choice) pairs for the
    experts' tiled products."""
    from purhie_b200.engine import StepEntry
    folder, cfg, w = models[name, dtype]
    eng = engine_for(folder, dtype, max_tokens=1024)
    toks = tokens(330, cfg["vocab"], 11)
    ref = P.forward(cfg, w, toks)
    close(run_cut(eng, "whole", toks, []), ref, TOL[dtype])
    eng.add_request("a"); eng.add_request("b"); eng.add_request("c")
    eng.step([StepEntry("b", toks[:5], []), StepEntry("c", toks[:9], [])])
    out = eng.step([StepEntry("b", toks[5:6], [0]), StepEntry("a", toks[:300], list(range(300))), StepEntry("c", toks[9:11], [0, 1])])
    close(out[1:301], ref[:300], TOL[dtype])
    close(out[:1], ref[5:6], TOL[dtype])
    close(out[301:], ref[9:11], TOL[dtype])
    eng.close()


def test_long_decoding_crosses_many_blocks_and_keeps_its_state(models):
    folder, cfg, w = models["A"]
    eng = engine_for(folder, "float32", max_tokens=256)
    toks = tokens(230, cfg["vocab"], 3)
    ref = P.forward(cfg, w, toks)
    got = run_cut(eng, "long", toks, [2] + [1] * 228)
    close(got, ref, TOL["float32"])
    eng.close()


def test_pages_behind_the_current_block_go_back_to_the_pool(models):
    """A model whose every layer masks by blocks keeps only the pages that the next position can still see."""
    from purhie_b200.engine import StepEntry
    cfg = config(32, 30, [(left(2, 1, 8, 8, 4, 16), right(1, 8, 8, 2.0, 2), None)])
    w = draw_weights(cfg, 1)
    import tempfile
    with tempfile.TemporaryDirectory() as tmp:
        folder = make_folder(tmp, cfg, w)
        eng = engine_for(folder, "float32", page_size=8, max_tokens=64)         # eight pages
        toks = tokens(200, cfg["vocab"], 2)
        ref = P.forward(cfg, f64(w), toks)
        eng.add_request("x")
        rows = []
        for at in range(0, 200, 10):                                             # 200 tokens through a pool of 64
            rows.append(eng.step([StepEntry("x", toks[at:at + 10], list(range(10)))]))
            assert eng.info()["free_pages"][0] >= 8 - 4
            eng.check_cache()
        close(np.concatenate(rows), ref, TOL["float32"])
        eng.close()


# ---- generation -----------------------------------------------------------------------------------------------------------
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
    folder, cfg, w = models["B"]
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


def test_a_folder_gives_the_rank_that_the_configuration_leaves_out(models, tmp_path):
    """Without `rank` the inner size of the decay's two products is the stored matrices'."""
    import copy
    folder, cfg, w = models["B"]
    bare = copy.deepcopy(cfg)
    for layer in bare["layers"]:
        del layer["mixer"]["right"]["rank"]
    other = make_folder(tmp_path, bare, {k: np.asarray(v, dtype=np.float32) for k, v in w.items()})
    toks = tokens(20, cfg["vocab"], 1)
    eng = engine_for(other, "float32")
    close(run_cut(eng, "x", toks, [7]), P.forward(cfg, w, toks), TOL["float32"])
    eng.close()


# ---- one key decides: far back, at page borders, either side of a block's edge --------------------------------------------
def spiked_model(tmp_path, key_at, length, mask):
    """One layer in which only the left mixer speaks (the right side's output weight is zero).  The last token's query
    matches the key of token ``key_at`` alone, through a dimension that is not rotated, and the values copy a coordinate
    that only that token has: if the key is missed (a page's edge, a table one entry short, the first tokens), or seen
    where the mask hides it, the logits move by much."""
    width, vocab = 32, 24
    cfg = config(width, vocab, [(left(2, 1, 16, 8, 8, mask, scale=1.0), right(1, 4, 4, 2.0, 2), None)], eps=1e-5)
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
    q = np.zeros((32, width), np.float32)
    k = np.zeros((16, width), np.float32)
    v = np.zeros((8, width), np.float32)
    for h in range(2):
        q[h * 16 + 12, 10] = 2.0                    # unrotated dimension 12 of each head asks
    k[12, 8] = 2.0                                  # ... and only the marked token's key answers there
    v[0, 9] = 1.0
    v[1:, :8] = rng.normal(0, 0.3, (7, 8))
    w["l0.mix.left.q"], w["l0.mix.left.k"], w["l0.mix.left.v"] = q, k, v
    for n in ("q.b", "k.b", "v.b"):
        w["l0.mix.left." + n] = np.zeros_like(w["l0.mix.left." + n])
    w["l0.mix.left.q.norm"] = np.ones(16, np.float32)            # a head with one coordinate is normed to 4 there: a score of 16
    w["l0.mix.left.k.norm"] = np.ones(16, np.float32)
    w["l0.mix.right.out"] = np.zeros(width, np.float32)
    w = {n: bf16_round(a) for n, a in w.items()}
    return make_folder(tmp_path, cfg, w), cfg, f64(w), toks


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("key_at,length,mask", [
    (0, 300, 1000), (0, 2, 1000), (7, 200, 1000), (8, 200, 1000), (143, 400, 1000),       # far back, page borders (pages of 8)
    (96, 100, 32), (95, 100, 32),          # the block's first position, and the position in front of it
    (96, 128, 32), (95, 127, 32),          # the asking token is the block's last, or the next block's first
    (96, 129, 32), (20, 30, 10), (19, 30, 10), (29, 31, 10), (30, 32, 31), (0, 31, 31),
])
def test_one_key_decides_the_last_token_when_the_mask_lets_it_be_seen(tmp_path, key_at, length, mask, dtype):
    folder, cfg, w, toks = spiked_model(tmp_path, key_at, length, mask)
    ref = P.forward(cfg, w, toks)[-1:]
    seen = key_at // mask == (length - 1) // mask
    without = list(toks)
    without[key_at] = 2
    moved = np.abs(P.forward(cfg, w, without)[-1:] - ref).max() > 0.2 * np.abs(ref).max()
    assert moved == seen                  # the marked key carries the answer exactly when it is in the asking token's block
    eng = engine_for(folder, dtype, page_size=8, max_tokens=1024)
    for rid, cuts in (("prompt", []), ("decoded", [length - 1]), ("cut", [max(key_at, 1), 2]), ("tail", [max(length - 3, 1), 1, 1])):
        got = run_cut(eng, rid, toks, cuts)[-1:]
        close(got, ref, TOL[dtype])
    eng.close()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("length", [3, 260])
def test_the_first_token_is_still_in_the_state_hundreds_of_tokens_later(tmp_path, length, dtype):
    """Only the right mixer speaks, its decay held near one: what the first token wrote into the state is what the last
    token reads, prompt or decoded, whole or cut at the first token."""
    width, vocab = 32, 24
    cfg = config(width, vocab, [(left(1, 1, 8, 8, 4, 50), right(2, 8, 4, 16.0, 2), None)], eps=1e-5)
    w = draw_weights(cfg, 12)
    w["l0.mix.left.out"] = np.zeros(width, np.float32)
    w["l0.mix.right.a2"] = np.zeros_like(w["l0.mix.right.a2"])
    w["l0.mix.right.a2.b"] = np.full(16, 9.0, np.float32)          # sigmoid(9)^(1/16): a loss of a hundred-thousandth per token
    toks = [1 + (i % 5) for i in range(length)]
    toks[0], toks[-1] = 20, 21
    embed = np.zeros((vocab, width), dtype=np.float32)
    rng = np.random.default_rng(4)
    embed[:, :8] = rng.normal(0, 0.05, (vocab, 8))
    embed[20, 8], embed[20, 9] = 6.0, -4.0
    embed[21, 10] = 6.0
    w["embed"] = embed
    q = np.zeros((16, width), np.float32)
    k = np.zeros((16, width), np.float32)
    v = np.zeros((8, width), np.float32)
    q[3, 10] = q[8 + 3, 10] = 3.0
    k[3, 8] = k[8 + 3, 8] = 3.0
    v[0, 9] = v[4 + 1, 9] = 1.0
    w["l0.mix.right.q"], w["l0.mix.right.k"], w["l0.mix.right.v"] = q, k, v
    w = {n: bf16_round(a) for n, a in w.items()}
    folder = make_folder(tmp_path, cfg, w)
    ref = P.forward(cfg, f64(w), toks)[-1:]
    without = list(toks)
    without[0] = 2
    assert np.abs(P.forward(cfg, f64(w), without)[-1:] - ref).max() > 0.2 * np.abs(ref).max()
    eng = engine_for(folder, dtype, page_size=8, max_tokens=1024)
    for rid, cuts in (("prompt", []), ("decoded", [length - 1]), ("cut", [1, 2]), ("tail", [max(length - 3, 1), 1, 1])):
        close(run_cut(eng, rid, toks, cuts)[-1:], ref, TOL[dtype])
    eng.close()


# ---- the mechanisms alone ----------------------------------------------------------------------------------------------
def test_layer_norm_without_bias_on_an_addend_and_rows_that_pass_unnormed(models):
    """x <- x + LN(a) with the next part reading x as it is: the norm 'none' in front of a part folds the addend with its
    transform in and hands the rows on."""
    from purhie_b200.parts import PartProbe
    folder, cfg, w = models["B"]
    rng = np.random.default_rng(0)
    x = rng.normal(0.5, 2.0, (9, cfg["width"])).astype(np.float32)
    add = rng.normal(0.0, 1.0, (9, cfg["width"])).astype(np.float32)
    kind, params = part_of(cfg, 1, "mixer_post_norm")
    assert kind == "layernorm" and "bias" not in params["names"]
    p = PartProbe("norm", kind, params)
    p.bind_folder(folder)
    summed, normed = p.norm(x, add)
    close(summed, x.astype(np.float64) + add, 1e-6)
    close(normed, P.layer_norm(x.astype(np.float64) + add, w["l1.norm1"], cfg["norm"]["eps"]), 1e-5)
    none = PartProbe("norm", *part_of(cfg, 1, "mixer_norm"))
    none.bind_folder(folder)
    summed, rows = none.norm(x, add)
    close(summed, x.astype(np.float64) + add, 1e-6)
    close(rows, x.astype(np.float64) + add, 1e-6)


def mixer_in_pieces(p, x, pieces, request=1):
    p.add_request(request)
    out, at = [], 0
    for n in pieces:
        out.append(p.mixer_step([(request, n)], x[at:at + n]))
        at += n
    p.release(request)
    return np.concatenate(out)


def test_attention_under_a_block_mask_alone(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("A", 1), ("A", 3), ("B", 0), ("B", 1), ("B", 2)):
        folder, cfg, w = models[name]
        m = cfg["layers"][layer]["mixer"]["left"]
        x = np.random.default_rng(layer).normal(0, 1.0, (45, cfg["width"])).astype(np.float32)
        ref = P.left_mixer(x.astype(np.float64), w, f"l{layer}.mix.left.", m, cfg["norm"]["eps"])
        kind, params = part_of(cfg, layer, "mixer")
        assert kind == "side_by_side" and params["left"]["kind"] == "attention" and params["left"]["params"]["chunk"] == m["mask"]["size"]
        p = PartProbe("mixer", "attention", params["left"]["params"])
        p.bind_folder(folder)
        assert p.cache_need().get("chunk") == m["mask"]["size"]
        p.mixer_cache(8, 16, 2)
        close(mixer_in_pieces(p, x, [9, 1, 35]), ref, 1e-4)
        close(mixer_in_pieces(p, x, [1, 2, 2, 40]), ref, 1e-4)


def test_the_decayed_state_alone_cut_batched_and_in_a_slot_used_again(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("A", 1), ("A", 2), ("B", 0), ("B", 1), ("C", 0), ("C", 2)):
        folder, cfg, w = models[name]
        m = cfg["layers"][layer]["mixer"]["right"]
        rng = np.random.default_rng(layer)
        xs = {r: rng.normal(0, 1.0, (n, cfg["width"])).astype(np.float32) for r, n in ((1, 33), (2, 6), (3, 1), (4, 19))}
        ref = {r: P.right_mixer(x.astype(np.float64), w, f"l{layer}.mix.right.", m, cfg["norm"]["eps"]) for r, x in xs.items()}
        kind, params = part_of(cfg, layer, "mixer")
        p = PartProbe("mixer", "gated_linear_attention", params["right"]["params"])
        p.bind_folder(folder)
        heads, vdim, padded = p.cache_need()["state_shape"]              # key channels padded to the kernel's threads
        assert (heads, vdim) == (m["heads"], m["vdim"]) and m["dim"] <= padded < 2 * max(m["dim"], 16)
        p.mixer_cache(8, 16, 2)                                  # two state slots
        p.add_request(1)
        close(p.mixer_step([(1, 33)], xs[1]), ref[1], 1e-4)     # whole
        p.release(1)
        p.add_request(2)                                         # the slot of request 1, zeroed
        p.add_request(3)
        out = p.mixer_step([(2, 2), (3, 1)], np.concatenate([xs[2][:2], xs[3]]))
        out2 = p.mixer_step([(2, 1)], xs[2][2:3])
        out3 = p.mixer_step([(2, 3)], xs[2][3:])
        close(np.concatenate([out[:2], out2, out3]), ref[2], 1e-4)
        close(out[2:], ref[3], 1e-4)
        p.release(3)
        p.add_request(4)
        a = p.mixer_step([(4, 7)], xs[4][:7])
        b = np.concatenate([p.mixer_step([(4, 1)], xs[4][i:i + 1]) for i in range(7, 19)])
        close(np.concatenate([a, b]), ref[4], 1e-4)


def test_the_decay_follows_tau_and_the_bias():
    """alpha = sigmoid(z)^(1/tau) over a range of z that reaches both ends, against the plain recurrence."""
    from purhie_b200.parts import PartProbe
    for tau in (1.0, 3.0, 64.0):
        cfg = config(16, 10, [(left(1, 1, 4, 4, 2, 8), right(2, 6, 3, tau, 4), None)])
        w = draw_weights(cfg, 5)
        w["l0.mix.right.a2.b"] = np.linspace(-12.0, 12.0, 12).astype(np.float32)
        import tempfile
        with tempfile.TemporaryDirectory() as tmp:
            folder = make_folder(tmp, cfg, w)
            x = np.random.default_rng(1).normal(0, 1.0, (24, 16)).astype(np.float32)
            ref = P.right_mixer(x.astype(np.float64), f64(w), "l0.mix.right.", cfg["layers"][0]["mixer"]["right"], cfg["norm"]["eps"])
            p = PartProbe("mixer", "gated_linear_attention", part_of(cfg, 0, "mixer")[1]["right"]["params"])
            p.bind_folder(folder)
            p.mixer_cache(8, 4, 1)
            close(mixer_in_pieces(p, x, [5, 1, 18]), ref, 1e-4)


def test_two_mixers_side_by_side_alone(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 1), ("B", 2)):
        folder, cfg, w = models[name]
        x = np.random.default_rng(layer).normal(0, 1.0, (30, cfg["width"])).astype(np.float32)
        ref = P.parallel_mixer(x.astype(np.float64), w, f"l{layer}.mix.", cfg["layers"][layer]["mixer"], cfg["norm"]["eps"])
        p = PartProbe("mixer", *part_of(cfg, layer, "mixer"))
        p.bind_folder(folder)
        need = p.cache_need()
        assert need["kind"] == "pages" and need["state_shape"]          # pages of the one, the state of the other
        p.mixer_cache(8, 16, 2)
        close(mixer_in_pieces(p, x, [30]), ref, 1e-4)
        close(mixer_in_pieces(p, x, [3, 1, 2, 24], request=2), ref, 1e-4)


def test_feed_forwards_dense_routed_and_the_shared_expert(models):
    from purhie_b200.parts import PartProbe
    for name, layer in (("A", 0), ("A", 1), ("A", 3), ("B", 0), ("B", 1), ("B", 2)):
        folder, cfg, w = models[name]
        mlp = cfg["layers"][layer]["mlp"]
        x = np.random.default_rng(layer).normal(0, 1.5, (21, cfg["width"])).astype(np.float32)
        h = x.astype(np.float64)
        pre = f"l{layer}.mlp."
        ref = P.dense_ff(h, w, pre) if mlp["kind"] == "dense" else P.moe_ff(h, w, pre, mlp)
        p = PartProbe("feed_forward", *part_of(cfg, layer, "feed_forward"))
        p.bind_folder(folder)
        close(p.feed_forward(x), ref, 1e-4)
        close(p.feed_forward(x[:1]), ref[:1], 1e-4)                        # one row alone chooses the same experts
    folder, cfg, w = models["A"]
    kind, params = part_of(cfg, 1, "feed_forward")
    shared = PartProbe("feed_forward", params["shared"]["kind"], params["shared"]["params"])
    shared.bind_folder(folder)
    x = np.random.default_rng(2).normal(0, 1.5, (5, cfg["width"])).astype(np.float32)
    close(shared.feed_forward(x), P.squared_relu_expert(x.astype(np.float64), w, "l1.mlp.shared."), 1e-4)


def test_the_choice_goes_by_corrected_scores_within_the_best_groups_and_the_weights_do_not(tmp_path):
    """Corrections that turn the order of the scores around, make choice scores negative and put the largest single score
    into a group that loses on its two best: the chosen set and the weights against the plain implementation, and the
    plain implementation against sets worked out by hand."""
    from purhie_b200.parts import PartProbe
    width = 16
    cfg = config(width, 10, [(left(1, 1, 4, 4, 2, 8), right(1, 4, 4, 2.0, 2), moe(8, 8, 2, 4, 2, 8))])
    w = draw_weights(cfg, 3)
    router = np.zeros((8, width), np.float32)
    router[np.arange(8), np.arange(8)] = 1.0                              # logit e = x[e]
    w["l0.mlp.router"] = router
    # groups (0,1) (2,3) (4,5) (6,7); logits chosen so that sigmoid scores are 0.9, 0.1 | 0.6, 0.62 | 0.5, 0.55 | 0.2, 0.3
    s = np.array([0.9, 0.1, 0.6, 0.62, 0.5, 0.55, 0.2, 0.3])
    x = np.zeros((3, width), np.float32)
    x[:, :8] = np.log(s / (1 - s))
    cases = [
        (np.zeros(8), [2, 3]),                                             # groups by two best: 1.22 and 1.05 win over 1.0; expert 0 is out
        (np.array([0, 0, -2, -2, -2.1, -2, -3, -3.0]), [0, 1]),           # kept groups (0,1) and (2,3); 0.1 beats the negative choice scores
        (np.array([-5, -5, -5, -5, -5, -5, 1.0, 0.0]), [6, 7]),           # the correction lifts the last group; weights stay 0.2 and 0.3
        (np.array([-5, -5, -5, -5, -5, -5, 1.0, -5.0]), [3, 6]),          # the second choice is negative (-4.38): a group left out counts
    ]                                                                      # as minus infinity, or one of its experts would come first
    for i, (corr, chosen) in enumerate(cases):
        w["l0.mlp.correction"] = corr.astype(np.float32)
        assert sorted(P.choose_experts(s, corr, 2, 4, 2)) == chosen
        ww = {n: bf16_round(np.asarray(a, np.float32)) for n, a in w.items()}
        ww["l0.mlp.router"] = router
        folder = make_folder(tmp_path / f"case{i}", cfg, ww)
        p = PartProbe("feed_forward", *part_of(cfg, 0, "feed_forward"))
        p.bind_folder(folder)
        h = x.astype(np.float64)
        ref = P.moe_ff(h, f64(ww), "l0.mlp.", cfg["layers"][0]["mlp"])
        by_hand = sum(s[e] * P.squared_relu_expert(h, f64(ww), f"l0.mlp.e{e}.") for e in chosen) + P.squared_relu_expert(h, f64(ww), "l0.mlp.shared.")
        close(ref, by_hand, 1e-6)
        close(p.feed_forward(x), ref, 1e-4)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_left_mixer_that_rotates_nothing_and_layers_in_another_order(tmp_path, dtype):
    """rot.dims 0 (no position encoding at all), a routed layer first, a layer without a feed-forward in the middle."""
    cfg = config(64, 50, [
        (left(4, 1, 16, 16, 0, 7), right(2, 16, 16, 2.0, 8), moe(16, 4, 2, 2, 1, 32)),
        (left(2, 2, 32, 8, 32, 20), right(1, 32, 64, 5.0, 4), None),
        (left(8, 4, 8, 8, 4, 3), right(4, 16, 8, 1.0, 16), dense(96)),
    ])
    w = draw_weights(cfg, 77)
    if dtype == "bfloat16":
        w = steady_choice(cfg, w, 3)
    folder = make_folder(tmp_path, cfg, w, "F32" if dtype == "float32" else "BF16")
    eng = engine_for(folder, dtype)
    toks = tokens(90, cfg["vocab"], 4)
    ref = P.forward(cfg, f64(w), toks)
    close(run_cut(eng, "whole", toks, []), ref, TOL[dtype])
    close(run_cut(eng, "cut", toks, [2, 19, 1, 1, 40, 2]), ref, TOL[dtype])
    eng.close()


@pytest.mark.parametrize("heads,dim,vdim", [(1, 128, 256), (2, 256, 128), (1, 512, 8), (3, 20, 130), (1, 72, 5)])
def test_states_too_large_for_one_block_and_odd_widths(tmp_path, heads, dim, vdim):
    """A head whose columns are spread over several blocks (the head norm then runs as a launch of its own), key channels
    that need 16 or 32 threads a column, value widths that are no multiple of four; whole, cut, and long enough for the
    chunked passes."""
    from purhie_b200.parts import PartProbe
    cfg = config(32, 20, [(left(1, 1, 8, 8, 4, 16), right(heads, dim, vdim, 6.0, 4), None)])
    w = draw_weights(cfg, heads * 1000 + dim)
    folder = make_folder(tmp_path, cfg, w)
    m = cfg["layers"][0]["mixer"]["right"]
    x = np.random.default_rng(dim).normal(0, 1.0, (150, 32)).astype(np.float32)
    ref = P.right_mixer(x.astype(np.float64), f64(w), "l0.mix.right.", m, cfg["norm"]["eps"])
    p = PartProbe("mixer", "gated_linear_attention", part_of(cfg, 0, "mixer")[1]["right"]["params"])
    p.bind_folder(folder)
    p.mixer_cache(8, 4, 2)
    close(mixer_in_pieces(p, x, [150]), ref, 2e-4)                       # chunks of 64, 64 and 22
    close(mixer_in_pieces(p, x, [1, 2, 17, 129, 1], request=2), ref, 2e-4)
