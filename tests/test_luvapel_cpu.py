"""Luvapel on the CPU: the plain model's mechanisms one by one, and the engine (configuration,
loader, run order, pages and states, step function, scheduler) over the kernels' plain
references against the plain model."""
import json
import os

import numpy as np
import pytest
import torch

from garuda_b200 import Engine, SamplingParams, StepEntry, ConfigError, WeightError
from garuda_b200.config.registry import build_model, read_model_config
from garuda_b200.parts.base import FixedState, PagedKV
from tests import helpers
from tests.luvapel_cases import CASES, LA, LB, LC, LD, model_dir, plain_logits, random_tokens, weights
from tests.plain import luvapel_plain as lp
from tests.plain.cpu_ops import CpuOps


def assert_close(got, want, dtype, what):
    """Against the 64-bit plain model, as a fraction of the largest logit: 32-bit sums in another
    order through up to five layers with sharpened weights."""
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(np.asarray(got) - want).max())
    assert got.shape == want.shape and np.isfinite(got).all(), what
    helpers.OBSERVED[f"luvapel/{dtype}"] = max(helpers.OBSERVED.get(f"luvapel/{dtype}", 0.0), err / scale)
    assert err <= 6e-5 * scale, f"{what}: max difference {err:.3e} (limit {6e-5 * scale:.3e})"


def engine(name, **kw):
    kw.setdefault("page_size", 8)
    kw.setdefault("kv_tokens", 512)
    kw.setdefault("context", 256)
    return Engine(model_dir(name), dtype="float32", ops=CpuOps(), cuda_graphs=False, **kw)


# ------------------------------------------------------------------ the plain model's mechanisms
def test_rms_has_eps_inside_the_root():
    assert np.allclose(lp.rms(np.array([[3.0, 4.0]]), 0.0), np.array([[3.0, 4.0]]) / np.sqrt(12.5))
    assert np.allclose(lp.rms(np.array([[2.0, 2.0]]), 5.0), 2.0 / 3.0)
    assert np.allclose(lp.rms(np.array([[0.0, 0.0]]), 4.0), 0.0)


def test_rotation_pairs_neighbours_and_leaves_the_rest():
    v = np.arange(1.0, 7.0).reshape(1, 1, 6)
    out = lp.rotate_interleaved(np.repeat(v, 2, 0), np.array([0, 3]), 100.0, 4)
    assert np.allclose(out[0], v[0])                              # position 0 turns nothing
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5                               # the pairs' angles at position 3
    assert np.allclose(out[1, 0, :2], [np.cos(a0) - 2 * np.sin(a0), 2 * np.cos(a0) + np.sin(a0)])
    assert np.allclose(out[1, 0, 2:4], [3 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 3 * np.sin(a1)])
    assert np.allclose(out[1, 0, 4:], [5.0, 6.0])                  # beyond the rotated width


def test_short_convolution_is_causal_and_starts_from_zeros():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    taps = np.array([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]])           # the last column weighs the current token
    y = lp.causal_conv(x, taps)
    assert np.allclose(y[:, 0], [2.0, 4.0, 6.5, 9.0, 11.5]) and np.allclose(y[:, 1], [0.0, 10.0, 20.0, 30.0, 40.0])


def test_gated_delta_by_hand():
    # one head, dim 2, vdim 1, one tap of weight one; the projections pick channels of h
    big = 40.0                                                     # silu(40) = 40, sigmoid(40) = 1
    W = {"p.q": np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0]]), "p.k": np.array([[1.0, 0, 0, 0], [0, 1.0, 0, 0]]),
         "p.v": np.array([[0, 0, 1.0, 0]]), "p.q.conv": np.ones((2, 1)), "p.k.conv": np.ones((2, 1)), "p.v.conv": np.ones((1, 1)),
         "p.b": np.array([[0, 0, 0, 1.0]]), "p.A_log": np.array([0.0]), "p.a": np.zeros((1, 4)), "p.dt_bias": np.array([0.0]),
         "p.g": np.array([[0, 0, 0, 1.0]]), "p.norm": np.array([2.0]), "p.o": np.array([[1.0]])}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "vdim": 1}
    h = np.array([[big, 0.0, big, big], [big, 0.0, 2 * big, big]])
    out = lp.gated_delta(W, "p.", h, m, 0.0)
    # a single value channel: o / rms(o) = +-1, times the weight 2, times silu(40) = 40
    assert np.allclose(np.abs(out), 80.0)
    # the state by hand: decay exp(-softplus(0)) = 1/2 per token, beta = 1, unit key (1, 0)
    S = 0.0
    for v in (big, 2 * big):
        S = 0.5 * S
        S = S + (v - S)
    assert np.isclose(S, 2 * big)


def test_general_delta_by_hand():
    # one head of two channels; r = k = (1, 0) on token 0 and (0, 1) on token 1, v = (3, 5) then (7, 11)
    eye = np.eye(6)
    W = {"p.r": eye[[0, 1]], "p.k": eye[[0, 1]], "p.v": eye[[2, 3]], "p.a": np.zeros((2, 6)), "p.a.b": np.array([50.0, 50.0]),
         "p.w1": np.zeros((1, 6)), "p.w2": np.zeros((2, 1)), "p.w0": np.array([-50.0, 50.0]), "p.g": np.zeros((2, 6)),
         "p.norm": np.ones(2), "p.o": np.eye(2)}
    m = {"heads": 1, "dim": 2}
    h = np.array([[1.0, 0, 3, 5, 0, 0], [1.0, 0, 7, 11, 0, 0]])
    out = lp.general_delta(W, "p.", h, m, 0.0)
    # token 0 writes row 0 = (3, 5). Token 1: row 0 decays by exp(-c * 0) = 1, then the whole of it is
    # removed along u = (1, 0) (a = 1), then (7, 11) is written: the read-out is (7, 11), normed, gate 1/2
    want = np.array([7.0, 11.0]) / np.sqrt((49 + 121) / 2) * 0.5
    assert np.allclose(out[1], want, atol=1e-5)
    # channel 1 decays by exp(-exp(-1/2)): write there and read it back one token later
    h = np.array([[0, 1.0, 3, 5, 0, 0], [1e-9, 1.0, 0, 0, 0, 0]])
    W2 = dict(W, **{"p.a.b": np.array([-50.0, -50.0])})          # nothing is removed
    S_row = np.array([3.0, 5.0]) * np.exp(-np.exp(-0.5))
    got = lp.general_delta(W2, "p.", h, m, 0.0)[1]
    assert np.allclose(got, S_row / np.sqrt((S_row ** 2).mean()) * 0.5, atol=1e-5)


def test_feed_forward_squares_the_relu():
    W = {"f.up": np.array([[1.0], [-1.0]]), "f.down": np.array([[1.0, 10.0]])}
    assert np.allclose(lp.feed_forward(W, "f.", np.array([[3.0], [-2.0]])), [[9.0], [40.0]])


def test_attention_alone_reads_exactly_its_window():
    # the delta-rule member silenced (its output norm's weight zero): what is left is the attention
    cfg, w = LD, dict(weights("LD"))
    w["l0.mix.right.out"] = np.zeros_like(w["l0.mix.right.out"])
    size = cfg["layers"][0]["mixer"]["left"]["mask"]["size"]
    toks = random_tokens("LD", 40, 1)
    base = lp.forward(cfg, w, toks)
    i = 30

    def changed(j):
        t = list(toks)
        t[j] = (t[j] + 7) % cfg["vocab"]
        return np.abs(lp.forward(cfg, w, t)[i] - base[i]).max()

    assert changed(i - size) == 0.0 and changed(i - size + 1) > 1e-6      # just outside, just inside the window
    assert changed(i + 1) == 0.0 and changed(i) > 1e-6


def test_values_are_the_keys_before_norm_and_rotation():
    # one key in the window of one position: the output is the gated, projected raw key of the token itself
    W = {"p.q": np.eye(2), "p.k": np.array([[0.0, 3.0], [4.0, 0.0]]), "p.q.norm": np.ones(2), "p.k.norm": np.ones(2) * 9.0,
         "p.temp": np.ones(1), "p.g": np.zeros((2, 2)), "p.o": np.eye(2)}
    m = {"heads": 1, "kv_heads": 1, "dim": 2, "scale": 1.0, "mask": {"size": 1}, "rot": {"base": 10.0, "dims": 2}}
    h = np.array([[1.0, 2.0], [5.0, 6.0]])
    out = lp.windowed_attention(W, "p.", h, m, 1e-5)
    assert np.allclose(out, (h @ W["p.k"].T) * 0.5)


# ------------------------------------------------------------------ configuration and loader
def test_configuration_errors_name_the_key():
    for drop, text in (("vocab", "'vocab'"), ("norm", "'norm.eps'"), ("embedding", "'embedding.scale'")):
        bad = {k: v for k, v in LA.items() if k != drop}
        with pytest.raises(ConfigError, match=text):
            read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    del bad["layers"][0]["mixer"]["left"]["scale"]
    with pytest.raises(ConfigError, match=r"layers\[0\]\.mixer\.left\.scale"):
        read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    bad["layers"][0]["type"] = "something"
    with pytest.raises(ConfigError, match="not a mixer of this design"):
        read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    bad["layers"][0]["mixer"]["left"]["vdim"] = 24
    with pytest.raises(ConfigError, match="values"):
        read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    bad["layers"][2]["weights_of"] = 1
    with pytest.raises(ConfigError, match="sizes differ"):
        read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    bad["layers"][4]["weights_of"] = 2                 # through layer 2 to layer 0, which is of the other kind
    with pytest.raises(ConfigError, match="sizes differ"):
        read_model_config(bad)
    for i, j, text in ((2, 2, "another layer"), (2, 9, "another layer")):
        bad = json.loads(json.dumps(LA))
        bad["layers"][i]["weights_of"] = j
        with pytest.raises(ConfigError, match=text):
            read_model_config(bad)
    bad = json.loads(json.dumps(LA))
    bad["layers"][0]["weights_of"] = 2
    with pytest.raises(ConfigError, match="back to itself"):
        read_model_config(bad)


def test_a_layer_may_name_a_later_layer_or_one_that_names_another(tmp_path):
    """The tensors are those of layer 2 alone: layer 0 names it, and layer 3 names layer 0."""
    from garuda_b200.weights import write_random_model
    from tests.helpers import folder_weights
    from tests.luvapel_cases import SHARPEN
    gd = {"type": "general_delta", "mixer": {"heads": 2, "dim": 8, "decay_rank": 3}, "mlp": {"kind": "dense", "ff": 24}}
    cfg = {"architecture": "Luvapel", "vocab": 61, "width": 24, "embedding": {"scale": 2.0}, "norm": {"eps": 1e-5},
           "layers": [dict(gd, weights_of=2), dict(LD["layers"][0]), gd, dict(gd, weights_of=0)]}
    cfg["layers"][1]["mixer"] = json.loads(json.dumps(LD["layers"][0]["mixer"]))
    _, model = build_model(cfg)
    assert [c.layer for c in model.spec.order] == [1, 0, 1, 1] and len(model.blocks) == 2
    assert not any(n.startswith(("l0.", "l3.")) for n in model.expected_tensors())
    d = write_random_model(str(tmp_path / "m"), cfg, 3, scale=SHARPEN)
    toks = np.random.default_rng(0).integers(0, 61, 30).tolist()
    ref = lp.forward(cfg, folder_weights(d), toks)
    e = Engine(d, dtype="float32", ops=CpuOps(), cuda_graphs=False, page_size=8, kv_tokens=128, context=64)
    got = e.step([StepEntry(1, toks[:17], range(17))]).numpy().copy()      # the next step writes the same buffer
    got = np.concatenate([got, e.step([StepEntry(1, toks[17:], range(13))]).numpy()])
    assert_close(got, ref, "float32", "layers that name other layers")


def test_run_order_and_cache_needs_come_from_the_configuration():
    _, model = build_model(LA)
    assert [c.layer for c in model.spec.order] == [0, 1, 0, 2, 1] and len(model.blocks) == 3
    # a layer that runs with another's tensors has pages and a state of its own
    assert [g.need for g in model.cache_groups] == [PagedKV(2, 16, 6, value_dim=16)]
    assert model.cache_groups[0].calls == ((0, 0), (2, 0))
    assert model.state_calls == [(0, 1), 1, (2, 1), 3, 4]
    assert model.need_at((0, 1)) == FixedState((4 * 12 * 20 + 2 * (2 * 2 * 12 + 4 * 20),))
    assert model.need_at(1) == FixedState((3 * 16 * 16,)) and model.need_at(3) == FixedState((2 * 24 * 24,))
    names = set(model.expected_tensors())
    assert "l0.mix.left.q.norm" in names and "l3.mix.w2" in names and not any(n.startswith(("l2.", "l4.")) for n in names)
    _, model = build_model(LB)
    assert [g.need for g in model.cache_groups] == [PagedKV(3, 8, None, value_dim=8)]


def test_the_decay_rank_comes_from_the_file(tmp_path):
    cfg = json.loads(json.dumps(LB))
    for layer in cfg["layers"]:
        layer["mixer"].pop("decay_rank", None)
    import shutil
    d = tmp_path / "m"
    shutil.copytree(model_dir("LB"), d)
    (d / "config.json").write_text(json.dumps(cfg))
    e = Engine(str(d), dtype="float32", ops=CpuOps(), cuda_graphs=False, page_size=8, kv_tokens=64, context=64)
    toks = random_tokens("LB", 9, 5)
    assert_close(e.step([StepEntry(1, toks, range(9))]).numpy(), plain_logits("LB", torch.float32, toks), "float32", "rank from the file")


def test_a_missing_tensor_is_reported(tmp_path):
    from garuda_b200.weights import SafetensorsFolder, write_safetensors
    f = SafetensorsFolder(model_dir("LB"))
    tensors = {n: f.tensor(n) for n in f.names() if n != "l1.mix.left.temp"}
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    (tmp_path / "m" / "config.json").write_text(json.dumps(LB))
    with pytest.raises(WeightError, match="l1.mix.left.temp"):
        Engine(str(tmp_path / "m"), dtype="float32", ops=CpuOps(), cuda_graphs=False)


# ------------------------------------------------------------------ the engine against the plain model
@pytest.mark.parametrize("name", ["LA", "LB", "LC", "LD"])
def test_whole_prompt(name):
    toks = random_tokens(name, 45, 2)
    e = engine(name)
    got = e.step([StepEntry(1, toks, range(len(toks)))]).numpy()
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} whole")


@pytest.mark.parametrize("name", ["LA", "LB"])
def test_token_by_token_from_the_first_token(name):
    toks = random_tokens(name, 40, 3)
    e = engine(name)
    got = np.stack([e.step([StepEntry(1, [t], [0])]).numpy()[0].copy() for t in toks])
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} token by token")


@pytest.mark.parametrize("name,cuts", [("LA", [2, 4, 5, 12, 13, 16, 24, 33, 35, 50]), ("LB", [1, 3, 8, 9, 17, 40, 50]),
                                       ("LD", [7, 9, 11, 26, 28, 50])])
def test_portions_cut_anywhere(name, cuts):
    toks = random_tokens(name, 50, 4)
    e = engine(name)
    rows, a = [], 0
    for b in cuts:
        rows.append(e.step([StepEntry(1, toks[a:b], range(b - a))]).numpy().copy())
        a = b
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", f"{name} in portions")


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again():
    name = "LA"
    e = engine(name, kv_tokens=72, max_concurrent=3)          # 9 pages of 8: a window of 6 holds two pages a request
    prompts = {i: random_tokens(name, n, 10 + i) for i, n in enumerate([60, 23, 41, 9, 37, 52])}
    at = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    live, waiting = [], list(prompts)
    rng = np.random.default_rng(0)
    while live or waiting:
        while waiting and len(live) < 3:
            live.append(waiting.pop(0))
        entries = []
        for i in live:
            n = int(rng.choice([1, 1, 2, 3, 7, 16]))
            n = min(n, len(prompts[i]) - at[i])
            entries.append(StepEntry(100 + i, prompts[i][at[i]:at[i] + n], range(n)))
        out = e.step(entries).numpy()
        row = 0
        for i, en in zip(list(live), entries):
            n = len(en.tokens)
            got[i].append(out[row:row + n].copy())
            row += n
            at[i] += n
            if at[i] == len(prompts[i]):
                e.runner.end(100 + i)
                live.remove(i)
        e.cache.manager.check_invariants()
    assert e.cache.manager.pages_reused > 0
    for i, toks in prompts.items():
        assert_close(np.concatenate(got[i]), plain_logits(name, torch.float32, toks), "float32", f"request {i} in a mixed batch")


def test_a_slot_used_again_starts_from_zero_state():
    name = "LB"                                               # no window: only the states can leak
    e = engine(name, max_concurrent=1)
    a, b = random_tokens(name, 30, 40), random_tokens(name, 17, 41)
    e.step([StepEntry(1, a, [])])
    e.runner.end(1)
    got = e.step([StepEntry(2, b, range(len(b)))]).numpy()
    assert_close(got, plain_logits(name, torch.float32, b), "float32", "the second user of a slot")


def test_long_decoding_after_a_prompt():
    name = "LA"
    toks = random_tokens(name, 120, 7)
    e = engine(name)
    rows = [e.step([StepEntry(1, toks[:20], range(20))]).numpy().copy()]
    rows += [e.step([StepEntry(1, [t], [0])]).numpy().copy() for t in toks[20:]]
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", "100 decoded tokens")


def test_greedy_generation_through_the_scheduler():
    name = "LA"
    e = engine(name, max_batch_tokens=16, prefill_chunk=8)
    prompts = [random_tokens(name, n, 20 + n) for n in (19, 5, 30)]
    results = e.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, r in zip(prompts, results):
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(lp.forward(LA, weights(name), seq)[-1])))
        assert r.tokens == seq[len(p):]
