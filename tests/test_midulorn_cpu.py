"""Midulorn on the CPU: the plain model's mechanisms one by one, and the engine (configuration,
loader, run order, pages and states, step function, scheduler) over the kernels' plain
references against the plain model."""
import json
import os

import numpy as np
import pytest
import torch

from garuda_b200 import Engine, SamplingParams, StepEntry, ConfigError, WeightError
from garuda_b200.config.registry import build_model, read_model_config
from garuda_b200.parts.base import FixedState, PagedKV, PagedLatent
from tests import helpers
from tests.midulorn_cases import CASES, MA, MB, MC, MD, model_dir, plain_logits, random_tokens, weights
from tests.plain import midulorn_plain as mp
from tests.plain.cpu_ops import CpuOps


def assert_close(got, want, dtype, what):
    """Against the 64-bit plain model, as a fraction of the largest logit: 32-bit sums in another
    order through up to six layers with sharpened weights."""
    scale = max(float(np.abs(want).max()), 1e-6)
    err = float(np.abs(np.asarray(got) - want).max())
    assert got.shape == want.shape and np.isfinite(got).all(), what
    helpers.OBSERVED[f"midulorn/{dtype}"] = max(helpers.OBSERVED.get(f"midulorn/{dtype}", 0.0), err / scale)
    assert err <= 5e-5 * scale, f"{what}: max difference {err:.3e} (limit {5e-5 * scale:.3e})"


def engine(name, **kw):
    kw.setdefault("page_size", 8)
    kw.setdefault("kv_tokens", 512)
    kw.setdefault("context", 256)
    return Engine(model_dir(name), dtype="float32", ops=CpuOps(), cuda_graphs=False, **kw)


# ------------------------------------------------------------------ the plain model's mechanisms
def test_rms_has_eps_inside_the_root():
    assert np.allclose(mp.rms(np.array([[3.0, 4.0]]), 1.0, 0.0), np.array([[3.0, 4.0]]) / np.sqrt(12.5))
    assert np.allclose(mp.rms(np.array([[2.0, 2.0]]), np.array([1.0, 3.0]), 5.0), [[2.0 / 3.0, 2.0]])


def test_xielu_by_hand():
    p, q = 0.3, -0.2
    ap, an = np.log1p(np.exp(p)), 0.5 + np.log1p(np.exp(q))
    z = np.array([2.0, 0.0, -1.5])
    want = [ap * 4.0 + 1.0, 0.0, an * (np.exp(-1.5) - 1.0 + 1.5) - 0.75]
    assert np.allclose(mp.xielu(z, p, q), want)


def test_rotation_pairs_a_channel_with_the_one_half_the_width_on():
    v = np.arange(1.0, 7.0).reshape(1, 6).repeat(2, 0)
    out = mp.rotate_half(v, [0, 3], 100.0, 4)
    assert np.allclose(out[0], v[0])                                   # position 0 turns nothing
    a0, a1 = 3.0, 3.0 * 100.0 ** -0.5                                   # the pairs' angles at position 3
    assert np.allclose(out[1, [0, 2]], [np.cos(a0) - 3 * np.sin(a0), 3 * np.cos(a0) + np.sin(a0)])
    assert np.allclose(out[1, [1, 3]], [2 * np.cos(a1) - 4 * np.sin(a1), 4 * np.cos(a1) + 2 * np.sin(a1)])
    assert np.allclose(out[1, 4:], [5.0, 6.0])                          # beyond the rotated width


def test_short_convolution_is_causal_and_starts_from_zeros():
    x = np.arange(1.0, 6.0)[:, None] * np.array([[1.0, 10.0]])
    taps = np.array([[0.5, 0.0, 2.0], [0.0, 1.0, 0.0]])                # the last column weighs the current token
    y = mp.causal_conv(x, taps)
    assert np.allclose(y[:, 0], [2.0, 4.0, 6.5, 9.0, 11.5]) and np.allclose(y[:, 1], [0.0, 10.0, 20.0, 30.0, 40.0])


def test_sink_counts_once_unscaled_and_has_no_value():
    s = np.array([[0.0, np.log(2.0), -np.inf]])
    p = mp.softmax_sink(s, np.log(5.0))
    assert np.allclose(p, [[1 / 8, 2 / 8, 0.0]])


def test_min_gru_by_hand():
    W = {"z": np.array([[1.0], [0.0]]), "z.b": np.array([0.0, 100.0]), "x": np.array([[2.0], [-1.0]]), "x.b": np.zeros(2),
         "g": np.array([[0.0], [0.0]]), "o": np.eye(2)}
    W["g"] = np.array([[1.0], [1.0]])
    h = np.array([[1.0], [-1.0]])
    out = mp.min_gru(W, "", h)
    sg = lambda z: 1 / (1 + np.exp(-z))
    z0, z1 = sg(1.0), sg(-1.0)
    s_a = [z0 * 2.5]                                                    # channel 0: candidates 2 + 1/2, sigmoid(-2)
    s_a.append((1 - z1) * s_a[0] + z1 * sg(-2.0))
    s_b = [sg(-1.0), 1.5]                                               # channel 1: the gate is one, the state is the candidate
    silu = [1.0 * sg(1.0), -1.0 * sg(-1.0)]
    assert np.allclose(out[:, 0], [s_a[0] * silu[0], s_a[1] * silu[1]]) and np.allclose(out[:, 1], [s_b[0] * silu[0], s_b[1] * silu[1]])


def test_router_weighs_by_the_softmax_over_all_experts_not_renormalized():
    d = 3
    W = {"router": np.array([[2.0, 0, 0], [1.0, 0, 0], [0.0, 0, 0]])}
    for e in range(3):
        W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"] = np.eye(d) * 10, np.eye(d), np.eye(d) * (e + 1)
    h = np.array([[1.0, 0.0, 0.0]])
    s = np.exp([2.0, 1.0, 0.0]) / np.exp([2.0, 1.0, 0.0]).sum()
    silu10 = 10.0 / (1 + np.exp(-10.0))
    assert np.allclose(mp.routed_ff(W, "", 3, 2, h)[0, 0], s[0] * silu10 * 1 + s[1] * silu10 * 2)


def test_attention_alone_reads_exactly_its_own_stretch():
    toks = random_tokens("MC", 30, 1)
    ref = mp.forward(MC, weights("MC"), toks)
    other = list(toks)
    other[17] = (toks[17] + 1) % MC["vocab"]                             # stretches of 9: 18..26 do not see 17
    alt = mp.forward(MC, weights("MC"), other)
    assert np.array_equal(alt[18:], ref[18:]) and not np.allclose(alt[17], ref[17])
    other = list(toks)
    other[18] = (toks[18] + 1) % MC["vocab"]
    alt = mp.forward(MC, weights("MC"), other)
    assert np.abs(alt[26] - ref[26]).max() > 1e-9 and np.array_equal(alt[27:], ref[27:]) and np.array_equal(alt[:18], ref[:18])


# ------------------------------------------------------------------ configuration, tensors, cache needs
def test_configuration_errors_name_the_key():
    def broken(change):
        cfg = json.loads(json.dumps(MB))
        change(cfg)
        return cfg
    cases = [(lambda c: c.pop("postln_alpha"), "postln_alpha"), (lambda c: c["layers"][1]["mixer"].pop("kv_heads"), "layers[1].mixer.kv_heads"),
             (lambda c: c["layers"][0]["mixer"]["rot"].pop("base"), "layers[0].mixer.rot.base"),
             (lambda c: c["layers"][1]["mlp"]["router"].pop("top"), "layers[1].mlp.router.top"),
             (lambda c: c["layers"][2]["mixer"].pop("width"), "layers[2].mixer.width"),
             (lambda c: c["layers"][3].update(type="window"), "layers[3].type"),
             (lambda c: c["layers"][0]["mlp"].update(kind="glu"), "layers[0].mlp.kind"),
             (lambda c: c.pop("logit_scale"), "logit_scale")]
    for change, key in cases:
        with pytest.raises(ConfigError, match=key.replace("[", r"\[").replace("]", r"\]")):
            read_model_config(broken(change))
    with pytest.raises(ConfigError, match="kv_heads"):
        read_model_config(broken(lambda c: c["layers"][1]["mixer"].update(heads=5)))
    with pytest.raises(ConfigError, match="rot.dims"):
        read_model_config(broken(lambda c: c["layers"][0]["mixer"]["rot"].update(dims=18)))


def test_run_order_and_cache_needs_come_from_the_configuration():
    _, model = build_model(MA)
    assert len(model.spec.order) == 5
    needs = {g.need: g.calls for g in model.cache_groups}
    assert needs[PagedKV(2, 12, None, value_dim=20, chunk=12)] == ((0, 0),)
    assert needs[PagedKV(1, 12, None, value_dim=40, chunk=5)] == ((3, 0),)
    assert needs[PagedLatent(26, None)] == (1,)
    assert model.need_at((0, 1)) == FixedState((2 * (4 * 12 + 2 * 12 + 2 * 20),)) and model.need_at(2) == FixedState((44,))
    assert model.need_at((3, 1)) == FixedState((1 * (2 * 12 + 12 + 40),))
    names = set(model.expected_tensors())
    assert {"l0.mix.q.conv", "l0.mix.vmix", "l1.mix.sink", "l1.mix.g", "l2.mix.z.b", "l3.mlp.e3.down", "l4.mlp.act", "final.norm"} <= names
    assert "head" not in names and "l2.norm2" not in names
    _, model = build_model(MB)
    # no convolution: pages only; no mask: every position stays
    assert model.need_at(3) == PagedKV(2, 32, None, value_dim=64, chunk=24) and model.need_at((4, 0)) == PagedKV(2, 64, None, value_dim=32)


def test_the_first_layer_with_mixed_values_is_their_source():
    _, model = build_model(MD)
    kinds = [b.mixer.value_mix for b in model.blocks if hasattr(b.mixer, "value_mix")]
    assert kinds == ["source", "mix", "mix"]
    _, model = build_model(MB)
    assert [b.mixer.value_mix for b in model.blocks if hasattr(b.mixer, "value_mix")] == [None, "source", None]


def test_a_missing_tensor_is_reported(tmp_path):
    from garuda_b200.weights import SafetensorsFolder, write_safetensors
    f = SafetensorsFolder(model_dir("MA"))
    tensors = {n: f.tensor(n) for n in f.names() if n != "l1.mix.sink"}
    os.makedirs(tmp_path / "m")
    write_safetensors(str(tmp_path / "m" / "model.safetensors"), tensors)
    (tmp_path / "m" / "config.json").write_text(json.dumps(MA))
    with pytest.raises(WeightError, match="l1.mix.sink"):
        Engine(str(tmp_path / "m"), dtype="float32", ops=CpuOps(), cuda_graphs=False)


def test_chunked_groups_give_back_the_stretches_in_front():
    host = helpers  # noqa: F841  (the host module is loaded through the engine below)
    e = engine("MC", kv_tokens=64)
    toks = random_tokens("MC", 40, 3)
    e.step([StepEntry(1, toks[:30], [])])
    m = e.cache.manager
    # stretches of 9, pages of 8: at length 30 the live stretch starts at 27, so pages 0..2 are back
    assert m.free_pages(0) == 8 - 1
    e.step([StepEntry(1, toks[30:36], [])])                               # 36 = 4 * 9: the next query starts a stretch
    assert m.free_pages(0) == 8 - 1
    e.step([StepEntry(1, toks[36:37], [])])
    m.check_invariants()
    assert m.free_pages(0) == 8 - 1 and m.pages_reused >= 0


# ------------------------------------------------------------------ the engine against the plain model
@pytest.mark.parametrize("name", ["MA", "MB", "MC", "MD"])
def test_whole_prompt(name):
    toks = random_tokens(name, 45, 2)
    e = engine(name)
    got = e.step([StepEntry(1, toks, range(len(toks)))]).numpy()
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} whole")


def test_the_residual_after_every_layer():
    toks = random_tokens("MA", 20, 6)
    e = engine("MA")
    seen = []
    e.runner.layer_probe = lambda i, x: seen.append(x.clone().numpy())
    e.step([StepEntry(1, toks, [])])
    want = []
    mp.forward(MA, weights("MA"), toks, want)
    assert len(seen) == len(want) == 5
    for i, (a, b) in enumerate(zip(seen, want)):
        assert np.abs(a - b).max() <= 2e-5 * np.abs(b).max(), f"layer {i}"


@pytest.mark.parametrize("name", ["MA", "MD"])
def test_token_by_token_from_the_first_token(name):
    toks = random_tokens(name, 40, 3)
    e = engine(name)
    got = np.stack([e.step([StepEntry(1, [t], [0])]).numpy()[0].copy() for t in toks])
    assert_close(got, plain_logits(name, torch.float32, toks), "float32", f"{name} token by token")


@pytest.mark.parametrize("name,cuts", [("MA", [2, 4, 5, 12, 13, 16, 24, 33, 35, 50]), ("MB", [1, 3, 8, 9, 17, 40, 50]),
                                       ("MD", [7, 9, 11, 26, 28, 33, 35, 50])])
def test_portions_cut_anywhere(name, cuts):
    toks = random_tokens(name, 50, 4)
    e = engine(name)
    rows, a = [], 0
    for b in cuts:
        rows.append(e.step([StepEntry(1, toks[a:b], range(b - a))]).numpy().copy())
        a = b
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", f"{name} in portions")


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again():
    name = "MA"
    e = engine(name, kv_tokens=136, max_concurrent=3)          # 17 pages of 8 for three requests of up to 60 tokens
    prompts = {i: random_tokens(name, n, 10 + i) for i, n in enumerate([60, 23, 41, 9, 37, 52])}
    at = {i: 0 for i in prompts}
    got = {i: [] for i in prompts}
    live, waiting = [], list(prompts)
    rng = np.random.default_rng(0)
    while live or waiting:
        while waiting and len(live) < 3 and sum(-(-len(prompts[i]) // 8) for i in live + waiting[:1]) <= 17:
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
    name = "MD"
    e = engine(name, max_concurrent=1)
    a, b = random_tokens(name, 30, 40), random_tokens(name, 17, 41)
    e.step([StepEntry(1, a, [])])
    e.runner.end(1)
    got = e.step([StepEntry(2, b, range(len(b)))]).numpy()
    assert_close(got, plain_logits(name, torch.float32, b), "float32", "the second user of a slot")


def test_long_decoding_after_a_prompt():
    name = "MA"
    toks = random_tokens(name, 120, 7)
    e = engine(name)
    rows = [e.step([StepEntry(1, toks[:20], range(20))]).numpy().copy()]
    rows += [e.step([StepEntry(1, [t], [0])]).numpy().copy() for t in toks[20:]]
    assert_close(np.concatenate(rows), plain_logits(name, torch.float32, toks), "float32", "100 decoded tokens")


def test_greedy_generation_through_the_scheduler():
    name = "MA"
    e = engine(name, max_batch_tokens=16, prefill_chunk=8)
    prompts = [random_tokens(name, n, 20 + n) for n in (19, 5, 30)]
    results = e.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12))
    for p, r in zip(prompts, results):
        seq = list(p)
        for _ in range(12):
            seq.append(int(np.argmax(mp.forward(MA, weights(name), seq)[-1])))
        assert r.tokens == seq[len(p):]
