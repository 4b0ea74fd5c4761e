"""Mokisun on a machine without a GPU: configuration and plan, the plain implementation's mechanisms against closed forms,
and the engine's host side (batching, pages behind windows, state slots handed out again) with the torch stand-in for the
CUDA library against the plain implementation."""
import copy

import numpy as np
import pytest
import torch

import plain_mokisun as plain
import traces
from mokisun_util import BLOCKS, CONFIGS, make_folder, plain_logits, requests


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {n: make_folder(c, str(tmp_path_factory.mktemp(f"mokisun_{n}")), 5 + i) for i, (n, c) in enumerate(CONFIGS.items())}


def test_plan_follows_the_layer_list():
    from hfcpu_b200.config import config_from_dict, MokisunConfig
    cfg = config_from_dict(CONFIGS["odd"])
    assert isinstance(cfg, MokisunConfig)
    plan = cfg.plan()
    assert plan.streams == 3
    assert [l.mixer.kind for l in plan.layers] == ["gated_linear_attention", "paged_attention", "parallel", "gated_linear_attention",
                                                   "parallel", "paged_attention"]
    assert all(l.block.kind == "hyper_residual" and l.block.args["streams"] == 3 for l in plan.layers)
    assert [l.ffn.kind if l.ffn else None for l in plan.layers] == ["moe", None, "moe", "moe", None, "moe"]
    assert [l.block.args["has_ffn"] for l in plan.layers] == [True, False, True, True, False, True]
    assert plan.layers[1].norm2 is None and plan.layers[0].norm1.kind == "dynamic_tanh"
    a = plan.layers[1].mixer.args
    assert a["sink"] == "learned" and a["window"] == 9 and a["v_head_dim"] == 40 and not a["values_are_keys"] and a["distance_slope_exp"] is None
    assert plan.layers[5].mixer.args["position"] is None and len(plan.positions) == 1
    left, ls = plan.layers[2].mixer.args["branches"][0]
    right, rs = plan.layers[2].mixer.args["branches"][1]
    assert (ls, rs) == (0.7, 1.3) and left.kind == "paged_attention" and right.kind == "gated_delta_rule"
    assert left.args["sink"] == "zero" and left.args["values_are_keys"] and left.args["distance_slope_exp"] == 8.0 and left.args["window"] == 13
    assert right.args["conv_taps"] == 3 and right.args["num_kv_heads"] == 2 and right.args["v_head_dim"] == 20
    f = plan.layers[0].ffn.args
    assert (f["experts"], f["identity"], f["top"], f["groups"], f["route_scale"]) == (5, 1, 2, (3, 2), 2.0)
    assert plan.layers[2].ffn.args["groups"] is None and plan.layers[2].ffn.args["identity"] == 0
    again = config_from_dict(cfg.to_dict())
    assert again.to_dict() == cfg.to_dict()
    assert config_from_dict(CONFIGS["thin"]).plan().streams == 1


def test_tensor_names():
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    specs = {s.name: s for s in build_model_specs(config_from_dict(CONFIGS["odd"]))}
    assert specs["embed"].shape == (211, 72) and specs["head"].shape == (211, 72) and specs["final.norm.alpha"].shape == ()
    assert specs["l0.mix.q"].shape == (72, 72) and specs["l0.mix.v"].shape == (120, 72) and specs["l0.mix.g"].shape == (120, 72)
    assert specs["l0.mix.a1"].shape == (5, 72) and specs["l0.mix.a2"].shape == (72, 5) and specs["l0.mix.a2.b"].shape == (72,)
    assert specs["l0.mix.norm"].shape == (40,) and specs["l0.mix.o"].shape == (72, 120)
    assert specs["l1.mix.sink"].shape == (6,) and specs["l1.mix.v"].shape == (120, 72) and "l1.norm2" not in specs
    assert "l2.mix.left.v" not in specs and "l2.mix.left.sink" not in specs and specs["l2.mix.left.k"].shape == (32, 72)
    assert specs["l2.mix.right.q"].shape == (48, 72) and specs["l2.mix.right.v"].shape == (80, 72)
    assert specs["l2.mix.right.q.conv"].shape == (48, 3) and specs["l2.mix.right.v.conv"].shape == (80, 3)
    assert specs["l2.mix.right.b"].shape == (4, 72) and specs["l2.mix.right.A_log"].shape == (4,)
    assert specs["l2.mix.right.dt_bias"].shape == (96,) and specs["l2.mix.right.a2"].shape == (96, 6)
    assert specs["l2.mix.right.g1"].shape == (7, 72) and specs["l2.mix.right.g2"].shape == (80, 7) and specs["l2.mix.right.norm"].shape == (20,)
    assert specs["l0.mlp.router"].shape == (6, 72) and specs["l0.mlp.correction"].shape == (6,) and "l0.mlp.e5.up" not in specs
    assert specs["l0.mlp.e4.down"].shape == (72, 40) and specs["l0.ls2"].shape == (72,)
    assert specs["l0.hc1.mix"].shape == (3, 3) and specs["l0.hc2.in"].shape == (3,) and "l1.hc2.in" not in specs and "l1.ls2" not in specs


@pytest.mark.parametrize("edit,word", [
    (lambda c: c["layers"][0].update(type="recurrent"), "not supported"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "not supported"),
    (lambda c: c["layers"][1]["mixer"].update(heads=7), "geometry"),
    (lambda c: c["layers"][1]["mixer"]["rot"].update(dims=7), "even"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(vdim=24), "vdim"),
    (lambda c: c["layers"][2]["mixer"]["left"].update(rot={"dims": 8, "base": 10.0}), "rotation"),
    (lambda c: c["layers"][2]["mixer"]["right"].update(kv_heads=3), "heads"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=7), "top"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][3]["mlp"]["router"]["groups"].update(keep=1), "groups"),
    (lambda c: c["layers"][0]["mixer"].pop("tau"), "tau"),
    (lambda c: c.pop("width"), "width"),
])
def test_bad_configurations_are_refused(edit, word):
    from hfcpu_b200.config import ConfigError, config_from_dict
    c = copy.deepcopy(CONFIGS["odd"])
    edit(c)
    with pytest.raises(ConfigError, match=word):
        config_from_dict(c)


# ---- the plain implementation's mechanisms against closed forms --------------------------------------
def test_plain_attention_sink_window_and_distance_bias():
    r = np.random.default_rng(0)
    q, k, v = r.normal(size=(7, 2, 4)), r.normal(size=(7, 1, 4)), r.normal(size=(7, 1, 3))
    sink = np.array([0.7, -1.2])
    o = plain.windowed_attention(q, k, v, 0.5, 3, sink)
    s = np.array([k[j, 0] @ q[5, 1] * 0.5 for j in (3, 4, 5)])
    p = np.exp(s) / (np.exp(s).sum() + np.exp(-1.2))
    assert np.allclose(o[5, 1], p @ v[3:6, 0])
    assert np.allclose(o[0, 0], v[0, 0] * np.exp(s0 := k[0, 0] @ q[0, 0] * 0.5) / (np.exp(s0) + np.exp(0.7)))
    # a sink of minus infinity is no sink; a window of one position sees itself only
    plainly = plain.windowed_attention(q, k, v, 0.5, 1, np.full(2, -np.inf))
    assert np.allclose(plainly[:, 0], v[:, 0]) and np.allclose(plainly[:, 1], v[:, 0])
    slopes = plain.distance_slopes(4)
    assert np.allclose(slopes, [0.25, 0.0625, 0.015625, 0.00390625])
    b = plain.windowed_attention(q, k, k, 1.0, 7, np.zeros(2), np.array([0.5, 2.0]))
    s = np.array([k[j, 0] @ q[6, 1] - 2.0 * (6 - j) for j in range(7)])
    assert np.allclose(b[6, 1], (np.exp(s) / (1 + np.exp(s).sum())) @ k[:, 0])


def test_plain_recurrences():
    r = np.random.default_rng(1)
    T, d, dv = 6, 3, 2
    q, k, v = r.normal(size=(T, 1, d)), r.normal(size=(T, 1, d)), r.normal(size=(T, 1, dv))
    # without decay and with beta = 1 and orthonormal keys the delta rule stores each value under its key exactly
    k[:3, 0] = np.eye(3)
    o = plain.delta_rule(k[:3], k[:3], v[:3], np.ones((3, 1)), np.ones((3, 1, d)))
    assert np.allclose(o, v[:3])
    # writing the same key twice replaces the value (beta = 1), and the read-out sees the token's own write
    kk = np.stack([k[0], k[0]])
    o = plain.delta_rule(kk, kk, v[:2], np.ones((2, 1)), np.ones((2, 1, d)))
    assert np.allclose(o[1], v[1])
    # the decay acts on key channels: a channel with decay 0 forgets
    g = np.ones((2, 1, d))
    g[1, 0, 0] = 0.0
    o = plain.delta_rule(np.stack([k[0], k[0]]), np.stack([k[0], k[1]]), v[:2], np.ones((2, 1)) * 0.0 + np.array([[1.0], [0.0]]), g)
    assert np.allclose(o[1], 0.0)
    # a short convolution: the last column is the current token's, zeros before the start
    x = np.arange(1.0, 6.0)[:, None]
    assert np.allclose(plain.short_convolution(x, np.array([[100.0, 10.0, 1.0]]))[:, 0], [1, 12, 123, 234, 345])


def test_plain_router_groups_identity_and_correction():
    W = {"r.router": np.eye(6) * 4.0, "r.correction": np.array([0.0, 0.0, 0.0, 0.0, 0.9, 0.0])}
    r = {"experts": 4, "identity": 2, "top": 2, "scale": 2.0, "groups": {"count": 3, "keep": 1}}
    h = np.zeros((3, 6))
    h[0, 1], h[1, 3], h[2, 0] = 1.0, 1.0, 1.0
    h[2, 2] = 0.9
    ids, w = plain.route(h, W, "r", r)
    s = np.exp(h * 4.0) / np.exp(h * 4.0).sum(-1, keepdims=True)
    # token 0: without the correction group 0 (expert 1) would win; the correction lifts output 4 and with it group 2,
    # the group of the identity experts; only that group's outputs can be chosen, and the weights are uncorrected scores
    assert sorted(ids[0]) == [4, 5] and np.allclose(sorted(w[0]), sorted(2.0 * s[0, [4, 5]]))
    # token 2: its two best outputs sit in groups 0 and 1, the correction still wins
    assert sorted(ids[2]) == [4, 5]
    W["r.correction"] = np.zeros(6)
    ids, w = plain.route(h, W, "r", r)
    assert sorted(ids[0]) == [0, 1] and sorted(ids[1]) == [2, 3] and sorted(ids[2]) == [0, 1]
    assert np.allclose(w.sum(-1) < 2.0, True)                       # not renormalized
    # identity experts hand the input through, weighted
    W.update({f"r.e{e}.{n}": np.zeros((6, 5) if n == "down" else (5, 6)) for e in range(4) for n in ("gate", "up", "down")})
    W["r.correction"] = np.array([0.0, 0.0, 0.0, 0.0, 0.9, 0.0])
    out = plain.feed_forward_moe(h, W, "r", {"router": r})
    assert np.allclose(out[0], 2.0 * (s[0, 4] + s[0, 5]) * h[0])


def test_plain_hyper_connections_with_one_copy_are_a_residual_sum():
    W = {"hc.in": np.array([1.0]), "hc.mix": np.array([[1.0]]), "hc.out": np.array([1.0]), "n": np.ones(4), "n.b": np.zeros(4),
         "n.alpha": np.array(1.0), "ls": np.full(4, 0.5)}
    X = np.random.default_rng(2).normal(size=(1, 3, 4))
    out = plain.hyper_step(X, W, "hc", lambda h: 2.0 * h, "n", "ls")
    assert np.allclose(out[0], X[0] + np.tanh(X[0]))
    W.update({"hc.in": np.array([1.0, 0.0]), "hc.mix": np.array([[0.0, 1.0], [1.0, 0.0]]), "hc.out": np.array([0.0, 2.0])})
    X = np.random.default_rng(3).normal(size=(2, 3, 4))
    out = plain.hyper_step(X, W, "hc", lambda h: 2.0 * h, "n", "ls")
    # mix is indexed [from, to]: the copies change places; the sublayer read copy 0 and wrote into copy 1
    assert np.allclose(out[0], X[1]) and np.allclose(out[1], X[0] + 2.0 * np.tanh(X[0]))


# ---- the engine's host side ------------------------------------------------------------------------
def test_pages_behind_windows_go_back_and_state_has_its_slots(emu, folders):
    import hfcpu_b200
    model = hfcpu_b200.load_model(folders["odd"], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=128, max_requests=2, ctx_max=128)
    by_window = {g.spec.window: g for g in eng.cache.groups}
    assert sorted(by_window) == [9, 13, 50, 50] or sorted(by_window) == [9, 13, 50]
    assert by_window[13].values is None and by_window[13].keys.shape[-2:] == (2, 16)          # values are the keys
    assert by_window[9].keys.shape[-1] == 24 and by_window[9].values.shape[-1] == 40
    assert not eng.can_fork                                     # a request cannot start on another's pages: its state is its own
    # state: layers 0 and 3 a matrix per head; layers 2 and 4 a matrix per head and the convolution's carried inputs
    shapes = {i: tuple(eng.slots.entry_state(i).shape) for i in range(6) if eng.slots.entry_state(i) is not None}
    assert shapes == {0: (2, 3 * 24 * 40), 2: (2, 4 * 24 * 20 + 2 * (2 * 2 * 24 + 4 * 20)), 3: (2, 2 * 40 * 24),
                      4: (2, 3 * 16 * 16 + 1 * (2 * 3 * 16 + 3 * 16))}
    eng.add_request("a")
    ids = requests(211, [100], seed=1)["r0"]
    eng.step([hfcpu_b200.StepEntry("a", ids[:61], [])])
    held = lambda g: [b for b, p in enumerate(g.tables["a"]) if p >= 0]
    # 61 tokens held; the next query is at 61: window 9 -> first key 53, window 13 -> 49, window 50 -> 12
    assert held(by_window[9]) == [6, 7] and held(by_window[13]) == [6, 7] and held(by_window[50]) == [1, 2, 3, 4, 5, 6, 7]
    assert all(float(eng.slots.entry_state(i)[0].abs().sum()) > 0 for i in shapes)
    eng.cache.check()
    eng.finish_request("a")
    assert eng.cache.pages_in_use() == 0


def test_a_slot_that_is_handed_out_again_starts_empty(emu, folders):
    import hfcpu_b200
    from hfcpu_b200 import StepEntry
    model = hfcpu_b200.load_model(folders["odd"], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=8, max_tokens=64, max_requests=1, ctx_max=64)
    ids = requests(211, [23, 17], seed=3)
    ref = {r: plain_logits(folders["odd"], v) for r, v in ids.items()}
    for r in ("r0", "r1", "r0"):
        eng.add_request(r)
        a = eng.step([StepEntry(r, ids[r][:5], [4])])[0].clone()
        b = eng.step([StepEntry(r, ids[r][5:6], [0])])[0].clone()
        c = eng.step([StepEntry(r, ids[r][6:], [len(ids[r]) - 7])])[0].clone()
        for got, p in ((a, 4), (b, 5), (c, len(ids[r]) - 1)):
            assert float((got.double() - ref[r][p]).abs().max() / ref[r][p].abs().max()) < 1e-4
        eng.finish_request(r)


@pytest.mark.parametrize("family", ["whole", "portions", "mixed", "one_by_one"])
@pytest.mark.parametrize("name", ["odd", "thin", "wide"])
def test_engine_host_side_matches_plain(emu, folders, name, family):
    import hfcpu_b200
    if name == "wide" and family != "mixed":
        pytest.skip("the large configuration runs the mixed trace only here")
    reqs = requests(CONFIGS[name]["vocab"], [1, 9, 37, 20, 2], seed=1)
    steps = {"whole": traces.whole, "portions": traces.portions, "mixed": traces.mixed, "one_by_one": traces.one_by_one}[family](reqs)
    model = hfcpu_b200.load_model(folders[name], torch.float32, "cpu")
    eng = hfcpu_b200.Engine(model, block_size=BLOCKS[name], max_tokens=traces.peak_tokens(steps), max_requests=4, ctx_max=256)
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == 4
    ref = {r: plain_logits(folders[name], ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    bad = traces.first_bad(got, ref, 2e-4)
    assert bad is None, f"first wrong row: request {bad[0]} position {bad[1]} (error {bad[2]:.3g})"


def test_greedy_generation_through_the_entry_point(emu, folders):
    import hfcpu_b200
    folder = folders["thin"]
    sess = hfcpu_b200.Session(folder, dtype="float32", device="cpu", kv_block=4, kv_pages=64, max_seqs=2, max_batched_tokens=16,
                              batch=8, ctx_max=128)
    prompts = list(requests(97, [7, 21, 1], seed=2).values())
    out = sess.generate(prompts, temp=0, max_tokens=6)
    cfg, W = plain.read_folder(folder)
    for p, comps in zip(prompts, out):
        assert comps[0].tokens == plain.greedy(cfg, W, p, 6)
    assert sess.engine.cache.pages_in_use() == 0
