"""Silupel on the GPU: each mechanism's kernels alone against the plain implementation's functions, then the engine under
every way of cutting the work, pages and slots used again, keys just inside and just outside every chunk in prompts and in
decoding, far keys, long decoding, and greedy generation through the entry point and the trace program."""
import copy
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_silupel as plain
import traces
from silupel_util import BLOCKS, CONFIGS, att, gru, lat, layer, make_folder, model, plain_logits, requests

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
# two runs of the engine against each other; in bfloat16 they take different kernels (prompt tiles, short portions, single
# tokens), each of which is within TOL of the exact result after eight layer runs
SELF_TOL = {"float32": 4e-5, "bfloat16": 2e-2}
KTOL = {"float32": 3e-6, "bfloat16": 8e-3}          # one kernel's output against float64


def K():
    from hfcpu_b200 import kernels
    return kernels


def dev(a, dtype=torch.float32):
    return torch.as_tensor(np.asarray(a), dtype=torch.float64).to(dtype).to(DEV).contiguous()


def f64(t):
    return t.double().cpu().numpy()


def rel(a, b):
    b = torch.as_tensor(np.asarray(b), dtype=torch.float64)
    return float((a.double().cpu() - b).abs().max() / b.abs().max().clamp_min(1e-30))


def rng(seed):
    return np.random.default_rng(seed)


def step_ctx(parts):
    """The step's index arrays for [(slot, number of tokens)]."""
    lens = [n for _, n in parts]
    return SimpleNamespace(token_seq=torch.tensor(np.repeat(np.arange(len(parts)), lens), dtype=torch.int32, device=DEV),
                           cu_tokens=torch.tensor(np.cumsum([0] + lens), dtype=torch.int32, device=DEV),
                           seq_slots=torch.tensor([s for s, _ in parts], dtype=torch.int32, device=DEV), num_seqs=len(parts))


# ---- each mechanism alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("E", [72, 256, 44, 1000, 3])
def test_layer_norm(dtype, E):
    """Rows with a large common offset: the variance must come from the deviations, not from the mean of the squares."""
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.parts import make_part
    dt, r = DT[dtype], rng(E)
    norm = make_part("norm", PartSpec("layernorm", {"size": E, "eps": 3e-5, "tensor": "n"}))
    w = dev(r.uniform(0.5, 1.5, E), dt)
    norm.bind({"n": w}, dt, torch.device(DEV))
    x = dev(3 * r.standard_normal((70, E)) + 40.0 * r.standard_normal((70, 1)))
    out = torch.empty(70, E, dtype=dt, device=DEV)
    norm.forward(x, out)
    assert rel(out, plain.layer_norm(f64(x), f64(w), 3e-5)) < (2e-4 if dtype == "float32" else KTOL[dtype])
    rows = torch.tensor([69, 0, 33], dtype=torch.int32, device=DEV)
    some = torch.empty(3, E, dtype=dt, device=DEV)
    norm.forward(x, some, rows=rows)
    assert torch.equal(some, out[rows.long()])
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("center", [True, False])
@pytest.mark.parametrize("E", [72, 256, 44])
def test_norm_with_token_shift_across_steps(dtype, center, E):
    """Three requests over three slots, cut differently: whole, in portions with a single token between, and token by
    token; then a new request in a freed slot, which must start from zeros."""
    dt, r, eps = DT[dtype], rng(E + center), 1e-5
    w, mu = dev(r.uniform(0.5, 1.5, E)), dev(r.uniform(-0.3, 1.2, E))
    state = torch.zeros(3, E, dtype=torch.float32, device=DEV)
    xs = {s: 2 * r.standard_normal((n, E)) + 1.0 for s, n in ((0, 9), (1, 9), (2, 5))}
    norm = plain.layer_norm if center else plain.rms_norm
    want = {s: plain.token_shift(norm(x, f64(w), eps), f64(mu)) for s, x in xs.items()}
    got = {s: [] for s in xs}
    cuts = [[(0, 0, 9), (1, 0, 4), (2, 0, 1)], [(2, 1, 2), (1, 4, 5)], [(1, 5, 9), (2, 2, 3)], [(2, 3, 4)], [(2, 4, 5)]]
    for cut in cuts:
        x = dev(np.concatenate([xs[s][a:b] for s, a, b in cut]))
        out = torch.empty(x.shape[0], E, dtype=dt, device=DEV)
        K().norm_shift(x, w, eps, center, mu, state, step_ctx([(s, b - a) for s, a, b in cut]), out)
        o = 0
        for s, a, b in cut:
            got[s].append(out[o:o + b - a])
            o += b - a
    for s in xs:
        assert rel(torch.cat(got[s]), want[s]) < (1e-5 if dtype == "float32" else KTOL[dtype]), s
    assert rel(state[1], norm(xs[1][-1:], f64(w), eps)[0]) < 1e-5                # what is left is the unshifted row
    state[0].zero_()                                                               # the slot is handed out again
    x = dev(xs[1][:3])
    out = torch.empty(3, E, dtype=dt, device=DEV)
    K().norm_shift(x, w, eps, center, mu, state, step_ctx([(0, 3)]), out)
    assert rel(out, want[1][:3]) < (1e-5 if dtype == "float32" else KTOL[dtype])
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("W,E", [(100, 72), (256, 256), (44, 44), (40, 136)])
def test_mingru_whole_against_cut(dtype, W, E):
    """The mixer part on one request whole, and on the same request in portions beside another request's single tokens: both
    branches of the candidate occur, gates cover (0, 1), and the state passes from step to step through the slot."""
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    from hfcpu_b200.parts import make_part
    dt, r = DT[dtype], rng(W + E)
    part = make_part("mixer", PartSpec("mingru", {"hidden_size": E, "width": W, "prefix": "m"}))
    tensors = {s.name: dev((1.0 if s.name.endswith(".b") else 0.35) * r.standard_normal(s.shape), dt) for s in part.tensor_specs()}
    part.bind(tensors, dt, torch.device(DEV))
    Wd = {k: f64(v) for k, v in tensors.items()}
    n = 75
    h = {s: dev(r.standard_normal((n, E)), dt) for s in (0, 1)}
    want = {s: plain.mingru({"width": W}, Wd, "m", f64(h[s])) for s in h}
    ws = Workspace(torch.device(DEV))
    state = torch.zeros(2, *part.state_spec().shape, dtype=torch.float32, device=DEV)
    got = {s: [] for s in h}
    at = {0: 0, 1: 0}
    for k, size in enumerate([1, 33, 2, 1, 31, 7]):
        cut = [(0, at[0], at[0] + size)] + ([(1, at[1], at[1] + 1)] if k else [])
        ctx = step_ctx([(s, b - a) for s, a, b in cut])
        ctx.buf, ctx.run_dtype = ws.get, dt
        xn = torch.cat([h[s][a:b] for s, a, b in cut])
        y = torch.zeros(xn.shape[0], E, dtype=torch.float32, device=DEV)
        part.forward(ctx, xn, y, None, state, True)
        o = 0
        for s, a, b in cut:
            got[s].append(y[o:o + b - a].clone())
            o += b - a
            at[s] = b
    assert at[0] == n
    assert rel(torch.cat(got[0]), want[0]) < (2e-5 if dtype == "float32" else 2e-2)
    assert rel(torch.cat(got[1]), want[1][:at[1]]) < (2e-5 if dtype == "float32" else 2e-2)
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(1, 72, 100), (5, 256, 512), (8, 2048, 1024), (130, 256, 320), (3, 44, 24), (2, 5000, 64)])
def test_product_tail_with_layer_norm_and_shift(dtype, shape):
    """The last product of a sublayer with what follows it in one call: the sum with the stream, the layer norm of the new
    stream, and, for steps of single tokens, the shift by each request's previous row with the slot's update; two such
    steps in a row over slots in scrambled order."""
    M, N, Kd = shape
    dt, r, eps = DT[dtype], rng(sum(shape)), 1e-5
    a, w, bias = dev(r.standard_normal((M, Kd)), dt), dev(0.2 * r.standard_normal((N, Kd)), dt), dev(r.standard_normal(N), dt)
    nw, mu = dev(r.uniform(0.5, 1.5, N)), dev(r.uniform(-0.3, 1.2, N))
    res = dev(r.standard_normal((M, N)) + 3.0)
    want_res = f64(res) + f64(a) @ f64(w).T + f64(bias)
    want_h = plain.layer_norm(want_res, f64(nw), eps)
    out_res, xn = res.clone(), torch.empty(M, N, dtype=dt, device=DEV)
    K().linear_residual_norm(a, w, bias, out_res, nw, eps, xn, center=True)
    tol = 2e-5 if dtype == "float32" else 2e-2
    assert rel(out_res, want_res) < tol and rel(xn, plain.layer_norm(f64(out_res), f64(nw), eps)) < (1e-5 if dtype == "float32" else KTOL[dtype])
    slots = r.permutation(M + 2)[:M]
    state = dev(r.standard_normal((M + 2, N)))
    before = f64(state)
    seq_slots = torch.tensor(slots, dtype=torch.int32, device=DEV)
    out_res = res.clone()
    K().linear_residual_norm(a, w, bias, out_res, nw, eps, xn, center=True, shift=(mu, state, seq_slots))
    h = plain.layer_norm(f64(out_res), f64(nw), eps)
    assert rel(xn, h + (before[slots] - h) * f64(mu)) < (1e-5 if dtype == "float32" else KTOL[dtype])
    assert rel(state[seq_slots.long()], h) < 1e-5 and float(np.abs(h - want_h).max() / np.abs(want_h).max()) < tol
    untouched = [s for s in range(M + 2) if s not in set(slots.tolist())]
    assert torch.equal(state[untouched].cpu(), torch.as_tensor(before[untouched], dtype=torch.float32))
    res2 = out_res.clone()
    K().linear_residual_norm(a, w, None, res2, nw, eps, xn, center=True, shift=(mu, state, seq_slots))
    h2 = plain.layer_norm(f64(res2), f64(nw), eps)
    assert rel(xn, h2 + (h - h2) * f64(mu)) < (2e-5 if dtype == "float32" else KTOL[dtype])
    K().check_device_errors()


def plain_scores_attend(q, k, v, positions, lo_of, scale, temp, cap, H, G):
    """q [n, H, d] at ``positions`` over keys k [m, G, d], values v [m, G, dv]; query i sees keys lo_of(pos) .. pos."""
    out = np.zeros((q.shape[0], H, v.shape[-1]))
    for i, pos in enumerate(positions):
        lo = lo_of(pos)
        for a in range(H):
            g = a // (H // G)
            s = (k[lo:pos + 1, g] @ q[i, a]) * scale * temp[a]
            if cap:
                s = cap * np.tanh(s / cap)
            out[i, a] = plain.softmax_rows(s[None])[0] @ v[lo:pos + 1, g]
    return out


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40), (8, 2, 64, 64), (4, 1, 128, 128), (4, 4, 64, 64), (3, 1, 20, 12)])
@pytest.mark.parametrize("cap", [0.0, 2.5, 40.0])
def test_score_factor_per_head_and_cap(dtype, geom, cap):
    """Raw scores of several times the cap, so that the cap matters, and factors of both signs; a prompt portion (the tiled
    prompt kernel where the sizes allow), a short portion behind it, and single tokens (the decode kernel), all over
    chunks of 48 positions."""
    from hfcpu_b200.kernels import attention_step_arrays, mask_code
    H, G, d, dv = geom
    dt, r = DT[dtype], rng(sum(geom) + int(cap))
    bs, n, chunk, scale = 16, 200, 48, 0.2
    pages = (n + bs - 1) // bs
    temp = r.uniform(0.6, 1.7, H) * np.where(np.arange(H) % 3 == 1, -1.0, 1.0)
    kd, vd = dev(1.5 * r.standard_normal((n, G, d)), dt), dev(r.standard_normal((n, G, dv)), dt)
    order = r.permutation(pages + 3)[:pages]
    kc = torch.zeros(pages + 3, bs, G, d, dtype=dt, device=DEV)
    vc = torch.zeros(pages + 3, bs, G, dv, dtype=dt, device=DEV)
    for p in range(n):
        kc[order[p // bs], p % bs], vc[order[p // bs], p % bs] = kd[p], vd[p]
    table = torch.full((1, pages + 2), -1, dtype=torch.int32, device=DEV)
    table[0, :pages] = torch.tensor(order, dtype=torch.int32)
    meta = SimpleNamespace(block_table=table, block_size=bs, max_blocks=pages + 2, group=0)
    hs = dev(temp)
    for first, count in ((0, 150), (150, 9), (159, 1), (199, 1)):
        positions = list(range(first, first + count))
        q = dev(1.5 * r.standard_normal((count, H, d)), dt)
        tiles = {kk: torch.tensor(vv, dtype=torch.int32, device=DEV) for kk, vv in attention_step_arrays([count], H // G).items()}
        ctx = SimpleNamespace(token_seq=torch.zeros(count, dtype=torch.int32, device=DEV), max_q_len=count, max_kv_len=first + count,
                              positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                              buf=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
        out = torch.empty(count, H * dv, dtype=dt, device=DEV)
        K().paged_attention(q.reshape(count, H * d), kc, vc, meta, ctx, H, G, d, mask_code(0, chunk), scale, out, tiles=tiles, dv=dv,
                            head_scales=hs, softcap=cap)
        want = plain_scores_attend(f64(q), f64(kd), f64(vd), positions, lambda p: p // chunk * chunk, scale, temp, cap, H, G)
        assert rel(out.view(count, H, dv), want) < (2e-5 if dtype == "float32" else 2e-2), (first, count)
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40, 8), (8, 2, 64, 64, 32), (4, 1, 128, 128, 128), (3, 3, 12, 20, 2)])
def test_attention_part_with_biases_gate_and_partial_rotation(dtype, geom):
    """The whole mixer on one prompt: biases on all four projections, rotation of a part of each head in the half-split
    layout with a stretched table, the factor per head, the cap, the chunk and the sigmoid gate."""
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    from hfcpu_b200.parts import make_part
    H, G, d, dv, nrot = geom
    dt, r, E, T, bs, chunk = DT[dtype], rng(sum(geom)), 72, 90, 8, 40
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv, "scale": 0.3, "softcap": 6.0, "mask": {"size": chunk},
         "rot": {"dims": nrot, "base": 900.0, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 32}}}
    rot = make_part("position", PartSpec("rotary", {"head_dim": d, "n_rot": nrot, "theta": 900.0, "pairing": "half",
                                                    "scaling": m["rot"]["scaling"]}))
    rot.prepare(256, torch.device(DEV))
    part = make_part("mixer", PartSpec("paged_attention", {
        "hidden_size": E, "num_heads": H, "num_kv_heads": G, "head_dim": d, "v_head_dim": dv, "scale": 0.3, "qkv_bias": True,
        "out_bias": True, "window": 0, "chunk": chunk, "softcap": 6.0, "head_scale_tensor": "temp",
        "out_gate": {"tensor": "g", "kind": "sigmoid"}, "position": "r", "prefix": "m",
        "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "bias_suffix": ".b"}), positions={"r": rot})
    tensors = {s.name: dev((1.0 if s.name.endswith(("temp", ".b")) else 0.35) * r.standard_normal(s.shape), dt) for s in part.tensor_specs()}
    assert sorted(tensors) == ["m.g", "m.k", "m.k.b", "m.o", "m.o.b", "m.q", "m.q.b", "m.temp", "m.v", "m.v.b"]
    part.bind(tensors, dt, torch.device(DEV))
    h = dev(r.standard_normal((T, E)), dt)
    want = plain.attention(m, {k: f64(v) for k, v in tensors.items()}, "m", f64(h))
    pages = (T + bs - 1) // bs
    cache = SimpleNamespace(k=torch.zeros(pages, bs, G, d, dtype=dt, device=DEV), v=torch.zeros(pages, bs, G, dv, dtype=dt, device=DEV), group=0)
    table = torch.arange(pages, dtype=torch.int32, device=DEV).view(1, pages)
    meta = SimpleNamespace(block_table=table, block_size=bs, max_blocks=pages, group=0, slots=torch.arange(T, dtype=torch.int32, device=DEV))
    tiles = {kk: torch.tensor(vv, dtype=torch.int32, device=DEV) for kk, vv in part.step_arrays(SimpleNamespace(q_lens=[T])).items()}
    ctx = SimpleNamespace(buf=Workspace(torch.device(DEV)).get, run_dtype=dt, positions=torch.arange(T, dtype=torch.int32, device=DEV),
                          token_seq=torch.zeros(T, dtype=torch.int32, device=DEV), max_q_len=T, max_kv_len=T,
                          group_meta=lambda g: meta, arrays=lambda key: tiles)
    y = torch.zeros(T, E, dtype=torch.float32, device=DEV)
    part.forward(ctx, h, y, cache, None, True)
    assert rel(y, want) < (3e-5 if dtype == "float32" else 2.5e-2)
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("shape", [(5, 72, 100), (130, 256, 512), (1, 44, 24), (300, 328, 392)])
def test_feed_forward_gated_with_tanh_gelu(dtype, shape):
    from hfcpu_b200.config import PartSpec
    from hfcpu_b200.engine.step import Workspace
    from hfcpu_b200.parts import make_part
    T, width, ff = shape
    r, dt = rng(sum(shape)), DT[dtype]
    part = make_part("ffn", PartSpec("gated", {"hidden_size": width, "intermediate_size": ff, "prefix": "m.mlp", "activation": "gelu_tanh",
                                               "names": {"gate": "gate", "up": "up", "down": "down"}}))
    tensors = {s.name: dev(0.3 * r.standard_normal(s.shape), dt) for s in part.tensor_specs()}
    part.bind(tensors, dt, torch.device(DEV))
    ctx = SimpleNamespace(buf=Workspace(torch.device(DEV)).get, run_dtype=dt)
    xn, res = dev(2 * r.standard_normal((T, width)), dt), dev(r.standard_normal((T, width)))
    want = f64(res) + plain.dense_ff({k: f64(v) for k, v in tensors.items()}, "m.mlp", f64(xn))
    out = res.clone()
    part.forward(ctx, xn, out)
    assert rel(out, want) < (2e-5 if dtype == "float32" else 2e-2)
    K().check_device_errors()


# ---- the engine -------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for i, (n, c) in enumerate(CONFIGS.items()):
        out[n] = make_folder(c, str(tmp_path_factory.mktemp(f"silupel_{n}")), 11 + i)
        out[n + "16"] = make_folder(c, str(tmp_path_factory.mktemp(f"silupel_{n}16")), 11 + i, torch.bfloat16)
    return out


LENGTHS = {"odd": [1, 19, 70, 130, 33], "wide": [3, 150, 64, 129, 260], "thin": [2, 9, 41]}
FAMILIES = {"whole": traces.whole, "tail": traces.tail_one_by_one, "portions": traces.portions, "mixed": traces.mixed}


def assert_rows(got, ref, tol, what="the plain implementation"):
    keys = sorted(got, key=lambda k: (str(k[0]), k[1]))
    errs = [float((got[k].double() - ref[k[0]][k[1]].double()).abs().max() / ref[k[0]][k[1]].double().abs().max()) for k in keys]
    over = [(k, e) for k, e in zip(keys, errs) if e > tol]
    assert not over, (f"{len(over)} of {len(keys)} rows differ from {what}; first: request {over[0][0][0]} position {over[0][0][1]} "
                      f"(error {over[0][1]:.3g})")


def engine_for(folder, block, dtype, max_tokens, max_requests=4):
    import hfcpu_b200
    m = hfcpu_b200.load_model(folder, DT[dtype], DEV)
    return hfcpu_b200.Engine(m, block_size=block, max_tokens=max_tokens, max_requests=max_requests, ctx_max=4096)


def check_clean(eng):
    K().check_device_errors()
    eng.cache.check()
    assert eng.cache.pages_in_use() == 0 and eng.slots.free_count == eng.max_requests


_WHOLE = {}


@pytest.mark.parametrize("family", list(FAMILIES))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(CONFIGS))
def test_cuttings_match_plain(folders, name, dtype, family):
    """Whole prompts, a tail decoded token by token, portions down to two tokens, and mixed batches of up to four requests
    in a pool sized for the peak, so that pages and slots are used again."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], LENGTHS[name], seed=3)
    steps = FAMILIES[family](reqs)
    eng = engine_for(folder, BLOCKS[name], dtype, traces.peak_tokens(steps, round_to=BLOCKS[name]))
    got = traces.run_in_process(eng, steps, check=eng.cache.check)
    check_clean(eng)
    ref = {r: plain_logits(folder, ids) for r, ids in reqs.items()}
    assert len(got) == sum(len(v) for v in reqs.values())
    assert_rows(got, ref, TOL[dtype])
    if family == "whole":
        _WHOLE[(name, dtype)] = got
    elif (name, dtype) in _WHOLE:
        base = _WHOLE[(name, dtype)]
        assert_rows(got, {r: torch.stack([base[(r, p)] for p in range(len(ids))]) for r, ids in reqs.items()}, SELF_TOL[dtype],
                    "the whole-prompt run")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_long_decoding(folders, name, dtype):
    """Every token a step of its own (from the second bfloat16 step on a replayed graph), two requests side by side, past
    several pages and chunks."""
    folder = folders[name if dtype == "float32" else name + "16"]
    reqs = requests(CONFIGS[name]["vocab"], [230, 75], seed=8)
    n = max(len(v) for v in reqs.values())
    steps = []
    for p in range(n):
        entries = [{"id": r, "tokens": [ids[p]], "want": [0], "_pos": p} for r, ids in reqs.items() if p < len(ids)]
        steps.append({"step": p, "entries": entries, "end": [r for r, ids in reqs.items() if p == len(ids) - 1]})
    eng = engine_for(folder, BLOCKS[name], dtype, 384)
    got = traces.run_in_process(eng, steps)
    check_clean(eng)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, TOL[dtype])


# Models of one layer: from its last position such a model sees exactly the tokens that its mixer lets through (and, through
# the token shift, nothing further back than the mixer does: the shift reaches one token back from each of them).
ONE_LAYER = {
    "chunk": lambda: model(150, 64, 1e-5, [layer(att(4, 2, 16, 24, 0.5, 24, 8, 100.0, 9.0), 48)]),
    "chunk_tiled": lambda: model(150, 64, 1e-5, [layer(att(4, 2, 64, 64, 0.3, 40, 32, 100.0, 9.0), 48)]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("which", list(ONE_LAYER))
def test_a_changed_token_shows_exactly_inside_the_chunk(tmp_path, which, dtype):
    """One token is changed at places around the edge of the last position's chunk: inside (and one before the chunk's first
    position, whose normed row the first key's shift reads) the logits must move as the plain implementation's do; further
    out they must not move at all.  The last tokens come as a portion and as single tokens."""
    cfg = ONE_LAYER[which]()
    size = cfg["layers"][0]["mixer"]["mask"]["size"]
    folder = make_folder(cfg, str(tmp_path / which), 21, DT[dtype], sharp=4.0)
    n = 3 * size + 5                                        # the last position is the chunk's sixth
    base = requests(150, [n], seed=2)["r0"]
    first = (n - 1) // size * size
    for place in (first - 2, first - 1, first, first + 1, n - 2):
        ids = list(base)
        ids[place] = (ids[place] + 71) % 150
        for tail in (1, 7):
            rows = []
            for seq in (base, ids):
                eng = engine_for(folder, 8, dtype, 256, max_requests=1)
                eng.add_request("a")
                import hfcpu_b200
                eng.step([hfcpu_b200.StepEntry("a", seq[:n - tail], [])])
                if tail == 1:
                    rows.append(eng.step([hfcpu_b200.StepEntry("a", seq[n - 1:], [0])])[0].float().cpu().clone())
                else:
                    rows.append(eng.step([hfcpu_b200.StepEntry("a", seq[n - tail:], [tail - 1])])[0].float().cpu().clone())
                eng.finish_request("a")
            moved = float((rows[0] - rows[1]).abs().max())
            want = plain_logits(folder, ids)[n - 1]
            assert float((rows[1].double() - want).abs().max() / want.abs().max()) < TOL[dtype]
            if place >= first - 1:
                assert moved > 1e-3, (place, tail)
            else:
                assert moved == 0.0, (place, tail)


def planted_folder(spec, folder, dtype, n, place, far, last):
    """A one-layer model of causal latent attention (no token shift) in which the key of token ``far`` at position ``place``
    is what the query of token ``last`` at position n - 1 looks for: the far token's embedding is made the direction that,
    through the projection of the rotated key part, lines up with the last query's rotated parts turned by the distance
    between the two positions."""
    cfg = model(150, 64, 1e-5, [layer(spec, 48)])
    m = spec["mixer"]

    def edit(t):
        W = {k: v.double().numpy() for k, v in t.items()}
        t["l0.shift"] = torch.zeros_like(t["l0.shift"])
        h_last = plain.layer_norm(W["embed"][last][None], W["l0.norm1"], 1e-5)
        cq = plain.rms_norm(h_last @ W["l0.mix.dq"].T, W["l0.mix.dq.norm"], 1e-5)
        q = (cq @ W["l0.mix.uq"].T).reshape(1, m["heads"], m["dim"] + m["rot_dim"])[..., m["dim"]:]
        u = plain.rotate_half_layout(q, [n - 1 - place], dict(m["rot"])).sum(1)[0]
        t["embed"][far] = torch.from_numpy(W["l0.mix.dkv"][m["kv_rank"]:].T @ u).float() * 50
    return make_folder(cfg, folder, 23, dtype, edit=edit, sharp=5.0)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mixer", ["latent", "latent_tiled"])
def test_a_far_key_is_found(tmp_path, mixer, dtype):
    """Hundreds of keys and one that stands out, far back, on both sides of page borders and right at the start: the last
    position's logits must be the plain implementation's, in which that key decides (taking the token away moves them by
    a large part of their size).  The last tokens come as a portion and as single tokens."""
    import hfcpu_b200
    spec = lat(4, 16, 8, 24, 32, 24, 0.5, 100.0) if mixer == "latent" else lat(4, 32, 16, 24, 32, 48, 0.4, 100.0)
    n = 420
    base = [t % 147 for t in requests(150, [n], seed=6)["r0"]]
    for place in (0, 1, 15, 16, 17, 255, 256, 300):
        folder = planted_folder(spec, str(tmp_path / f"{mixer}_{place}"), DT[dtype], n, place, 149, 148)
        ids = list(base)
        ids[place], ids[n - 1] = 149, 148
        want = plain_logits(folder, ids)[n - 1]
        without = list(ids)
        without[place] = 147
        assert float((plain_logits(folder, without)[n - 1] - want).abs().max()) > 0.2 * float(want.abs().max()), place
        for tail in (1, 5):
            eng = engine_for(folder, 16, dtype, 448, max_requests=1)
            eng.add_request("a")
            eng.step([hfcpu_b200.StepEntry("a", ids[:n - tail], [])])
            row = eng.step([hfcpu_b200.StepEntry("a", ids[n - tail:], [tail - 1])])[0].float().cpu()
            eng.finish_request("a")
            assert float((row.double() - want).abs().max() / want.abs().max()) < TOL[dtype], (place, tail)


def test_greedy_generation_through_the_entry_point(folders):
    import hfcpu_b200
    for name in ("odd", "wide"):
        folder = folders[name]
        sess = hfcpu_b200.Session(folder, dtype="float32", kv_block=BLOCKS[name], kv_pages=96, max_seqs=4,
                                  max_batched_tokens=48, batch=32, ctx_max=512)
        prompts = list(requests(CONFIGS[name]["vocab"], [7, 33, 1, 60], seed=2).values())
        out = sess.generate(prompts, temp=0, max_tokens=10)
        cfg, W = plain.read_folder(folder)
        for p, comps in zip(prompts, out):
            assert comps[0].tokens == plain.greedy(cfg, W, p, 10)
        assert sess.engine.cache.pages_in_use() == 0


def test_bfloat16_generation_replays_graphs(folders):
    """Steady decoding in bfloat16 goes through captured graphs (the shift's row and the recurrence's state included) and
    repeats itself; more requests than slots, so that slots are used again."""
    import hfcpu_b200
    sess = hfcpu_b200.Session(folders["wide16"], dtype="bfloat16", kv_block=16, kv_pages=128, max_seqs=2, ctx_max=512)
    prompts = list(requests(1032, [19, 130, 64, 5], seed=2).values())
    a = sess.generate(prompts, temp=0, max_tokens=24)
    assert sess.engine.use_graphs and any(s[0] == "ready" for s in sess.engine._graphs.values())
    b = sess.generate(prompts, temp=0, max_tokens=24)
    assert [c[0].tokens for c in a] == [c[0].tokens for c in b] and all(len(c[0].tokens) == 24 for c in a)
    # and they are the tokens of the plain implementation's first steps where it has a clear winner
    cfg, W = plain.read_folder(folders["wide16"])
    for got, p in zip(a, prompts):
        row = np.sort(plain.forward(cfg, W, p)[-1])
        if row[-1] - row[-2] > 0.5:
            assert got[0].tokens[0] == int(np.argmax(plain.forward(cfg, W, p)[-1]))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(folders, tmp_path, dtype):
    folder = folders["odd" if dtype == "float32" else "odd16"]
    reqs = requests(211, [1, 19, 70, 33, 50], seed=5)
    steps = traces.mixed(reqs)
    got = traces.run_trace_program(folder, dtype, steps, str(tmp_path), traces.peak_tokens(steps), 211, block_size=8)
    assert_rows(got, {r: plain_logits(folder, ids) for r, ids in reqs.items()}, TOL[dtype])


def test_command_line_generates(folders):
    import subprocess
    import sys
    from conftest import ROOT
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "hfb200"), "--model", folders["wide16"], "--op", "generate",
                        "--stdin-mode", "none", "--prompt-ids", "5,17,3,900", "--temp", "0", "--max-tokens", "6", "--ctx-max", "256",
                        "--kv-pages", "32"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "stop=length" in r.stdout or "length" in r.stdout
