"""Mokisun on the GPU: each mechanism's kernels alone against the plain implementation's functions, then the engine under
every way of cutting the work, pages and state slots used again, keys just inside and just outside every window in prompts
and in decoding, tokens far back that only the recurrent state remembers, long decoding, and greedy generation through
the entry point and the trace program."""
import copy
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import plain_mokisun as plain
import traces
from mokisun_util import BLOCKS, CONFIGS, att, gla, layer, make_folder, model, moe, par, plain_logits, requests

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}
TOL = {"float32": 2e-4, "bfloat16": 3e-2}
SELF_TOL = {"float32": 4e-5, "bfloat16": 1.5e-2}
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


def i32(a):
    return torch.tensor(a, dtype=torch.int32, device=DEV)


def step_ctx(lens, slots):
    """What the recurrent kernels read of a step: requests with ``lens`` tokens each, side by side, in state slots ``slots``."""
    cu = np.concatenate([[0], np.cumsum(lens)])
    seq = np.concatenate([np.full(n, i) for i, n in enumerate(lens)])
    return SimpleNamespace(token_seq=i32(seq.tolist()), cu_tokens=i32(cu.tolist()), seq_slots=i32(list(slots)), num_seqs=len(lens),
                           max_q_len=max(lens))


# ---- each mechanism alone ---------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("S,E,T", [(1, 44, 5), (2, 72, 33), (3, 256, 70), (8, 40, 3), (4, 1000, 9)])
def test_hyper_connection_passes(dtype, S, E, T):
    """The copies of the stream: spreading the embedding, reading them with weights through the norm, and the write-back
    from one or two sources in pieces, or from chosen experts among which some stand for the sublayer's input."""
    dt, r = DT[dtype], rng(S * E + T)
    emb = dev(r.standard_normal((T, E)))
    x = torch.empty(T, S * E, device=DEV)
    K().hc_spread(emb, x, S)
    assert torch.equal(x.view(T, S, E), emb[:, None, :].expand(T, S, E))
    X = r.standard_normal((S, T, E))
    x = dev(X.transpose(1, 0, 2).reshape(T, S * E))
    W = {"n": f64(dev(r.uniform(0.5, 1.5, E), dt)), "n.b": f64(dev(0.1 * r.standard_normal(E), dt)), "n.alpha": f64(dev(0.7, dt))}
    norm = (dev(W["n.alpha"], dt), dev(W["n"], dt), dev(W["n.b"], dt))
    a = r.uniform(0.3, 1.1, S)
    # read: every row with weights; chosen rows as the plain sum
    out = torch.empty(T, E, dtype=dt, device=DEV)
    K().hc_in_norm(x, S, dev(a), None, norm, out)
    assert rel(out, plain.dynamic_tanh(np.tensordot(f64(dev(a)), X, axes=(0, 0)), W, "n")) < KTOL[dtype]
    rows = [T - 1, 0, T // 2]
    out = torch.empty(3, E, dtype=dt, device=DEV)
    K().hc_in_norm(x, S, None, i32(rows), norm, out)
    assert rel(out, plain.dynamic_tanh(X.sum(0)[rows], W, "n")) < KTOL[dtype]
    total = torch.empty(3, E, device=DEV)
    K().hc_in_norm(x, S, None, i32(rows), None, total)
    assert rel(total, X.sum(0)[rows]) < 3e-6
    # write-back from two sources, the first in three pieces, with factors, and the next sublayer's input from the same pass
    B, d_out, c = r.uniform(-0.3, 1.0, (S, S)), r.uniform(0.4, 1.1, S), r.uniform(0.3, 1.2, E)
    y1, y2 = r.standard_normal((3, T, E)), r.standard_normal((1, T, E))
    nxt = r.uniform(0.3, 1.1, S)
    W.update({"hc.in": np.ones(S), "hc.mix": f64(dev(B)), "hc.out": f64(dev(d_out)), "ls": f64(dev(c, dt))})
    y = f64(dev(y1)).sum(0) * 0.7 + f64(dev(y2))[0] * 1.3
    want = np.tensordot(W["hc.mix"].T, X, axes=(1, 0)) + W["hc.out"][:, None, None] * (W["ls"] * y)
    xx, out = x.clone(), torch.empty(T, E, dtype=dt, device=DEV)
    K().hc_update(xx, S, [(dev(y1), 3, 0.7), (dev(y2), 1, 1.3)], None, dev(c, dt), dev(B), dev(d_out), dev(nxt), norm, out)
    assert rel(xx.view(T, S, E), want.transpose(1, 0, 2)) < 3e-6
    assert rel(out, plain.dynamic_tanh(np.tensordot(f64(dev(nxt)), want, axes=(0, 0)), W, "n")) < KTOL[dtype]
    # write-back from chosen experts; ids at or above n_real stand for the sublayer's input
    top, n_real = 3, 4
    ids = r.integers(0, 6, (T, top))
    wts, ey, h = r.uniform(0.1, 0.9, (T, top)), r.standard_normal((T * top, E)), r.standard_normal((T, E))
    hh = f64(dev(h, dt))
    pick = np.where((ids >= n_real)[..., None], hh[:, None, :], f64(dev(ey)).reshape(T, top, E))
    y = (f64(dev(wts))[..., None] * pick).sum(1)
    want = np.tensordot(W["hc.mix"].T, X, axes=(1, 0)) + W["hc.out"][:, None, None] * (W["ls"] * y)
    xx = x.clone()
    K().hc_update(xx, S, [], (dev(ey), dev(wts), i32(ids.tolist()), n_real, dev(h, dt)), dev(c, dt), dev(B), dev(d_out), None, None, None)
    assert rel(xx.view(T, S, E), want.transpose(1, 0, 2)) < 3e-6
    K().check_device_errors()


def paged(k, v, bs, dt, extra=3, seed=0):
    """Keys [n, G, d] (and values) scattered over pages in a shuffled order; returns caches and the block table."""
    n = k.shape[0]
    pages = (n + bs - 1) // bs
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(pages + extra, generator=g).tolist()[:pages]
    kc = torch.zeros(pages + extra, bs, *k.shape[1:], dtype=dt, device=DEV)
    kd = dev(k, dt)
    vc = vd = None
    if v is not None:
        vc = torch.zeros(pages + extra, bs, *v.shape[1:], dtype=dt, device=DEV)
        vd = dev(v, dt)
    for j in range(n):
        kc[perm[j // bs], j % bs] = kd[j]
        if v is not None:
            vc[perm[j // bs], j % bs] = vd[j]
    return kc, vc, kd, vd, torch.tensor([perm], dtype=torch.int32, device=DEV), pages


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [44, 1, 7, 64, 400, 1000])
@pytest.mark.parametrize("geom", [(6, 3, 24, 40, "learned"), (4, 2, 16, 16, "biased"), (8, 2, 64, 64, "learned"), (8, 2, 64, 64, "biased"),
                                  (4, 1, 128, 128, "learned"), (4, 4, 128, 128, "biased"), (3, 1, 32, 32, "zero")])
def test_window_edges_with_sinks_and_distance_bias(dtype, window, geom):
    """One key carries a score far above the rest; it is placed just inside and just outside the window of the last query
    (which comes in a portion of three and as a single token), on both sides of page borders and far away, and the
    output must follow it or ignore it.  "learned": a sink per head; "biased": values are the keys, a sink of zero and a
    bias linear in the distance; "zero": the sink of zero alone."""
    H, G, d, dv, form = geom
    dt, bs, n, scale = DT[dtype], 8, 431, 0.5
    last = n - 1
    lo = max(0, last - window + 1)
    slopes = plain.distance_slopes(H) if form == "biased" else None
    sink = rng(H).uniform(-2, 3, H) if form == "learned" else np.zeros(H)
    for planted in sorted({lo, lo - 1, max(lo - 2, 0), last, min(lo + 1, last), 0, bs - 1, bs, 7 * bs - 1, 7 * bs, 40 * bs - 1}):
        if planted < 0:
            continue
        r = rng(planted + window)
        k = 0.3 * r.standard_normal((n, G, d))
        q = np.zeros((n, H, d))
        q[-3:] = 0.1 * r.standard_normal((3, H, d))
        v = None if form == "biased" else r.standard_normal((n, G, dv))
        # the planted key: far above the rest in the last head, whose distance bias is the flattest
        k[planted] = 3.0
        q[-3:] += 16.0 / (3.0 * d * scale)
        kc, vc, kd, vd, bt, pages = paged(k, v, bs, dt, seed=planted)
        meta = SimpleNamespace(block_table=bt, block_size=bs, max_blocks=pages)
        kk = f64(kd)
        vv = kk if form == "biased" else f64(vd)
        qq = f64(dev(q, dt))
        want_all = plain.windowed_attention(qq, kk, vv, scale, window, sink, slopes, rows=[n - 3, n - 2, n - 1])
        for positions in ([n - 3, n - 2, n - 1], [n - 1]):
            qd = dev(q[positions], dt).reshape(len(positions), H * d).contiguous()
            ctx = SimpleNamespace(token_seq=torch.zeros(len(positions), dtype=torch.int32, device=DEV),
                                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV), max_q_len=len(positions))
            out = torch.empty(len(positions), H * dv, dtype=dt, device=DEV)
            extra = {"sinks": dev(sink)} if form == "learned" else {"zero_sink": True}
            if form == "biased":
                K().paged_attention(qd, kc, None, meta, ctx, H, G, d, window, scale, out, dv=dv, values_in_keys=True, slopes=dev(slopes), **extra)
            else:
                K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, window, scale, out, dv=dv, **extra)
            assert rel(out.view(-1, H, dv), want_all[positions]) < (2e-5 if dtype == "float32" else 2e-2), (planted, positions)
            seen = lo <= planted
            took = rel(out.view(-1, H, dv)[-1, H - 1], vv[planted, G - 1]) < 0.05
            assert took == seen, f"key {planted} ({'inside' if seen else 'outside'} [{lo}, {last}]) took={took}"
    K().check_device_errors()


@pytest.mark.parametrize("window", [44, 100, 129, 400, 1000])
@pytest.mark.parametrize("geom", [(8, 2, 64, "learned"), (8, 2, 64, "biased"), (4, 1, 128, "learned"), (16, 4, 128, "biased"), (4, 4, 64, "zero"),
                                  (16, 1, 128, "biased")])
def test_window_edges_with_sinks_and_distance_bias_tiled_kernels(window, geom):
    """The same for the kernels that serve whole steps in bfloat16 with head sizes 64 and 128: a prompt portion of 150
    tokens (tcgen05 tiles, two query tiles of which the second is short), one of 70, a short portion of 3 and a single
    token (the decode kernel, its keys split over several blocks), each with the engine's own tile lists."""
    from hfcpu_b200.kernels import attention_step_arrays
    H, G, d, form = geom
    dt, bs, n, scale = torch.bfloat16, 16, 431, 0.5
    last = n - 1
    lo = max(0, last - window + 1)
    slopes = plain.distance_slopes(H) if form == "biased" else None
    sink = rng(H + d).uniform(-2, 3, H) if form == "learned" else np.zeros(H)
    for planted in sorted({lo, lo - 1, last, 0, bs - 1, bs, 9 * bs - 1, 9 * bs}):
        if planted < 0:
            continue
        r = rng(planted + window + d)
        k = 0.3 * r.standard_normal((n, G, d))
        v = None if form == "biased" else r.standard_normal((n, G, d))
        k[planted] = 3.0
        kc, vc, kd, vd, bt, pages = paged(k, v, bs, dt, seed=planted)
        meta = SimpleNamespace(block_table=bt, block_size=bs, max_blocks=pages, group=0)
        kk = f64(kd)
        vv = kk if form == "biased" else f64(vd)
        for count in (150, 70, 3, 1):
            positions = list(range(n - count, n))
            q = np.zeros((n, H, d))
            q[positions] = 0.1 * r.standard_normal((count, H, d))
            q[-1] += 16.0 / (3.0 * d * scale)
            qd = dev(q[positions], dt).reshape(count, H * d).contiguous()
            qq = np.zeros((n, H, d))
            qq[positions] = f64(qd).reshape(count, H, d)
            tiles = {t: torch.tensor(a, dtype=torch.int32, device=DEV) for t, a in attention_step_arrays([count], H // G).items()}
            ctx = SimpleNamespace(token_seq=torch.zeros(count, dtype=torch.int32, device=DEV), max_q_len=count, max_kv_len=n,
                                  positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                                  buf=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
            out = torch.empty(count, H * d, dtype=dt, device=DEV)
            extra = {"sinks": dev(sink)} if form == "learned" else {"zero_sink": True}
            if form == "biased":
                K().paged_attention(qd, kc, None, meta, ctx, H, G, d, window, scale, out, tiles=tiles, dv=d, values_in_keys=True,
                                    slopes=dev(slopes), **extra)
            else:
                K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, window, scale, out, tiles=tiles, **extra)
            want = plain.windowed_attention(qq, kk, vv, scale, window, sink, slopes, rows=positions)
            assert rel(out.view(-1, H, d), want[positions]) < 2e-2, (planted, count)
            seen = lo <= planted
            took = rel(out.view(-1, H, d)[-1, H - 1], vv[planted, G - 1]) < 0.05
            assert took == seen, f"{count} tokens: key {planted} ({'inside' if seen else 'outside'} [{lo}, {last}]) took={took}"
    K().check_device_errors()


def test_a_large_sink_in_the_tiled_kernels():
    """A sink far above every score takes nearly all of the weight, one far below takes none: against the plain kernel of
    the same library, for a prompt portion and for single tokens of requests of unequal length in one step."""
    from hfcpu_b200.kernels import attention_step_arrays
    H, G, d, bs, scale, dt = 8, 2, 64, 16, 0.3, torch.bfloat16
    r = rng(77)
    lens = [300, 17, 129]
    for q_lens in ([1, 1, 1], [100, 1, 70]):
        ks = [0.5 * r.standard_normal((n, G, d)) for n in lens]
        pages_each = [(n + bs - 1) // bs for n in lens]
        total = sum(pages_each) + 2
        perm = torch.randperm(total, generator=torch.Generator().manual_seed(5)).tolist()
        kc = torch.zeros(total, bs, G, d, dtype=dt, device=DEV)
        vc = torch.zeros(total, bs, G, d, dtype=dt, device=DEV)
        table = torch.full((len(lens), max(pages_each)), -1, dtype=torch.int32)
        at = 0
        for i, n in enumerate(lens):
            for j in range(pages_each[i]):
                table[i, j] = perm[at]
                m = min(bs, n - j * bs)
                kc[perm[at], :m] = dev(ks[i][j * bs:j * bs + m], dt)
                vc[perm[at], :m] = dev(r.standard_normal((m, G, d)), dt)
                at += 1
        meta = SimpleNamespace(block_table=table.to(DEV), block_size=bs, max_blocks=table.shape[1], group=0)
        T = sum(q_lens)
        seq = [i for i, c in enumerate(q_lens) for _ in range(c)]
        positions = [lens[i] - c + j for i, c in enumerate(q_lens) for j in range(c)]
        qd = dev(r.standard_normal((T, H * d)), dt)
        tiles = {t: torch.tensor(a, dtype=torch.int32, device=DEV) for t, a in attention_step_arrays(q_lens, H // G).items()}
        ctx = SimpleNamespace(token_seq=i32(seq), max_q_len=max(q_lens), max_kv_len=max(lens), positions=i32(positions),
                              buf=lambda name, shape, dtype: torch.empty(shape, dtype=dtype, device=DEV))
        for sinks in (np.full(H, 30.0), np.full(H, -30.0), np.linspace(-4, 6, H)):
            tiled, simple = (torch.empty(T, H * d, dtype=dt, device=DEV) for _ in range(2))
            K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, 64, scale, tiled, tiles=tiles, sinks=dev(sinks))
            K().paged_attention(qd, kc, vc, meta, ctx, H, G, d, 64, scale, simple, sinks=dev(sinks))
            assert float((tiled.float() - simple.float()).abs().max()) < 2e-2 * max(float(simple.float().abs().max()), 1e-3)
            if sinks[0] == 30.0:
                assert float(tiled.float().abs().max()) < 1e-6
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_sink_takes_its_share(dtype):
    """With scores near zero a large sink leaves almost nothing for the keys and a very negative one changes nothing; the
    sink is not scaled and counts once, whatever the number of keys."""
    dt, H, G, d, n = DT[dtype], 4, 2, 16, 50
    r = rng(3)
    k, v = np.zeros((n, G, d)), r.standard_normal((n, G, d))
    kc, vc, kd, vd, bt, pages = paged(k, v, 8, dt)
    meta = SimpleNamespace(block_table=bt, block_size=8, max_blocks=pages)
    ctx = SimpleNamespace(token_seq=i32([0]), positions=i32([n - 1]), max_q_len=1)
    q = torch.zeros(1, H * d, dtype=dt, device=DEV)
    out = torch.empty(1, H * d, dtype=dt, device=DEV)
    sink = np.array([-30.0, 0.0, np.log(10.0), np.log(3.0 * 10)])
    K().paged_attention(q, kc, vc, meta, ctx, H, G, d, 10, 7.0, out, sinks=dev(sink))
    mean = f64(vd)[n - 10:].mean(0)                     # uniform weights over the window's ten keys
    share = 10.0 / (10.0 + np.exp(sink))
    want = np.stack([mean[h // 2] * share[h] for h in range(H)])
    assert rel(out.view(H, d), want) < (1e-5 if dtype == "float32" else 1e-2)
    K().paged_attention(q, kc, vc, meta, ctx, H, G, d, 10, 7.0, out, zero_sink=True)
    assert rel(out.view(H, d), np.stack([mean[h // 2] * 10.0 / 11.0 for h in range(H)])) < (1e-5 if dtype == "float32" else 1e-2)
    K().check_device_errors()


# ---- the recurrent mixers' kernels ---------------------------------------------------------------------
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
@pytest.mark.parametrize("geom", [(4, 24, 4, 20, 4, 2), (2, 12, 2, 8, 2, 1), (8, 64, 8, 32, 8, 4), (3, 40, 5, 7, 0, 0)])
def test_short_convolution_carries_its_inputs(taps, geom):
    """Three requests in slots 2, 0 and 3, cut into steps of unequal portions (single tokens among them): the result is
    that of each request convolved whole, and a slot that is cleared and used again starts from zeros."""
    n_a, d_a, n_b, d_b, n_unit, n_scaled = geom
    C = n_a * d_a + n_b * d_b
    r = rng(taps * 100 + C)
    w = r.uniform(-1, 1, (C, taps))
    lens, slots = [23, 9, 14], [2, 0, 3]
    xs = [r.standard_normal((n, C)) for n in lens]
    carried = torch.full((4, max(taps - 1, 1), C), 7.0, device=DEV)          # rubbish that a new request must not see
    carried[slots] = 0.0

    def want(x):
        y = plain.silu(plain.short_convolution(f64(dev(x)), f64(dev(w))))
        col = 0
        for u in range(n_a + n_b):
            n = d_a if u < n_a else d_b
            if u < n_unit:
                y[:, col:col + n] /= np.sqrt((y[:, col:col + n] ** 2).sum(-1, keepdims=True) + 1e-6)
            if u < n_scaled:
                y[:, col:col + n] *= 0.25
            col += n
        return y
    got = [[] for _ in lens]
    done = [0, 0, 0]
    cuts = [[5, 1, 1, 16], [2, 7], [1, 1, 12]]
    for step in range(4):
        live = [i for i in range(3) if step < len(cuts[i])]
        part = [xs[i][done[i]:done[i] + cuts[i][step]] for i in live]
        x = dev(np.concatenate(part))
        out = torch.empty(x.shape[0], C, device=DEV)
        K().short_conv(x, 1, dev(w), carried, step_ctx([len(p) for p in part], [slots[i] for i in live]), out, n_a, d_a, n_b, d_b,
                       n_unit=n_unit, n_scaled=n_scaled, scale=0.25, unit_eps=1e-6)
        o = 0
        for i, p in zip(live, part):
            got[i].append(out[o:o + len(p)])
            o += len(p)
            done[i] += len(p)
    for i in range(3):
        assert rel(torch.cat(got[i]), want(xs[i])) < 3e-6
    # slot 2 again, cleared: as if nothing had been there
    carried[2] = 0.0
    x = dev(xs[1])
    out = torch.empty(x.shape[0], C, device=DEV)
    K().short_conv(x, 1, dev(w), carried, step_ctx([lens[1]], [2]), out, n_a, d_a, n_b, d_b, n_unit=n_unit, n_scaled=n_scaled,
                   scale=0.25, unit_eps=1e-6)
    assert rel(out, want(xs[1])) < 3e-6
    K().check_device_errors()


@pytest.mark.parametrize("H,d", [(3, 24), (2, 128), (5, 7)])
def test_decays_from_their_logits(H, d):
    r = rng(H * d)
    T = 19
    z = r.standard_normal((2, T, H * d + 5)) * 3
    z[0, 0, 5] = 40.0                      # softplus far out on both sides
    z[0, 1, 5] = -40.0
    bias, rate = r.uniform(-1.5, 1.5, H * d), np.exp(r.uniform(-1.5, 1.5, H))
    zz = f64(dev(z)).sum(0)[:, 5:] + f64(dev(bias))
    out = torch.empty(T, H * d, device=DEV)
    K().decay(dev(z), 2, dev(bias), dev(rate), 1.0, out, H, d, z_stride=H * d + 5, z_col0=5)
    assert rel(out, np.exp(-np.repeat(f64(dev(rate)), d) * plain.softplus(zz))) < 3e-6
    tau = 6.0
    K().decay(dev(z), 2, dev(bias), torch.full((H,), 1 / tau, device=DEV), -1.0, out, H, d, z_stride=H * d + 5, z_col0=5)
    assert rel(out, plain.sigmoid(zz) ** (1 / tau)) < 3e-6
    K().check_device_errors()


def scan_inputs(r, T, H, Hq, d, dv, slow=False):
    q, k = r.standard_normal((T, Hq, d)) / np.sqrt(d), r.standard_normal((T, Hq, d))
    k /= np.sqrt((k * k).sum(-1, keepdims=True))
    v = r.standard_normal((T, H, dv))
    a = r.uniform(0.97 if slow else 0.3, 1.0, (T, H, d))
    b = r.standard_normal((T, H)) * 2
    return q, k, v, a, b


def plain_scan(q, k, v, a, b, H, Hq, delta):
    rep = H // Hq
    qq, kk = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    if delta:
        return plain.delta_rule(qq, kk, v, plain.sigmoid(b), a)
    T, _, d = qq.shape
    o = np.zeros_like(v)
    for h in range(H):
        S = np.zeros((d, v.shape[2]))
        for t in range(T):
            S = a[t, h][:, None] * S + np.outer(kk[t, h], v[t, h])
            o[t, h] = S.T @ qq[t, h]
    return o


@pytest.mark.parametrize("delta", [False, True])
@pytest.mark.parametrize("geom", [(3, 3, 24, 40), (4, 2, 24, 20), (2, 1, 12, 8), (8, 4, 64, 32), (4, 4, 128, 64), (2, 2, 128, 128),
                                  (1, 1, 200, 5), (2, 1, 300, 33), (6, 1, 16, 16)])
def test_recurrence_whole_in_portions_and_token_by_token(delta, geom):
    """Both forms of the recurrence: three requests of unequal length whole and side by side; then the same in portions
    of changing size (two tokens and one among them) with the state waiting in its slot between steps; then a slot
    cleared and used again.  The operands are column slices of wider arrays, as the products leave them."""
    H, Hq, d, dv = geom
    r = rng(H * d + dv + delta)
    lens, slots = [41, 3, 18], [1, 3, 0]
    data = [scan_inputs(r, n, H, Hq, d, dv) for n in lens]
    data = [tuple(f64(dev(x)) for x in item) for item in data]
    want = [plain_scan(*item, H, Hq, delta) for item in data]
    state = torch.full((4, H, dv, d), 3.0, device=DEV)

    def run(parts, use_slots):
        """parts: per request a (lo, hi) range of its tokens."""
        T = sum(hi - lo for lo, hi in parts)
        wide = torch.zeros(T, 2 * Hq * d + H * dv + 9, device=DEV)
        parts_i = [(i, p) for i, p in enumerate(parts) if p[1] > p[0]]
        rows = lambda j, w: dev(np.concatenate([data[i][j][p[0]:p[1]].reshape(p[1] - p[0], w) for i, p in parts_i]))
        wide[:, 4:4 + Hq * d] = rows(0, Hq * d)
        wide[:, 4 + Hq * d:4 + 2 * Hq * d] = rows(1, Hq * d)
        wide[:, 4 + 2 * Hq * d:4 + 2 * Hq * d + H * dv] = rows(2, H * dv)
        a, b = rows(3, H * d), rows(4, H)
        o = torch.empty(T, H * dv, device=DEV)
        ctx = step_ctx([p[1] - p[0] for _, p in parts_i], [use_slots[i] for i, _ in parts_i])
        K().linear_scan(wide[:, 4:4 + Hq * d], wide[:, 4 + Hq * d:4 + 2 * Hq * d], wide[:, 4 + 2 * Hq * d:4 + 2 * Hq * d + H * dv], a,
                        b if delta else None, 1.0, state, ctx, o, H, Hq, d, dv)
        out, at = {}, 0
        for i, p in parts_i:
            out[i] = o[at:at + p[1] - p[0]].view(-1, H, dv)
            at += p[1] - p[0]
        return out
    state[slots] = 0.0
    got = run([(0, n) for n in lens], slots)
    for i in range(3):
        assert rel(got[i], want[i]) < 2e-5, f"whole, request {i}"
    state[slots] = 0.0
    pieces = [[] for _ in lens]
    at = [0, 0, 0]
    sizes = [[7, 2, 1, 1, 30], [1, 2, 0, 0, 0], [0, 5, 1, 12, 0]]
    for step in range(5):
        parts = [(at[i], at[i] + sizes[i][step]) for i in range(3)]
        res = run(parts, slots)
        for i in res:
            pieces[i].append(res[i])
            at[i] = parts[i][1]
    for i in range(3):
        assert rel(torch.cat(pieces[i]), want[i]) < 2e-5, f"portions, request {i}"
    state[3] = 0.0
    got = run([(0, 0), (0, 0), (0, lens[2])], [0, 0, 3])
    assert rel(got[2], want[2]) < 2e-5
    K().check_device_errors()


@pytest.mark.parametrize("delta", [False, True])
def test_the_state_remembers_a_token_hundreds_back(delta):
    """One early token writes a value under a key that no later token touches (later keys are orthogonal to it, decays
    near one); the last query, decoded alone after the prompt came in two portions, asks for that key and must read the
    value back, weakened by exactly the product of the decays in between."""
    H, Hq, d, dv, T, planted = 2, 1, 32, 16, 700, 3
    r = rng(11 + delta)
    q, k, v, a, b = scan_inputs(r, T, H, Hq, d, dv, slow=True)
    a[:] = r.uniform(0.995, 1.0, a.shape)
    k[:, :, 0] = 0.0
    k /= np.sqrt((k * k).sum(-1, keepdims=True))
    k[planted] = 0.0
    k[planted, :, 0] = 1.0
    v[planted] = 5.0 + np.arange(dv)
    b[planted] = 30.0                                   # beta = 1
    q[-1] = 0.0
    q[-1, :, 0] = 1.0
    data = tuple(f64(dev(x)) for x in (q, k, v, a, b))
    want = plain_scan(*data, H, Hq, delta)
    fade = data[3][planted + 1:, :, 0].prod(0)
    assert np.allclose(want[-1], fade[:, None] * data[2][planted], rtol=1e-9)
    state = torch.zeros(3, H, dv, d, device=DEV)
    outs = []
    for lo, hi in ((0, 300), (300, T - 1), (T - 1, T)):
        o = torch.empty(hi - lo, H * dv, device=DEV)
        K().linear_scan(dev(q[lo:hi].reshape(hi - lo, -1)), dev(k[lo:hi].reshape(hi - lo, -1)), dev(v[lo:hi].reshape(hi - lo, -1)),
                        dev(a[lo:hi].reshape(hi - lo, -1)), dev(b[lo:hi]) if delta else None, 1.0, state, step_ctx([hi - lo], [1]), o,
                        H, Hq, d, dv)
        outs.append(o)
    assert rel(torch.cat(outs).view(T, H, dv), want) < 3e-5
    assert rel(outs[-1].view(H, dv), fade[:, None] * data[2][planted]) < 3e-5
    assert float(state[0].abs().sum()) == 0 and float(state[2].abs().sum()) == 0
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("H,dv", [(3, 40), (4, 20), (2, 128), (1, 8), (5, 33)])
def test_head_norm_with_gate(dtype, H, dv):
    dt, T, r = DT[dtype], 13, rng(H + dv)
    o = r.standard_normal((T, H, dv)) * r.uniform(0.01, 30, (T, H, 1))
    o[0, 0] = 0.0                                       # a head of zeros: eps keeps the quotient finite
    w, g = r.uniform(0.5, 1.6, dv), r.standard_normal((3, T, H * dv + 6)) * 2
    oo, ww = f64(dev(o)), f64(dev(w, dt))
    z = f64(dev(g)).sum(0)[:, 6:].reshape(T, H, dv)
    for gate, fn in (("silu", plain.silu), ("sigmoid", plain.sigmoid)):
        out = torch.empty(T, H * dv, dtype=dt, device=DEV)
        K().gate_norm(dev(o).view(T, H * dv), dev(w, dt), 1e-5, dev(g), 3, H * dv + 6, 6, gate, out, H, dv)
        assert rel(out.view(T, H, dv), plain.rms_norm(oo, 1e-5) * ww * fn(z)) < KTOL[dtype]
    K().check_device_errors()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("r_cfg", [(5, 1, 2, (3, 2)), (4, 0, 1, None), (6, 2, 3, (4, 2)), (3, 3, 2, (2, 1)), (16, 4, 4, (5, 3)), (2, 1, 3, (1, 1)),
                                   (60, 4, 6, (8, 3)), (7, 0, 7, (7, 7))])
def test_softmax_router_with_groups_and_correction(dtype, r_cfg):
    """Softmax scores, a correction that changes who is chosen but not the weights, groups that shut experts out (with
    negative choice scores an excluded expert must not come back as a zero), weights not renormalised."""
    experts, identity, top, groups = r_cfg
    dt, E, T, n_all = DT[dtype], 72, 257, experts + identity
    r = rng(n_all * top)
    h = dev(r.standard_normal((T, E)), dt)
    w = dev(r.standard_normal((n_all, E)) * 0.4, dt)
    corr = r.uniform(-0.6, 0.1, n_all)                  # mostly negative choice scores
    W = {"r.router": f64(w), "r.correction": f64(dev(corr))}
    rc = {"experts": experts, "identity": identity, "top": top, "scale": 1.7}
    if groups:
        rc["groups"] = {"count": groups[0], "keep": groups[1]}
    want_ids, want_w = plain.route(f64(h), W, "r", rc)
    ids = torch.empty(T, top, dtype=torch.int32, device=DEV)
    wts = torch.empty(T, top, device=DEV)
    logits = torch.empty(T, n_all, device=DEV)
    K().moe_route_softmax(h, w, dev(corr), top, groups[0] if groups else 1, groups[1] if groups else 1, 1.7, ids, wts, logits)
    assert rel(logits, f64(h) @ f64(w).T) < 1e-5
    # rows on which the choice is close in the plain implementation may differ in order; no row may differ in its set by
    # more than a close call
    z = f64(h) @ f64(w).T
    s = np.exp(z - z.max(-1, keepdims=True))
    s /= s.sum(-1, keepdims=True)
    got_ids = ids.cpu().numpy()
    bad = 0
    for t in range(T):
        if sorted(got_ids[t]) != sorted(want_ids[t]):
            c = s[t] + W["r.correction"]
            odd = set(got_ids[t]) ^ set(want_ids[t])
            assert max(c[list(odd)]) - min(c[list(odd)]) < 1e-5, f"row {t}: chose {got_ids[t]}, plain {want_ids[t]}"
            bad += 1
        else:
            order = np.argsort(got_ids[t])
            assert np.allclose(wts[t].cpu().numpy()[order], want_w[t][np.argsort(want_ids[t])], rtol=2e-5, atol=1e-7)
    assert bad <= 2
    K().check_device_errors()
