"""The kernel interface the parts call.  One backend exists in the product: the CUDA library.

The functions here check shapes and types, refuse sizes the kernels do not take with a clear
error, and forward to the backend.  There is no CPU path: without the library or without a GPU
the first call raises.  (Tests may install a stand-in backend with :func:`set_backend` to exercise
the host-side logic on a machine without a GPU.)
"""
from __future__ import annotations

from typing import Optional

import torch

from ..config.base import UnsupportedError

_backend = None

MAX_HEAD_DIM = 256          # heads that go through the q|k|v tails
MAX_LATENT_ROW = 640        # a latent row [latent | rotated part] the plain attention kernel walks
ERROR_BITS = {1: "a token id outside the vocabulary", 2: "a block-table entry that names no page",
              4: "a cache slot outside the pool", 8: "a device-side wait that ran out",
              16: "a position outside the rotary table"}


class PhaseProfile:
    """Device time per phase of the forward pass, for ``--profile``: parts wrap their kernel calls in
    ``kernels.phase(name)``; while the profile is on, each phase is bracketed by CUDA events on the current stream
    and ``take()`` returns milliseconds per name and clears them.  Off, ``phase`` costs one attribute test.  The
    reference keeps per-phase accumulators with the same names (src/model.h:75-79, src/ops.c:593-604)."""
    NAMES = ("embed", "glue", "qkv", "attn", "wo", "gate_up", "silu", "down", "head", "quant", "sample")

    class _Null:
        def __enter__(self):
            return self

        def __exit__(self, *a):
            return False

    class _Span:
        def __init__(self, owner, name):
            self.owner, self.name = owner, name

        def __enter__(self):
            self.a, self.b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            self.a.record()
            return self

        def __exit__(self, *a):
            self.b.record()
            self.owner.spans.append((self.name, self.a, self.b))
            return False

    def __init__(self):
        self.enabled, self.spans, self._null = False, [], self._Null()

    def enable(self, on: bool) -> None:
        self.enabled = bool(on) and torch.cuda.is_available()
        self.spans = []

    def phase(self, name: str):
        return self._Span(self, name) if self.enabled else self._null

    def take(self) -> dict:
        out = {n: 0.0 for n in self.NAMES}
        if self.spans:
            torch.cuda.synchronize()
            for name, a, b in self.spans:
                out[name] = out.get(name, 0.0) + a.elapsed_time(b)
        self.spans = []
        return out


profile = PhaseProfile()
phase = profile.phase


def backend():
    global _backend
    if _backend is None:
        from .native import NativeBackend
        _backend = NativeBackend()
    return _backend


def set_backend(b) -> None:
    global _backend
    _backend = b


def check_head_dim(d: int) -> None:
    if d % 16 or not 16 <= d <= MAX_HEAD_DIM:
        raise UnsupportedError(f"head_dim {d} is not supported: the attention kernels take multiples of 16 "
                               f"from 16 to {MAX_HEAD_DIM}")


def _need(cond: bool, msg: str) -> None:
    if not cond:
        raise ValueError(msg)


def embed(ids: torch.Tensor, table: torch.Tensor, out: torch.Tensor) -> None:
    _need(ids.dtype == torch.int32 and ids.dim() == 1, "embed: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.shape == (ids.shape[0], table.shape[1]), "embed: out must be float32 [T, E]")
    backend().embed(ids, table, out)


def embed_pair(ids, table, scale: float, pair, buckets: int, mul_prev: int, mul_cur: int, ctx, prev_state, out) -> None:
    """out = table[ids] * scale + pair[row], row = (previous * mul_prev + id * mul_cur) mod buckets, or ``buckets`` for a
    request's first token; ``prev_state`` (int32 [slots]: token + 1, 0 = none) carries the previous token from step to
    step and is brought up to date.  ``pair`` None: the scaled embedding alone."""
    _need(ids.dtype == torch.int32 and ids.dim() == 1, "embed_pair: ids must be int32 [T]")
    _need(out.dtype == torch.float32 and out.shape == (ids.shape[0], table.shape[1]), "embed_pair: out must be float32 [T, E]")
    if pair is not None:
        _need(pair.shape == (buckets + 1, table.shape[1]), "embed_pair: the pair table must be [buckets + 1, E]")
        _need(prev_state is not None and prev_state.dtype == torch.int32 and prev_state.dim() == 1,
              "embed_pair: the previous tokens must be int32 [slots]")
    backend().embed_pair(ids, table, float(scale), pair, int(buckets), int(mul_prev), int(mul_cur), ctx, prev_state, out)


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    _need(x.dtype == torch.float32 and x.dim() == 2, "rmsnorm: x must be float32 [N, E]")
    _need(w.shape == (x.shape[1],) and out.shape[1] == x.shape[1], "rmsnorm: width mismatch")
    _need(rows is None or (rows.dtype == torch.int32 and rows.shape[0] == out.shape[0]), "rmsnorm: rows must be int32 [M]")
    _need(rows is not None or out.shape[0] == x.shape[0], "rmsnorm: row count mismatch")
    backend().rmsnorm(x, w, float(eps), out, rows)


def linear(a: torch.Tensor, w: torch.Tensor, bias: Optional[torch.Tensor], out: torch.Tensor, accumulate: bool) -> None:
    """out (=|+=) a @ w.T (+ bias); ``accumulate`` adds into a float32 ``out`` (the residual stream)."""
    _need(a.dim() == 2 and w.dim() == 2 and a.shape[1] == w.shape[1], "linear: inner sizes differ")
    _need(out.shape == (a.shape[0], w.shape[0]), "linear: out must be [M, N]")
    _need(bias is None or bias.shape == (w.shape[0],), "linear: bias must be [N]")
    _need(not accumulate or out.dtype == torch.float32, "linear: accumulation needs a float32 output")
    backend().linear(a, w, bias, out, bool(accumulate))


def rope_kv_write(qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d) -> None:
    _need(qkv.shape[1] == (H + 2 * G) * d and q_out.shape == (qkv.shape[0], H * d), "rope_kv_write: shape mismatch")
    _need(k_cache.shape[2:] == (G, d) and v_cache.shape == k_cache.shape, "rope_kv_write: cache geometry mismatch")
    _need(k_cache.dtype == qkv.dtype == q_out.dtype, "rope_kv_write: element types differ")
    _need(n_rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (n_rot // 2, 2) and cos_sin.dtype == torch.float32),
          "rope_kv_write: cos/sin table must be float32 [positions, n_rot/2, 2]")
    backend().rope_kv_write(qkv, cos_sin, int(n_rot), positions, slots, q_out, k_cache, v_cache, H, G, d)


def attention_step_arrays(q_lens, heads_per_group: int):
    """Tile lists of a step's tokens for the tiled attention kernels, as named int32 arrays.

    A tile holds consecutive tokens of one request: its request index (``seq``), its first token's index in the
    step (``t0``) and its token count (``nt``).  The heads that share a key/value head are packed into a tile's rows
    beside the tokens, so a tile of R rows takes R // heads_per_group tokens.  Tile heights: "1" = 16 rows (a step of
    single tokens; the decode kernels), "4" = 64 rows (short portions), "8" = 128 rows and "16" = two tiles of 128
    rows per work item (portions of 64 tokens and more).  A height too small for the heads per group is left out."""
    import numpy as np
    max_q, S = max(q_lens), len(q_lens)
    heights = ["1"] if max_q == 1 else (["8", "16"] if max_q >= 64 else ["4"])
    out = {}
    for h in heights:
        per = (16 * int(h)) // heads_per_group if h != "16" else 2 * (128 // heads_per_group)
        if per < 1:
            continue
        if max_q == 1:
            seq = t0 = np.arange(S, dtype=np.int32)
            nt = np.ones(S, dtype=np.int32)
        else:
            ls, lt, ln, at = [], [], [], 0
            for s_i, n in enumerate(q_lens):
                for a in range(0, n, per):
                    ls.append(s_i)
                    lt.append(at + a)
                    ln.append(min(per, n - a))
                at += n
            seq, t0, nt = (np.asarray(x, dtype=np.int32) for x in (ls, lt, ln))
        out[h + ".seq"], out[h + ".t0"], out[h + ".nt"] = seq, t0, nt
    return out


def mask_code(window: int = 0, chunk: int = 0) -> int:
    """The one number that names a mask to the attention kernels: ``window`` > 0 (a query sees itself and the window - 1
    positions before it), -``chunk`` (a query sees the keys of its own chunk of that many positions, counted from
    position 0), or 0 (every key)."""
    window, chunk = int(window or 0), int(chunk or 0)
    _need(window >= 0 and chunk >= 0 and not (window and chunk), "a mask is a window or chunks, not both")
    return window if window else -chunk


def tiled_attention_takes(dtype, head_dim: int, block_size: int) -> bool:
    """Whether the tiled tensor-core attention kernels serve heads of this type and size (with value heads of the same
    size) from pages of ``block_size`` tokens; everything else goes to the plain kernel."""
    b = backend()
    return (dtype == torch.bfloat16 and head_dim in (64, 128) and 64 % int(block_size) == 0
            and getattr(b, "attention", "plain") == "fast")


def set_launch_overlap(on: bool) -> None:
    """Whether a kernel may be launched so that it starts (and waits) before the kernel in front of it has finished.  A
    backend without such launches ignores it."""
    fn = getattr(backend(), "set_launch_overlap", None)
    if fn is not None:
        fn(bool(on))


def paged_attention(q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tiles=None, dv=None, values_in_keys=False,
                    sinks=None, zero_sink=False, slopes=None, head_scales=None, softcap: float = 0.0) -> None:
    """``window``: a :func:`mask_code`.  ``tiles``: the device arrays of :func:`attention_step_arrays` for this step
    (without them only the plain kernel runs).  ``dv``: the size of a value head where it is not ``d``; ``out`` is then
    [T, H * dv].  ``values_in_keys``: there is no array of values, a value is the first ``dv`` elements of its key.
    ``sinks`` (float32 [H]): a score per head that joins the softmax's denominator once and has no value; ``zero_sink``:
    such a score of 0 for every head (one is added to the denominator).  ``slopes`` (float32 [H]): slope * (query
    position - key position) is taken off every score.  ``head_scales`` (float32 [H]): the scaled score of head h is
    multiplied by head_scales[h]; ``softcap`` > 0: the score becomes softcap * tanh(score / softcap), after the factors and
    before the bias and the softmax."""
    dv = d if dv is None else int(dv)
    extra = {}
    if head_scales is not None or softcap:
        _need(head_scales is None or (head_scales.shape == (H,) and head_scales.dtype == torch.float32),
              "attention: head_scales are float32 [H]")
        _need(softcap >= 0, "attention: softcap must be positive (0: none)")
    if sinks is not None or zero_sink or slopes is not None:
        _need(sinks is None or (sinks.shape == (H,) and sinks.dtype == torch.float32), "attention: sinks are float32 [H]")
        _need(slopes is None or (slopes.shape == (H,) and slopes.dtype == torch.float32), "attention: slopes are float32 [H]")
        _need(not (zero_sink and sinks is not None), "attention: a learned sink or a sink of zero, not both")
        extra = {"sinks": sinks, "zero_sink": bool(zero_sink), "slopes": slopes}
    if head_scales is not None or softcap:
        extra.update(head_scales=head_scales, softcap=float(softcap))
    if values_in_keys:
        _need(0 < dv <= d <= MAX_LATENT_ROW and v_cache is None, "attention: values inside keys need dv <= d <= %d" % MAX_LATENT_ROW)
        _need(q.shape[1] == H * d and out.shape == (q.shape[0], H * dv) and k_cache.shape[2:] == (G, d), "attention: shape mismatch")
        _need(q.dtype == k_cache.dtype == out.dtype, "attention: element types differ")
        backend().paged_attention(q, k_cache, None, meta, ctx, H, G, d, int(window), float(scale), out, tiles or {}, dv=dv, **extra)
        return
    _need(0 < d <= MAX_HEAD_DIM and 0 < dv <= MAX_HEAD_DIM, "attention: head sizes must be 1..%d" % MAX_HEAD_DIM)
    _need(q.shape[1] == H * d and out.shape == (q.shape[0], H * dv), "attention: shape mismatch")
    _need(k_cache.shape[2:] == (G, d) and v_cache.shape[2:] == (G, dv), "attention: cache geometry mismatch")
    _need(q.dtype == k_cache.dtype == v_cache.dtype == out.dtype, "attention: element types differ")
    if dv == d:
        backend().paged_attention(q, k_cache, v_cache, meta, ctx, H, G, d, int(window), float(scale), out, tiles or {}, **extra)
    else:
        backend().paged_attention(q, k_cache, v_cache, meta, ctx, H, G, d, int(window), float(scale), out, tiles or {}, dv=dv, **extra)


def swiglu(gu: torch.Tensor, out: torch.Tensor, interleaved: bool = False) -> None:
    """out = silu(gate) * up; gate and up are the two halves of a row of ``gu``, or alternate along it."""
    _need(gu.shape == (out.shape[0], 2 * out.shape[1]) and gu.dtype == out.dtype, "swiglu: shape mismatch")
    backend().swiglu(gu, out, bool(interleaved))


def linear_swiglu(a: torch.Tensor, w: torch.Tensor, gu_buf: torch.Tensor, out: torch.Tensor) -> None:
    """out = silu(g) * u where [g0, u0, g1, u1, ...] = a @ w.T (rows of ``w`` alternate gate, up).  ``gu_buf``
    [M, 2F] is scratch for the unfused form."""
    _need(a.shape[1] == w.shape[1] and w.shape[0] == 2 * out.shape[1] and out.shape[0] == a.shape[0],
          "linear_swiglu: shape mismatch")
    _need(gu_buf.shape == (a.shape[0], w.shape[0]), "linear_swiglu: scratch must be [M, 2F]")
    backend().linear_swiglu(a, w, gu_buf, out)


def linear_residual_norm(a, w, bias, residual, norm_w, eps, xn_out, center: bool = False, shift=None) -> None:
    """residual += a @ w.T (+ bias); then, if ``xn_out`` is given, xn_out = rmsnorm(residual) * norm_w.  ``center``: the
    norm takes the mean off first (layer norm; ``norm_w`` float32).  ``shift`` = (mu, state, seq_slots), for a step in which
    every request brings one token: xn_out = h + (previous h - h) * mu with h the norm's output, the previous h from the
    request's row of ``state`` (float32 [slots, N]), which then receives h (``norm_w`` and ``mu`` float32)."""
    _need(a.shape[1] == w.shape[1] and residual.shape == (a.shape[0], w.shape[0]) and residual.dtype == torch.float32,
          "linear_residual_norm: shape mismatch")
    _need(xn_out is None or (xn_out.shape == residual.shape and norm_w.shape == (w.shape[0],)),
          "linear_residual_norm: norm shape mismatch")
    if center or shift is not None:
        _need(xn_out is not None and norm_w.dtype == torch.float32, "linear_residual_norm: this norm takes a float32 weight")
        if shift is not None:
            mu, state, seq_slots = shift
            _need(mu.shape == (w.shape[0],) and mu.dtype == torch.float32 and state.dtype == torch.float32 and state.dim() == 2
                  and state.shape[1] == w.shape[0] and seq_slots.shape[0] == a.shape[0],
                  "linear_residual_norm: the shift takes (float32 [N], float32 [slots, N], a slot per row)")
        backend().linear_residual_norm(a, w, bias, residual, norm_w, float(eps), xn_out, center=bool(center), shift=shift)
        return
    backend().linear_residual_norm(a, w, bias, residual, norm_w, float(eps), xn_out)


def linear_rope_kv(a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d) -> None:
    """q|k|v = a @ w.T + bias, then :func:`rope_kv_write`; ``qkv_buf`` [T, (H+2G)d] is scratch for the unfused form."""
    _need(w.shape[0] == (H + 2 * G) * d and q_out.shape == (a.shape[0], H * d), "linear_rope_kv: shape mismatch")
    _need(k_cache.shape[2:] == (G, d) and v_cache.shape == k_cache.shape and k_cache.dtype == q_out.dtype,
          "linear_rope_kv: cache geometry mismatch")
    backend().linear_rope_kv(a, w, bias, qkv_buf, cos_sin, int(n_rot), positions, slots, q_out, k_cache, v_cache, H, G, d)


ACTIVATIONS = {"silu": 0, "relu": 1, "gelu_tanh": 2, "relu2": 3, "none": 4}       # relu2: the square of relu
ACT_GLU = 256               # added to an activation code: gated form of the grouped product
MOE_TILE = 128              # places of one expert per tile of the grouped product ...
MOE_TILE_FEW = 16           # ... and in steps of few tokens, whose blocks only stream weights: more, smaller tiles


def moe_tile(pairs: int) -> int:
    """Places per tile for a step with ``pairs`` (token, choice) pairs."""
    return MOE_TILE_FEW if pairs <= 512 else MOE_TILE



def _act(name: str) -> int:
    if name not in ACTIVATIONS:
        raise UnsupportedError(f"activation '{name}' is not supported (known: {', '.join(ACTIVATIONS)})")
    return ACTIVATIONS[name]


def _dyt_ok(p, E, what):
    alpha, w, b = p
    _need(alpha.numel() == 1 and w.shape == (E,) and b.shape == (E,) and alpha.dtype == w.dtype == b.dtype,
          f"{what}: norm parameters must be a scalar and two vectors [E] of one type")


def dyt(x: torch.Tensor, params, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> None:
    """Dynamic Tanh norm: out = tanh(alpha * x) * w + b, ``params`` = (alpha, w, b); with ``rows`` (int32) only
    those rows of ``x``, in that order."""
    _need(x.dim() == 2 and out.shape[1] == x.shape[1], "dyt: width mismatch")
    _dyt_ok(params, x.shape[1], "dyt")
    _need(rows is None or (rows.dtype == torch.int32 and rows.shape[0] == out.shape[0]), "dyt: rows must be int32 [M]")
    _need(rows is not None or out.shape[0] == x.shape[0], "dyt: row count mismatch")
    backend().dyt(x, params, out, rows)


def _mix_ok(mix, residual, what):
    if mix is not None:
        y, w = mix
        _need(w.dim() == 2 and w.shape[0] == residual.shape[0] and y.shape == (w.shape[0] * w.shape[1], residual.shape[1])
              and y.dtype == torch.float32 and w.dtype == torch.float32, f"{what}: mix = (float32 [M * top, E], float32 [M, top])")


def dyt_residual(y: Optional[torch.Tensor], post, residual: torch.Tensor, nxt=None, out: Optional[torch.Tensor] = None,
                 mix=None) -> None:
    """residual += dyt_post(y + mix); with ``nxt`` and ``out`` also out = dyt_nxt(residual).  ``mix`` = (rows [M * top,
    E], weights [M, top]) adds ``sum_j weights[m, j] * rows[m * top + j]`` (j in order) to y, which may then be None."""
    _need(residual.dtype == torch.float32 and (y.shape == residual.shape if y is not None else mix is not None), "dyt_residual: shape mismatch")
    _mix_ok(mix, residual, "dyt_residual")
    _dyt_ok(post, residual.shape[1], "dyt_residual")
    _need((nxt is None) == (out is None), "dyt_residual: the next norm and its output come together")
    if nxt is not None:
        _dyt_ok(nxt, residual.shape[1], "dyt_residual")
        _need(out.shape == residual.shape, "dyt_residual: output shape mismatch")
    if mix is None:
        backend().dyt_residual(y, post, residual, nxt, out)
    else:
        backend().dyt_residual(y, post, residual, nxt, out, mix=mix)


def linear_dyt_residual(a, w, bias, y_buf, post, residual, nxt=None, out=None, mix=None) -> None:
    """residual += dyt_post(a @ w.T + bias + mix), and with ``nxt`` / ``out`` the next norm of the new residual, as
    :func:`dyt_residual`; ``y_buf`` [M, N] float32 is scratch for the form that finishes the product first."""
    _mix_ok(mix, residual, "linear_dyt_residual")
    _need(a.shape[1] == w.shape[1] and residual.shape == (a.shape[0], w.shape[0]) and residual.dtype == torch.float32,
          "linear_dyt_residual: shape mismatch")
    _need(y_buf.shape == residual.shape and y_buf.dtype == torch.float32, "linear_dyt_residual: scratch must be float32 [M, N]")
    _dyt_ok(post, w.shape[0], "linear_dyt_residual")
    _need((nxt is None) == (out is None), "linear_dyt_residual: the next norm and its output come together")
    if nxt is not None:
        _dyt_ok(nxt, w.shape[0], "linear_dyt_residual")
        _need(out.shape == residual.shape, "linear_dyt_residual: output shape mismatch")
    if mix is None:
        backend().linear_dyt_residual(a, w, bias, y_buf, post, residual, nxt, out)
    else:
        backend().linear_dyt_residual(a, w, bias, y_buf, post, residual, nxt, out, mix=mix)


def linear_rope_norm_kv(a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d, dv,
                        norm_eps, norm_weights=None, value_mix=None, pairing: str = "half") -> None:
    """The q|k|v product and its tail for attention with unit-rms queries and keys: row = [H heads of d | G key heads
    of d | G value heads of dv] (G = 0: the layer has no keys and values of its own; dv = 0: the row has no value heads,
    the layer's values are its keys, and ``v_cache`` is None); ``pairing``: which dimensions turn together, "half"
    (i, i + n_rot/2) or "interleaved" (2i, 2i + 1); rotation of the first ``n_rot``
    dimensions of query and key heads, then, unless ``norm_eps`` is None, x / sqrt(mean(x^2) + eps) per head, times
    ``norm_weights`` = (q weight, k weight), float32 [d] each, where the norm has weights; queries to ``q_out``, keys
    and values to the cache at ``slots``.  ``value_mix`` = (first [T, G * dv] float32, mode, lambda): mode 1 leaves the
    row's values in ``first``, mode 2 stores (1 - lambda) v + lambda first instead of v.  ``qkv_buf`` [T, row] float32 is
    scratch."""
    if norm_weights is not None:
        _need(norm_eps is not None and all(x.shape == (d,) and x.dtype == torch.float32 for x in norm_weights),
              "linear_rope_norm_kv: norm weights are float32 [d] and come with a norm")
    if value_mix is not None:
        _need(G > 0 and value_mix[0].shape == (a.shape[0], G * dv) and value_mix[0].dtype == torch.float32 and value_mix[1] in (1, 2),
              "linear_rope_norm_kv: value mixing takes (float32 [T, G * dv], 1 | 2, lambda)")
    C = H * d + G * (d + dv)
    _need(w.shape[0] == C and q_out.shape == (a.shape[0], H * d) and a.shape[1] == w.shape[1], "linear_rope_norm_kv: shape mismatch")
    _need(qkv_buf.shape == (a.shape[0], C) and qkv_buf.dtype == torch.float32, "linear_rope_norm_kv: scratch must be float32 [T, row]")
    _need(0 < d <= MAX_HEAD_DIM and 0 <= dv <= MAX_HEAD_DIM and n_rot % 2 == 0 and 0 <= n_rot <= d, "linear_rope_norm_kv: bad head sizes")
    _need(pairing in ("half", "interleaved"), "linear_rope_norm_kv: pairing is 'half' or 'interleaved'")
    _need(dv > 0 or value_mix is None, "linear_rope_norm_kv: a row without values mixes none")
    if G:
        _need(k_cache.shape[2:] == (G, d) and k_cache.dtype == q_out.dtype, "linear_rope_norm_kv: cache geometry mismatch")
        _need((v_cache is None) if dv == 0 else (v_cache.shape[2:] == (G, dv) and v_cache.dtype == q_out.dtype),
              "linear_rope_norm_kv: cache geometry mismatch (values)")
    _need(n_rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (n_rot // 2, 2) and cos_sin.dtype == torch.float32),
          "linear_rope_norm_kv: cos/sin table must be float32 [positions, n_rot/2, 2]")
    extra = {}
    if norm_weights is not None:
        extra["norm_weights"] = norm_weights
    if value_mix is not None:
        extra["value_mix"] = (value_mix[0], int(value_mix[1]), float(value_mix[2]))
    if pairing != "half":
        extra["pairing"] = pairing
    backend().linear_rope_norm_kv(a, w, bias, qkv_buf, cos_sin, int(n_rot), positions, slots, q_out, k_cache, v_cache,
                                  H, G, d, dv, None if norm_eps is None else float(norm_eps), **extra)


def linear_latent_split(a, w, buf, q_norm_w, kv_norm_w, eps, cos_sin, positions, slots, cq_out, cache, q_rank, kv_rank, rot) -> None:
    """Latent attention's down product and its tail: row = a @ w.T = [q_rank | kv_rank | rot]; the first two parts are
    normed (x / sqrt(mean(x^2) + eps) times a float32 weight), the query latent goes to ``cq_out``, the key/value latent
    and the last part, rotated in pairs (2i, 2i + 1), form the token's row of ``cache`` [pages, block, 1, kv_rank + rot].
    ``buf`` [T, row] float32 is scratch."""
    C = q_rank + kv_rank + rot
    _need(w.shape[0] == C and a.shape[1] == w.shape[1] and buf.shape == (a.shape[0], C) and buf.dtype == torch.float32,
          "linear_latent_split: shape mismatch")
    _need(q_norm_w.shape == (q_rank,) and kv_norm_w.shape == (kv_rank,) and q_norm_w.dtype == kv_norm_w.dtype == torch.float32,
          "linear_latent_split: norm weights are float32 [q_rank] and [kv_rank]")
    _need(cq_out.shape == (a.shape[0], q_rank) and cache.shape[2:] == (1, kv_rank + rot) and cache.dtype == cq_out.dtype,
          "linear_latent_split: output geometry mismatch")
    _need(rot % 2 == 0 and (rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (rot // 2, 2) and cos_sin.dtype == torch.float32)),
          "linear_latent_split: cos/sin table must be float32 [positions, rot/2, 2]")
    backend().linear_latent_split(a, w, buf, q_norm_w, kv_norm_w, float(eps), cos_sin, positions, slots, cq_out, cache,
                                  int(q_rank), int(kv_rank), int(rot))


def linear_latent_query(a, w, buf, cos_sin, positions, q_plain, q_att, H, d, rot, att_col) -> None:
    """Latent attention's query product and its tail: row = a @ w.T = H heads of [d plain | rot rotated]; the plain parts
    go to ``q_plain`` [T, H * d], the rotated ones (pairs (2i, 2i + 1)) into ``q_att`` [T, H * row] at column ``att_col``
    of each head's row.  ``buf`` [T, H * (d + rot)] float32 is scratch."""
    T = a.shape[0]
    _need(w.shape[0] == H * (d + rot) and a.shape[1] == w.shape[1] and buf.shape == (T, w.shape[0]) and buf.dtype == torch.float32,
          "linear_latent_query: shape mismatch")
    _need(q_plain.shape == (T, H * d) and q_att.shape[0] == T and q_att.shape[1] % H == 0 and att_col + rot <= q_att.shape[1] // H
          and q_plain.dtype == q_att.dtype, "linear_latent_query: output geometry mismatch")
    _need(rot % 2 == 0 and (rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (rot // 2, 2) and cos_sin.dtype == torch.float32)),
          "linear_latent_query: cos/sin table must be float32 [positions, rot/2, 2]")
    backend().linear_latent_query(a, w, buf, cos_sin, positions, q_plain, q_att, int(H), int(d), int(rot), int(att_col))


def linear_latent_query_absorb(a, w_uq, buf, cos_sin, positions, w_ukt, q_plain, q_att, H, d, rot) -> None:
    """Latent attention's query, ready for attention over the cached rows: ``q = a @ w_uq.T`` (H heads of [d plain | rot
    rotated]); per head, ``q_att`` [T, H * (kv_rank + rot)] receives ``w_ukt[h] @ q_plain`` (w_ukt [H, kv_rank, d]) in its
    first kv_rank columns and the rotated part behind them.  One kernel behind the product in bfloat16; else
    :func:`linear_latent_query` and :func:`headwise_linear` with ``q_plain`` [T, H * d] between them."""
    R = w_ukt.shape[1]
    _need(w_ukt.shape == (H, R, d) and q_att.shape == (a.shape[0], H * (R + rot)) and w_ukt.dtype == q_att.dtype,
          "linear_latent_query_absorb: shape mismatch")
    b = backend()
    if hasattr(b, "linear_latent_query_absorb") and q_att.dtype == torch.bfloat16:
        _need(w_uq.shape[0] == H * (d + rot) and a.shape[1] == w_uq.shape[1] and buf.shape == (a.shape[0], w_uq.shape[0])
              and buf.dtype == torch.float32, "linear_latent_query_absorb: shape mismatch")
        _need(rot % 2 == 0 and (rot == 0 or (cos_sin is not None and cos_sin.shape[1:] == (rot // 2, 2) and cos_sin.dtype == torch.float32)),
              "linear_latent_query_absorb: cos/sin table must be float32 [positions, rot/2, 2]")
        b.linear_latent_query_absorb(a, w_uq, buf, cos_sin, positions, w_ukt, q_att, int(H), int(d), int(rot))
        return
    linear_latent_query(a, w_uq, buf, cos_sin, positions, q_plain, q_att, H, d, rot, R)
    headwise_linear(q_plain, w_ukt, q_att, H, d, R + rot)


def headwise_linear(x, w, out, H: int, in_row: int, out_row: int) -> None:
    """A product per head: out[t, h, :N] = w[h] @ x[t, h, :K] with w [H, N, K]; a row of ``x`` holds H heads ``in_row``
    apart, a row of ``out`` H heads ``out_row`` apart (a head's result may be the first N columns of a wider row)."""
    _need(w.dim() == 3 and w.shape[0] == H and x.shape[1] == H * in_row and out.shape == (x.shape[0], H * out_row)
          and in_row >= w.shape[2] and out_row >= w.shape[1], "headwise_linear: shape mismatch")
    _need(x.dtype == out.dtype == w.dtype, "headwise_linear: element types differ")
    backend().headwise_linear(x, w, out, int(H), int(in_row), int(out_row))


def linear_glu(a: torch.Tensor, w: torch.Tensor, gu_buf: torch.Tensor, out: torch.Tensor, act: str) -> None:
    """out = act(g) * u where [g0, u0, g1, u1, ...] = a @ w.T (rows of ``w`` alternate gate, up)."""
    _need(a.shape[1] == w.shape[1] and w.shape[0] == 2 * out.shape[1] and out.shape[0] == a.shape[0], "linear_glu: shape mismatch")
    _need(gu_buf.shape == (a.shape[0], w.shape[0]), "linear_glu: scratch must be [M, 2F]")
    if act == "silu":
        backend().linear_swiglu(a, w, gu_buf, out)
    else:
        backend().linear_glu(a, w, gu_buf, out, _act(act))


def linear_act(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor, act: str) -> None:
    """out = act(a @ w.T)."""
    _need(a.shape[1] == w.shape[1] and out.shape == (a.shape[0], w.shape[0]), "linear_act: shape mismatch")
    backend().linear_act(a, w, out, _act(act))


def scale_(x: torch.Tensor, s: float) -> None:
    _need(x.dtype == torch.float32 and x.is_contiguous(), "scale_: float32, contiguous")
    backend().scale_(x, float(s))


def moe_route(h, w, b, top: int, ids, weights, logits) -> None:
    """Router: ``logits`` = h @ w.T + b accumulated in float32 (a product like any other: exact products of the stored
    values, float32 sums); the ``top`` largest logits of a token choose its experts (``ids`` int32 [T, top], largest
    first, the lower index among equals), ``weights`` = softmax over the chosen logits only."""
    T, E = h.shape[0], w.shape[0]
    _need(h.shape[1] == w.shape[1] and (b is None or b.shape == (E,)) and 1 <= top <= E, "moe_route: shape mismatch")
    _need(ids.shape == (T, top) and ids.dtype == torch.int32 and weights.shape == (T, top) and weights.dtype == torch.float32,
          "moe_route: ids int32 [T, top], weights float32 [T, top]")
    _need(logits.shape == (T, E) and logits.dtype == torch.float32, "moe_route: logits float32 [T, experts]")
    backend().moe_route(h, w, b, int(top), ids, weights, logits)


def moe_max_tiles(pairs: int, experts: int, tile: int = 0) -> int:
    """Room for the tile lists of :func:`moe_group`: no grouping of ``pairs`` places over ``experts`` has more tiles."""
    return pairs // (tile or moe_tile(pairs)) + min(experts, pairs)


def moe_group(ids, experts: int, order, tile_expert, tile_p0, tile_n, n_tiles) -> None:
    """Groups the (token, choice) pairs of ``ids`` [T, top] by expert, on the device: ``order[p]`` = the pair at
    place p; tiles of at most ``moe_tile(pairs)`` places of one expert; their number in ``n_tiles`` [1]."""
    pairs = ids.numel()
    _need(order.numel() >= pairs and min(tile_expert.numel(), tile_p0.numel(), tile_n.numel()) >= moe_max_tiles(pairs, experts)
          and n_tiles.numel() >= 1, "moe_group: lists too short")
    backend().moe_group(ids, int(experts), order, tile_expert, tile_p0, tile_n, n_tiles, moe_tile(pairs))


def moe_gemm(a, w, out, act: str, order, src_div: int, scatter: bool, tile_expert, tile_p0, tile_n, n_tiles, pairs: int,
             glu: bool = False) -> None:
    """Grouped product over the places of :func:`moe_group`: out[dst(p)] = act(a[src(p)] @ w[expert(p)].T) with
    w [E, N, K]; src(p) = order[p] // src_div if src_div else p; dst(p) = order[p] if scatter else p.  ``glu``: the rows
    of an expert's matrix alternate gate, up, and out [.., N / 2] = act(gate) * up."""
    _need(w.dim() == 3 and a.shape[1] == w.shape[2], "moe_gemm: shape mismatch")
    _need(out.shape[1] == (w.shape[1] // 2 if glu else w.shape[1]) and (not glu or w.shape[1] % 2 == 0), "moe_gemm: output width mismatch")
    backend().moe_gemm(a, w, out, _act(act) | (ACT_GLU if glu else 0), order, int(src_div), bool(scatter), tile_expert, tile_p0,
                       tile_n, n_tiles, moe_max_tiles(int(pairs), w.shape[0]), moe_tile(int(pairs)))


def moe_combine(y, weights, out) -> None:
    """out[t] = sum_j weights[t, j] * y[t * top + j] in float32, j in order."""
    T, top = weights.shape
    _need(y.shape == (T * top, out.shape[1]) and out.shape[0] == T and out.dtype == torch.float32, "moe_combine: shape mismatch")
    backend().moe_combine(y, weights, out)


def moe_route_softmax(h, w, correction, top: int, n_groups: int, keep: int, scale: float, ids, weights, logits) -> None:
    """Router whose scores are a softmax over all of its outputs: s = softmax(h @ w.T) (float32); choice score = s +
    ``correction`` (or s); the outputs form ``n_groups`` equal groups of neighbours, a group's score is its largest
    choice score, and only outputs of the ``keep`` best groups can be chosen; ``ids`` = the ``top`` largest choice scores
    (largest first, the lower index among equals), ``weights`` = s[ids] * scale, not renormalised."""
    T, E = h.shape[0], w.shape[0]
    _need(h.shape[1] == w.shape[1] and (correction is None or correction.shape == (E,)) and 1 <= top <= E, "moe_route_softmax: shape mismatch")
    _need(n_groups >= 1 and E % n_groups == 0 and 1 <= keep <= n_groups and keep * (E // n_groups) >= top,
          "moe_route_softmax: the kept groups must hold at least `top` outputs")
    _need(ids.shape == (T, top) and ids.dtype == torch.int32 and weights.shape == (T, top) and weights.dtype == torch.float32,
          "moe_route_softmax: ids int32 [T, top], weights float32 [T, top]")
    _need(logits.shape == (T, E) and logits.dtype == torch.float32, "moe_route_softmax: logits float32 [T, outputs]")
    backend().moe_route_softmax(h, w, correction, int(top), int(n_groups), int(keep), float(scale), ids, weights, logits)


def product_sums(a, w, buf, finished: bool = False):
    """float32 sums of ``a @ w.T`` for a kernel that goes on from them: returns (sums, splits), sums [splits, M, N].  Where
    the tensor-core product is split over its inner dimension the pieces lie in the backend's one scratch area (valid
    until the next product) and whoever reads them sums them in order; else, and always with ``finished``, the product
    is in ``buf`` ([M, N] float32) and splits is 1."""
    _need(a.shape[1] == w.shape[1] and buf.shape == (a.shape[0], w.shape[0]) and buf.dtype == torch.float32,
          "product_sums: buf must be float32 [M, N]")
    return backend().product_sums(a, w, buf, bool(finished))


# ---- hyper-connections: the residual stream in S copies, x [T, S * E] float32 ------------------------------------
def _hc_ok(x, S, E, what):
    _need(x.dtype == torch.float32 and x.dim() == 2 and x.shape[1] == S * E and 1 <= S <= HC_MAX_STREAMS,
          f"{what}: the stream is float32 [T, copies * width] with at most {HC_MAX_STREAMS} copies")


HC_MAX_STREAMS = 8


def hc_spread(emb, x, S: int) -> None:
    """Every copy of the stream = emb [T, E] (float32)."""
    _hc_ok(x, S, emb.shape[1], "hc_spread")
    _need(emb.dtype == torch.float32 and emb.shape[0] == x.shape[0], "hc_spread: shape mismatch")
    backend().hc_spread(emb, x, int(S))


def hc_in_norm(x, S: int, in_w, rows, norm, out) -> None:
    """out[m] = norm(sum_s in_w[s] * x[row(m), s]): ``in_w`` float32 [S] (None: the plain sum), ``rows`` int32 [M] (None:
    every row), ``norm`` = the (alpha, w, b) of a Dynamic Tanh (None: no norm)."""
    E = out.shape[1]
    _hc_ok(x, S, E, "hc_in_norm")
    _need(in_w is None or (in_w.shape == (S,) and in_w.dtype == torch.float32), "hc_in_norm: in_w is float32 [copies]")
    _need(rows is None or (rows.dtype == torch.int32 and rows.shape[0] == out.shape[0]), "hc_in_norm: rows must be int32 [M]")
    _need(rows is not None or out.shape[0] == x.shape[0], "hc_in_norm: row count mismatch")
    if norm is not None:
        _dyt_ok(norm, E, "hc_in_norm")
    backend().hc_in_norm(x, int(S), in_w, rows, norm, out)


def hc_update(x, S: int, sources, mix, scale, hc_mix, hc_out, next_in=None, next_norm=None, out=None) -> None:
    """One sublayer's write-back.  y = scale .* (sum over ``sources`` of factor * (sum of the source's planes) + the
    weighted sum of ``mix``); then every copy d of the stream from the old copies: x'[d] = sum_s hc_mix[s, d] x[s] +
    hc_out[d] y; with ``out``, out = next_norm(sum_d next_in[d] x'[d]) from the same pass (next_in None: the plain sum;
    next_norm None: no norm).  ``sources``: up to two (planes float32 [splits, T, E], splits, factor); ``mix`` = (rows
    float32 [T * top, E], weights float32 [T, top], ids int32 [T, top] or None, n_real, h [T, E]): a choice whose id is at or
    above n_real stands for the sublayer's input h itself.  ``scale``: [E] or None."""
    T = x.shape[0]
    E = x.shape[1] // S
    _hc_ok(x, S, E, "hc_update")
    _need(len(sources) <= 2 and (sources or mix is not None), "hc_update: one or two sources, or a mix")
    for y, splits, _ in sources:
        _need(y.dtype == torch.float32 and splits >= 1 and y.numel() >= splits * T * E, "hc_update: a source is float32 [splits, T, E]")
    if mix is not None:
        my, mw, mids, n_real, mh = mix
        _need(mw.dim() == 2 and mw.shape[0] == T and my.shape == (T * mw.shape[1], E) and my.dtype == torch.float32
              and mw.dtype == torch.float32, "hc_update: mix = (float32 [T * top, E], float32 [T, top], ...)")
        _need(mids is None or (mids.shape == mw.shape and mids.dtype == torch.int32 and mh is not None and mh.shape == (T, E)),
              "hc_update: ids int32 [T, top] come with the sublayer's input [T, E]")
    _need(scale is None or scale.shape == (E,), "hc_update: scale is [E]")
    _need(hc_mix.shape == (S, S) and hc_out.shape == (S,) and hc_mix.dtype == hc_out.dtype == torch.float32,
          "hc_update: hc_mix float32 [S, S], hc_out float32 [S]")
    _need(next_in is None or (next_in.shape == (S,) and next_in.dtype == torch.float32), "hc_update: next_in is float32 [S]")
    _need(out is not None or (next_norm is None and next_in is None), "hc_update: the next norm needs an output")
    if out is not None:
        _need(out.shape == (T, E), "hc_update: output shape mismatch")
        if next_norm is not None:
            _dyt_ok(next_norm, E, "hc_update")
    backend().hc_update(x, int(S), [(y, int(n), float(f)) for y, n, f in sources], mix, scale, hc_mix, hc_out, next_in, next_norm, out)


# ---- recurrent mixers (float32 throughout) -----------------------------------------------------------------------
CONV_MAX_TAPS = 16
SCAN_MAX_HEAD = 512


def decay(z, splits: int, bias, rate, sign: float, out, H: int, d: int, z_stride: int = 0, z_col0: int = 0) -> None:
    """out[t, h, i] = exp(-rate[h] * softplus(sign * (z[t, h, i] + bias[h, i]))); z = the sum of ``splits`` float32 planes
    [T, z_stride] read from column ``z_col0`` on (z_stride 0: planes [T, H * d]).  sign +1 with rate = exp(A): exp(-exp(A)
    softplus(z + bias)); sign -1 with rate = 1 / tau: sigmoid(z + bias)^(1 / tau)."""
    T = out.shape[0]
    stride = int(z_stride) or H * d
    _need(out.shape == (T, H * d) and out.dtype == torch.float32 and z.dtype == torch.float32 and z.numel() >= splits * T * stride
          and z_col0 + H * d <= stride, "decay: z float32 [splits, T, stride], out float32 [T, H * d]")
    _need(rate.shape == (H,) and rate.dtype == torch.float32 and (bias is None or bias.shape == (H * d,)), "decay: rate float32 [H], bias [H * d]")
    backend().decay(z, int(splits), bias, rate, float(sign), out, int(H), int(d), stride, int(z_col0))


def short_conv(x, splits: int, w, carried, ctx, out, n_a: int, d_a: int, n_b: int, d_b: int, n_unit: int = 0, n_scaled: int = 0,
               scale: float = 1.0, unit_eps: float = 0.0) -> None:
    """Causal convolution over time per channel, then silu: x = the sum of ``splits`` float32 planes [T, C]; w [C, taps],
    the last column the current token's; ``carried`` [slots, taps - 1, C] float32 holds each request's last inputs
    (zeros for a new request) and is brought up to date.  A row is ``n_a`` heads of ``d_a`` channels, then ``n_b`` of
    ``d_b``: the first ``n_unit`` heads are then divided by sqrt(sum(x^2) + unit_eps), the first ``n_scaled`` of them also
    times ``scale``.  A request's tokens continue from its slot ``ctx.seq_slots``."""
    T, C = out.shape
    taps = w.shape[1]
    _need(C == n_a * d_a + n_b * d_b and w.shape[0] == C and 1 <= taps <= CONV_MAX_TAPS, "short_conv: channel count or taps mismatch")
    _need(out.dtype == torch.float32 and x.dtype == torch.float32 and x.numel() >= splits * T * C, "short_conv: x float32 [splits, T, C]")
    _need(carried.dtype == torch.float32 and carried.dim() == 3 and carried.shape[1:] == (max(taps - 1, 1), C)
          and carried.stride()[1:] == (C, 1), "short_conv: carried is float32 [slots, taps - 1, C]")
    _need(0 <= n_scaled <= n_unit <= n_a + n_b, "short_conv: scaled heads are among the unit heads")
    backend().short_conv(x, int(splits), w, carried, ctx, out, int(n_a), int(d_a), int(n_b), int(d_b), int(n_unit), int(n_scaled),
                         float(scale), float(unit_eps))


def linear_scan(q, k, v, a, beta_logit, q_scale: float, state, ctx, o, H: int, Hq: int, d: int, dv: int) -> None:
    """The gated linear recurrence per head, along each request's tokens from its slot's state: S <- diag(a) S + k u^T,
    o = S^T q * q_scale, with u = v, or, with ``beta_logit`` [T, H], u = sigmoid(beta) (v - (diag(a) S)^T k).  q, k: rows
    of ``Hq`` heads of ``d`` (head h reads head h // (H / Hq)); a: H heads of d; v, o: H heads of dv; all float32, each may
    be a column slice of a wider array (row strides are taken from the tensors).  ``state`` float32 [slots, H, dv, d]."""
    T = o.shape[0]
    for t, n, what in ((q, Hq * d, "q"), (k, Hq * d, "k"), (v, H * dv, "v"), (a, H * d, "a"), (o, H * dv, "o")):
        _need(t.dtype == torch.float32 and t.shape == (T, n) and t.stride(1) == 1, f"linear_scan: {what} is float32 [T, {n}] with unit column stride")
    _need(beta_logit is None or (beta_logit.dtype == torch.float32 and beta_logit.shape == (T, H) and beta_logit.stride(1) == 1),
          "linear_scan: beta_logit is float32 [T, H]")
    _need(H % Hq == 0 and d <= SCAN_MAX_HEAD and state.dtype == torch.float32 and state.shape[1:] == (H, dv, d)
          and state.stride()[1:] == (dv * d, d, 1),
          "linear_scan: state is float32 [slots, H, dv, d]")
    backend().linear_scan(q, k, v, a, beta_logit, float(q_scale), state, ctx, o, int(H), int(Hq), int(d), int(dv))


def gate_norm(o, w, eps: float, g, g_splits: int, g_stride: int, g_col0: int, gate: str, out, H: int, dv: int) -> None:
    """out[t, h] = o[t, h] / sqrt(mean(o[t, h]^2) + eps) * w * gate(g[t, h]); o float32 [T, H * dv]; w [dv]; g = the sum of
    ``g_splits`` float32 planes [T, g_stride] read from column ``g_col0`` on; gate "silu" or "sigmoid"."""
    T = o.shape[0]
    _need(o.dtype == torch.float32 and o.shape == (T, H * dv) and out.shape == (T, H * dv) and w.shape == (dv,), "gate_norm: shape mismatch")
    _need(g.dtype == torch.float32 and g.numel() >= g_splits * T * g_stride and g_col0 + H * dv <= g_stride and gate in ("silu", "sigmoid"),
          "gate_norm: g float32 [splits, T, stride]; gate silu or sigmoid")
    backend().gate_norm(o, w, float(eps), g, int(g_splits), int(g_stride), int(g_col0), 0 if gate == "silu" else 1, out, int(H), int(dv))


# ---- layer norm, token shift, gates, minGRU ----------------------------------------------------------------------
def layernorm(x, w, eps: float, out, rows: Optional[torch.Tensor] = None, center: bool = True) -> None:
    """out = (x - mean) / sqrt(var + eps) * w over rows of the float32 stream (``center`` False: x / sqrt(mean(x^2) + eps)
    * w); ``w`` float32 [E]; with ``rows`` (int32) only those rows, in that order."""
    _need(x.dtype == torch.float32 and x.dim() == 2, "layernorm: x must be float32 [N, E]")
    _need(w.shape == (x.shape[1],) and w.dtype == torch.float32 and out.shape[1] == x.shape[1], "layernorm: the weight is float32 [E]")
    _need(rows is None or (rows.dtype == torch.int32 and rows.shape[0] == out.shape[0]), "layernorm: rows must be int32 [M]")
    _need(rows is not None or out.shape[0] == x.shape[0], "layernorm: row count mismatch")
    backend().layernorm(x, w, float(eps), bool(center), out, rows)


def norm_shift(x, w, eps: float, center: bool, mu, state, ctx, out) -> None:
    """The norm of :func:`layernorm` with the token shift behind it: out[t] = h_t + (h_(t-1) - h_t) * mu, h = norm(x); the
    previous token's h comes from the step's previous row or, for a request's first token of the step, from the request's
    row of ``state`` (float32 [slots, E]), which then receives the h of the request's last token of the step."""
    T, E = x.shape
    _need(x.dtype == torch.float32 and out.shape == (T, E), "norm_shift: x must be float32 [T, E] and out [T, E]")
    _need(w.shape == (E,) and mu.shape == (E,) and w.dtype == mu.dtype == torch.float32, "norm_shift: weight and shift are float32 [E]")
    _need(state is not None and state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == E,
          "norm_shift: the state is float32 [slots, E]")
    backend().norm_shift(x, w, float(eps), bool(center), mu, state, ctx, out)


def gate_mul(a, g, g_splits: int, g_stride: int, g_col0: int, bias, gate: str, out) -> None:
    """out = a * sigmoid(g) or a * silu(g); ``g`` is the float32 sums of a product ([splits, T, g_stride], read from column
    ``g_col0`` on) plus ``bias`` (float32 [C]) where there is one; ``a`` and ``out`` [T, C] in the run's type."""
    _need(gate in ("silu", "sigmoid"), "gate_mul: gate is 'silu' or 'sigmoid'")
    _need(a.shape == out.shape and a.dtype == out.dtype and a.dim() == 2, "gate_mul: a and out must agree")
    _need(g.dtype == torch.float32 and g_col0 + a.shape[1] <= g_stride and g.numel() >= g_splits * a.shape[0] * g_stride,
          "gate_mul: the gate's sums are float32 [splits, T, g_stride]")
    _need(bias is None or (bias.shape == (a.shape[1],) and bias.dtype == torch.float32), "gate_mul: the bias is float32 [C]")
    backend().gate_mul(a, g, int(g_splits), int(g_stride), int(g_col0), bias, gate, out)


def mingru_scan(row, splits: int, bias_z, bias_x, state, ctx, out, W: int) -> None:
    """minGRU over the step's tokens, request by request from each request's state: ``row`` is the float32 sums of the
    product [update gate | candidate | output gate] ([splits, T, 3 W]); z = sigmoid(a + bias_z), u = b + bias_x,
    cand = u + 1/2 where u >= 0 and sigmoid(u) where u < 0, S <- (1 - z) S + z cand, out = S * silu(g).  ``state`` float32
    [slots, W] holds S between steps; ``out`` [T, W] in the run's type."""
    _need(row.dtype == torch.float32 and row.numel() >= splits * out.shape[0] * 3 * W and out.shape[1] == W,
          "mingru_scan: rows are float32 [splits, T, 3 W]")
    _need(state is not None and state.dtype == torch.float32 and state.dim() == 2 and state.shape[1] == W,
          "mingru_scan: the state is float32 [slots, W]")
    _need(all(b is None or b.shape == (W,) for b in (bias_z, bias_x)), "mingru_scan: biases are [W]")
    backend().mingru_scan(row, int(splits), bias_z, bias_x, state, ctx, out, int(W))


def argmax(logits: torch.Tensor, out: torch.Tensor) -> None:
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.shape == (logits.shape[0],),
          "argmax: logits float32 [M, V], out int32 [M]")
    backend().argmax(logits, out)


def sample(logits, temps, top_ks, top_ps, min_ps, uniforms, out) -> None:
    """One token per row; greedy where temps <= 0, else top-k / min-p / top-p sampling with the row's draw."""
    M = logits.shape[0]
    _need(logits.dtype == torch.float32 and out.dtype == torch.int32 and out.shape == (M,), "sample: bad logits / out")
    for t, dt in ((temps, torch.float32), (top_ks, torch.int32), (top_ps, torch.float32), (min_ps, torch.float32),
                  (uniforms, torch.float32)):
        _need(t.dtype == dt and t.shape == (M,), "sample: per-row parameters must be [M]")
    backend().sample(logits, temps, top_ks, top_ps, min_ps, uniforms, out)


class DeviceFault(RuntimeError):
    """A kernel recorded an error in the device error word; what it computed is not to be trusted."""

    def __init__(self, word: int):
        self.word = int(word)
        super().__init__("a kernel met " + "; ".join(v for k, v in ERROR_BITS.items() if word & k))


def check_device_errors() -> None:
    """Raise if any kernel recorded an error since the last check (synchronises the stream)."""
    b = backend()
    word = b.error_word() if hasattr(b, "error_word") else 0
    if word:
        raise DeviceFault(word)
