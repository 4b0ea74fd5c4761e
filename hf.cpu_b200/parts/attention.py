"""Grouped-query attention over the paged cache.

Per token: ``q, k, v = xn W{q,k,v}^T + b``; rotary on q and k; k (after rotation) and v go into
the cache at the token's slot; head h attends with the key/value head ``h // (H/G)`` over keys
``0 .. pos`` (or the last ``window`` of them), scores scaled by ``1/sqrt(head_dim)`` after the
dot, softmax, weighted values; ``out = att Wo^T`` is added to the residual
(src/model.c:581-609, :499-528).  q, k and v are one matrix product over concatenated rows
(src/model.c:581-585 runs the three jobs in one pass).

Options beyond the reference's layer, each a constructor argument: ``scale`` (the factor on the scores, where it is
not ``1/sqrt(head_dim)``), ``v_head_dim`` (value heads of another size than query/key heads), ``qk_norm_eps`` (after
the rotation every query and key head is divided by its root mean square, ``x / sqrt(mean(x^2) + eps)``, no weight;
the cache holds the keys in that form), and ``own_kv=False`` (the layer has no key and value projections: its queries
attend over the cache of the schedule entry it is pointed at, which a layer with the same head counts and rotation
has filled).  ``qk_norm_weights`` = {"q": suffix, "k": suffix} names one weight vector [head_dim] each, shared by the heads,
that the normed queries and keys are multiplied by.  ``chunk`` > 0 replaces the causal mask by a chunked one: a query
sees the earlier keys of its own chunk of that many positions, chunks counted from position 0 of the request.
``v_mix``: "first" marks the first layer of a model whose values are mixed into later layers' (its own values stay as
they are, and it leaves them behind for the step's other layers); "later" replaces a layer's values by
``(1 - lambda) v + lambda v_first`` before they are cached, ``lambda`` being the scalar tensor ``v_mix_tensor`` and
``v_first`` the same token's values of the "first" layer, whose value heads must have the same count and size.
``sink``: "learned" adds exp(sink_h) to the softmax's denominator, sink_h a stored number per head (tensor ``sink_tensor``)
that has no key, no value and no scale; "zero" does the same with a score of 0 (one is added to the denominator).
``distance_slope_exp`` = c: ``2^(-c (h + 1) / H) * (i - j)`` is taken off the score of query i and key j in head h.
``values_are_keys``: the layer has no value projection, a key as it is cached also serves as its value (one array of
rows in the cache).  A rotary encoding with the pairing "interleaved" turns the dimensions (2i, 2i + 1) together.
``head_scale_tensor`` names a stored number per head by which the head's scaled scores are multiplied; ``softcap`` = c > 0
turns a score s into ``c tanh(s / c)`` (after the factors, before the softmax).  ``out_gate`` = {"tensor": name, "kind":
"sigmoid" | "silu"}: the concatenated heads' outputs are multiplied element by element by ``kind(W_gate h)`` before the
output product, ``W_gate`` [H * v_head_dim, hidden] reading the same input as the other projections.
"""
from __future__ import annotations

import math

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .base import CacheSpec, Mixer, register_part


class OutputProduct:
    """What mixers that end in one product over the concatenated heads share: ``self._attend(ctx, xn, cache,
    write_cache)`` gives the heads' outputs, ``self.w_o`` / ``self.b_o`` carry them back to the stream."""

    def forward(self, ctx, xn, residual, cache, state, write_cache, accumulate=True):
        """``accumulate=False`` stores the sublayer's output in ``residual`` (float32) instead of adding it."""
        att = self._attend(ctx, xn, cache, write_cache)
        with kernels.phase("wo"):
            kernels.linear(att, self.w_o, self.b_o, residual, accumulate=accumulate)

    def forward_into_norm(self, ctx, xn, cache, state, write_cache, y_buf, residual, post, next_norm, out):
        """residual += post(mixer output), the output product handed to the norm (see ``DynamicTanh.add_product_into``)."""
        att = self._attend(ctx, xn, cache, write_cache)
        with kernels.phase("wo"):
            return post.add_product_into(att, self.w_o, self.b_o, y_buf, residual, next_norm, out)

    def forward_sources(self, ctx, xn, cache, state, write_cache, y_buf, finished=False):
        """The mixer's output as float32 sums for a block that adds it to the stream in a pass of its own: [(planes,
        splits)] of the output product (``y_buf`` [T, E] float32 holds it where it is not split, and always with
        ``finished``)."""
        att = self._attend(ctx, xn, cache, write_cache) if state is None else self._attend(ctx, xn, cache, write_cache, state)
        with kernels.phase("wo"):
            if self.b_o is not None:
                kernels.linear(att, self.w_o, self.b_o, y_buf, accumulate=False)
                return [(y_buf, 1)]
            return [kernels.product_sums(att, self.w_o, y_buf, finished)]

    def forward_then_norm(self, ctx, xn, residual, cache, state, write_cache, norm, out):
        args = norm.fused_args()
        if args is None:
            self.forward(ctx, xn, residual, cache, state, write_cache)
            return False
        att = self._attend(ctx, xn, cache, write_cache)
        with kernels.phase("wo"):
            kernels.linear_residual_norm(att, self.w_o, self.b_o, residual, args[0], args[1], out, **(args[2] if len(args) > 2 else {}))
        return True


class PagedAttention(OutputProduct, Mixer):
    graph_safe = True
    V_FIRST = "attn_v_first"          # the scratch buffer in which a step's first value-mixing layer leaves its values

    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int,
                 qkv_bias: bool, out_bias: bool, window: int, position, prefix: str,
                 positions=None, names=None, scale=None, v_head_dim=None, qk_norm_eps=None, own_kv: bool = True,
                 bias_suffix: str = ".bias", weight_suffix: str = ".weight", qk_norm_weights=None, chunk: int = 0,
                 v_mix=None, v_mix_tensor: str = "vmix", sink=None, sink_tensor: str = "sink", distance_slope_exp=None,
                 values_are_keys: bool = False, head_scale_tensor=None, softcap=None, out_gate=None, **_):
        self.E, self.H, self.G, self.d = int(hidden_size), int(num_heads), int(num_kv_heads), int(head_dim)
        if self.H % self.G:
            raise UnsupportedError(f"unsupported attention geometry: {self.H} heads over {self.G} key/value heads")
        self.dv = int(v_head_dim) if v_head_dim else self.d
        self.values_are_keys = bool(values_are_keys)
        if self.values_are_keys and (self.dv != self.d or v_mix or not own_kv):
            raise UnsupportedError("keys that serve as values have their size, are not mixed, and are the layer's own")
        if sink not in (None, "zero", "learned"):
            raise UnsupportedError(f"attention sink '{sink}' is not known (zero, learned)")
        self.sink = sink
        self.slope_exp = None if distance_slope_exp is None else float(distance_slope_exp)
        self.qk_norm_eps = None if qk_norm_eps is None else float(qk_norm_eps)
        self.own_kv = bool(own_kv)
        # the q|k|v tail that normalises heads also takes the other two options; the reference's layer keeps its own
        self.chunk = int(chunk or 0)
        if v_mix not in (None, "first", "later"):
            raise UnsupportedError(f"v_mix '{v_mix}' is not known (first, later)")
        self.v_mix = v_mix
        if self.v_mix and not self.own_kv:
            raise UnsupportedError("a layer without values of its own cannot mix them")
        if qk_norm_weights and self.qk_norm_eps is None:
            raise UnsupportedError("weights on the query and key norm need that norm (qk_norm_eps)")
        self.softcap = float(softcap) if softcap else 0.0
        if self.softcap < 0:
            raise UnsupportedError("attention: the cap on the scores must be positive")
        self.gate_kind = (out_gate or {}).get("kind", "sigmoid") if out_gate else None
        if self.gate_kind not in (None, "sigmoid", "silu"):
            raise UnsupportedError(f"attention: output gate '{self.gate_kind}' is not known (sigmoid, silu)")
        self.general = (self.qk_norm_eps is not None or self.dv != self.d or not self.own_kv or self.v_mix is not None
                        or self.values_are_keys or self.sink is not None or self.slope_exp is not None
                        or head_scale_tensor is not None or self.softcap > 0 or out_gate is not None
                        or getattr((positions or {}).get(position), "pairing", "half") != "half")
        if self.general:
            if not (0 < self.d <= kernels.MAX_HEAD_DIM and 0 < self.dv <= kernels.MAX_HEAD_DIM):
                raise UnsupportedError(f"head sizes {self.d} / {self.dv} are not supported (1 to {kernels.MAX_HEAD_DIM})")
        else:
            kernels.check_head_dim(self.d)
        self.wsuf, self.bsuf = weight_suffix, bias_suffix
        self.qkv_bias, self.out_bias, self.window = bool(qkv_bias), bool(out_bias), int(window)
        self.mask = kernels.mask_code(self.window, self.chunk)
        self.rotary = (positions or {}).get(position) if position else None
        if position and self.rotary is None:
            raise UnsupportedError(f"attention names position encoding '{position}', which the plan does not define")
        self.pairing = getattr(self.rotary, "pairing", "half") if self.rotary is not None else "half"
        n = {"q": "q_proj", "k": "k_proj", "v": "v_proj", "o": "o_proj"}
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.norm_names = {k: f"{prefix}.{v}" for k, v in (qk_norm_weights or {}).items()}
        if self.norm_names and set(self.norm_names) != {"q", "k"}:
            raise UnsupportedError("qk_norm_weights names one weight for q and one for k")
        self.v_mix_name = f"{prefix}.{v_mix_tensor}" if self.v_mix else None
        self.sink_name = f"{prefix}.{sink_tensor}" if self.sink == "learned" else None
        self.head_scale_name = f"{prefix}.{head_scale_tensor}" if head_scale_tensor else None
        self.gate_name = f"{prefix}.{out_gate['tensor']}" if out_gate else None
        self.sinks = self.slopes = self.head_scales = None          # float32 [H]
        self.w_gate = None
        self.scale = 1.0 / math.sqrt(self.d) if scale is None else float(scale)
        self.w_qkv = self.b_qkv = self.w_o = self.b_o = None
        self.norm_w = None              # (q weight, k weight), float32
        self.v_lambda = 0.0

    @property
    def QD(self):
        return self.H * self.d

    @property
    def KD(self):
        return self.G * self.d

    @property
    def VD(self):
        return 0 if self.values_are_keys else self.G * self.dv

    @property
    def OD(self):
        return self.H * self.dv

    def cache_spec(self):
        return CacheSpec(self.G, self.d, self.window, 0 if self.dv == self.d else self.dv, chunk=self.chunk,
                         values_in_keys=self.values_are_keys)

    def step_arrays_key(self):
        return ("paged_attention_tiles", self.H // self.G)

    def step_arrays(self, batch):
        # the tile lists of the attention kernels: how they cut the step's tokens is the kernels' business
        return kernels.attention_step_arrays(batch.q_lens, self.H // self.G)

    def _projections(self):
        """(key of ``names``, output features) of the projections in the fused product's row order."""
        if not self.own_kv:
            return [("q", self.QD)]
        return [("q", self.QD), ("k", self.KD)] + ([] if self.values_are_keys else [("v", self.VD)])

    def tensor_specs(self):
        s = [TensorSpec(self.names[x] + self.wsuf, (n, self.E)) for x, n in self._projections()]
        s.append(TensorSpec(self.names["o"] + self.wsuf, (self.E, self.OD)))
        if self.qkv_bias:
            s += [TensorSpec(self.names[x] + self.bsuf, (n,)) for x, n in self._projections()]
        if self.out_bias:
            s.append(TensorSpec(self.names["o"] + self.bsuf, (self.E,)))
        s += [TensorSpec(self.norm_names[x], (self.d,), init="norm") for x in sorted(self.norm_names)]
        if self.v_mix_name:
            s.append(TensorSpec(self.v_mix_name, (), init="half"))       # the first layer's is stored too, and unused
        if self.sink_name:
            s.append(TensorSpec(self.sink_name, (self.H,)))
        if self.head_scale_name:
            s.append(TensorSpec(self.head_scale_name, (self.H,), init="norm"))
        if self.gate_name:
            s.append(TensorSpec(self.gate_name + self.wsuf, (self.OD, self.E)))
        return s

    def bind(self, tensors, run_dtype, device):
        # q, k and v rows go straight into the one matrix the product reads, a tensor at a time
        self.w_qkv = fused_rows(tensors, [self.names[x] + self.wsuf for x, _ in self._projections()], device)
        if self.qkv_bias:
            self.b_qkv = fused_rows(tensors, [self.names[x] + self.bsuf for x, _ in self._projections()], device)
        self.w_o = tensors[self.names["o"] + self.wsuf].contiguous()
        if self.out_bias:
            self.b_o = tensors[self.names["o"] + self.bsuf].contiguous()
        if self.norm_names:
            self.norm_w = tuple(tensors[self.norm_names[x]].to(torch.float32).contiguous() for x in ("q", "k"))
        if self.v_mix_name:
            lam = tensors[self.v_mix_name]
            self.v_lambda = float(lam.to(torch.float32).reshape(-1)[0].item()) if self.v_mix == "later" else 0.0
        if self.sink_name:
            self.sinks = tensors[self.sink_name].to(torch.float32).contiguous()
        if self.head_scale_name:
            self.head_scales = tensors[self.head_scale_name].to(torch.float32).contiguous()
        if self.gate_name:
            self.w_gate = tensors[self.gate_name + self.wsuf].contiguous()
        if self.slope_exp is not None:
            h = torch.arange(1, self.H + 1, dtype=torch.float64)
            self.slopes = torch.pow(2.0, -self.slope_exp * h / self.H).to(torch.float32).to(device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_qkv, self.b_qkv, self.w_o, self.b_o, self.w_gate)
                   if w is not None)

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        seen = 0                        # (query, key) pairs: token i of n new ones over a history of m sees m - n + i + 1
        for n, m in zip(q_lens, kv_lens):
            for_all = n * (m - n) + n * (n + 1) // 2
            if self.window > 0:
                for_all = sum(min(self.window, m - n + i + 1) for i in range(n)) if m > self.window else for_all
            elif self.chunk > 0:
                for_all = sum((m - n + i) % self.chunk + 1 for i in range(n))
            seen += for_all
        gate = self.w_gate.numel() if self.w_gate is not None else 0
        return 2.0 * T * (self.w_qkv.numel() + self.w_o.numel() + gate) + 2.0 * (self.QD + self.OD) * seen

    def _attend(self, ctx, xn, cache, write_cache):
        T = xn.shape[0]
        q = ctx.buf("attn_q", (T, self.QD), xn.dtype)
        meta = ctx.group_meta(cache.group)
        cos_sin = self.rotary.cos_sin if self.rotary is not None else None
        n_rot = self.rotary.n_rot if self.rotary is not None else 0
        if write_cache and not self.own_kv:
            raise ValueError("a layer without key and value projections must read another schedule entry's cache")
        if self.general:
            # the product's sums stay float32 until rotation and the heads' normalisation are done
            G = self.G if self.own_kv else 0
            dv_row = 0 if self.values_are_keys else self.dv
            qkv = ctx.buf("attn_qkv32", (T, self.QD + G * (self.d + dv_row)), torch.float32)
            mix = None
            if self.v_mix:
                first = ctx.buf(self.V_FIRST, (T, self.VD), torch.float32)
                mix = (first, 1 if self.v_mix == "first" else 2, self.v_lambda)
            with kernels.phase("qkv"):
                kernels.linear_rope_norm_kv(xn, self.w_qkv, self.b_qkv, qkv, cos_sin, n_rot, ctx.positions,
                                            meta.slots if write_cache else None, q, cache.k, None if self.values_are_keys else cache.v,
                                            self.H, G, self.d, dv_row, self.qk_norm_eps, norm_weights=self.norm_w, value_mix=mix,
                                            pairing=self.pairing)
        else:
            qkv = ctx.buf("attn_qkv", (T, self.QD + 2 * self.KD), xn.dtype)
            with kernels.phase("qkv"):
                kernels.linear_rope_kv(xn, self.w_qkv, self.b_qkv, qkv, cos_sin, n_rot, ctx.positions,
                                       meta.slots if write_cache else None, q, cache.k, cache.v, self.H, self.G, self.d)
        att = ctx.buf("attn_out", (T, self.OD), xn.dtype)
        with kernels.phase("attn"):
            kernels.paged_attention(q, cache.k, None if self.values_are_keys else cache.v, meta, ctx, self.H, self.G, self.d,
                                    self.mask, self.scale, att, tiles=ctx.arrays(self.step_arrays_key()), dv=self.dv,
                                    values_in_keys=self.values_are_keys, sinks=self.sinks, zero_sink=self.sink == "zero",
                                    slopes=self.slopes, head_scales=self.head_scales, softcap=self.softcap)
        if self.w_gate is not None:
            # the gate reads the mixer's input as the projections do; its sums stay float32 up to the sigmoid
            with kernels.phase("qkv"):
                g, splits = kernels.product_sums(xn, self.w_gate, ctx.buf("attn_gate32", (T, self.OD), torch.float32))
            with kernels.phase("attn"):
                kernels.gate_mul(att, g, splits, self.OD, 0, None, self.gate_kind, att)
        return att


register_part("mixer", "paged_attention", PagedAttention)
