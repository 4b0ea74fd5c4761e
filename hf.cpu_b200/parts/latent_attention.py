"""Latent attention: queries, keys and values all pass through low-rank latents, and only the key/value latent is cached.

Per token, with h the mixer's input:

* ``[a | b | r] = h W_down^T``: ``a`` (``q_rank``) and ``b`` (``kv_rank``) are normed (``x / sqrt(mean(x^2) + eps) * w``)
  into the query latent ``cq`` and the key/value latent ``c``; ``r`` (``rot_dim``) is rotated by the token's position and
  is the one rotated key part that all heads share.  The cache row of a token is ``[c | r]``: one "head" of
  ``kv_rank + rot_dim`` values, no array of values.
* ``q = cq W_uq^T``: per head ``dim`` plain and ``rot_dim`` rotated dimensions.
* A head's plain key is ``Wuk_h c`` and its value ``Wuv_h c``.  Neither is ever made: since
  ``q_plain . (Wuk_h c) = (Wuk_h^T q_plain) . c``, the head's query is carried into the latent space and attention runs over
  the cached rows themselves, as attention with one shared key/value head whose value is the first ``kv_rank`` elements
  of its key: ``score = ([Wuk_h^T q_plain | q_rot] . [c | r]) * scale``, ``out_h = Wuv_h (sum_j p_j c_j)``.
* ``out = concat(out_h) W_o^T`` is added to the residual.

Where the cached row has a size the tiled tensor-core attention kernels take (they want value heads as wide as key
heads), the whole row serves as the value: the rotated columns of the weighted sum are computed and not read.  Other
sizes take the plain kernel, which reads a value as the first ``kv_rank`` elements of its key.

The mask is a sliding window (``window`` > 0) or causal (0).  The rotation takes its table from a shared position
encoding (which may be scaled for long contexts).  The kernels turn dimensions (2i, 2i + 1) together.  An encoding with
the pairing "half" (dimension i with i + rot_dim/2) is served by them too: the rotated part enters the scores only as
``q_rot . k_rot``, which does not change when both are permuted alike, so the rows of the two projections that make
the rotated parts are reordered once, when the weights are bound (i -> 2i, i + rot_dim/2 -> 2i + 1), and the cache
holds the rotated key part in that order.  The reference has no such layer; the
nearest thing in it is the grouped attention of src/model.c:581-609.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .attention import OutputProduct
from .base import CacheSpec, Mixer, register_part


class LatentAttention(OutputProduct, Mixer):
    graph_safe = True

    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, q_rank: int,
                 kv_rank: int, scale: float, norm_eps: float, window: int, position, prefix: str, positions=None,
                 names=None, **_):
        self.E, self.H, self.d, self.dr, self.dv = (int(hidden_size), int(num_heads), int(head_dim), int(rot_dim),
                                                    int(v_head_dim))
        self.Qr, self.R = int(q_rank), int(kv_rank)
        self.scale, self.eps, self.window = float(scale), float(norm_eps), int(window)
        self.row = self.R + self.dr                     # what a token holds in the cache, and a head's query over it
        if min(self.E, self.H, self.d, self.dv, self.Qr, self.R) < 1 or self.dr < 0 or self.dr % 2:
            raise UnsupportedError("latent attention: sizes must be positive and the rotated part even")
        if self.row > kernels.MAX_LATENT_ROW:
            raise UnsupportedError(f"latent attention: kv_rank + rot_dim = {self.row} exceeds {kernels.MAX_LATENT_ROW}")
        self.rotary = (positions or {}).get(position) if position else None
        if self.dr and self.rotary is None:
            raise UnsupportedError(f"latent attention names position encoding '{position}', which the plan does not define")
        if self.rotary is not None and self.rotary.n_rot != self.dr:
            raise UnsupportedError("latent attention rotates its whole rotated part")
        self.reorder = self.rotary is not None and self.rotary.pairing == "half"
        n = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o"}
        n.update(names or {})
        self.names = {k: f"{prefix}.{v}" for k, v in n.items()}
        self.w_down = self.w_uq = self.w_ukt = self.w_uv = self.w_o = self.b_o = None
        self.norm_q = self.norm_kv = None

    def cache_spec(self):
        return CacheSpec(1, self.row, self.window, values_in_keys=True)

    def step_arrays_key(self):
        return ("paged_attention_tiles", self.H)            # all heads share the one cached row: one group of H heads

    def step_arrays(self, batch):
        return kernels.attention_step_arrays(batch.q_lens, self.H)

    def tensor_specs(self):
        n = self.names
        return [TensorSpec(n["dq"], (self.Qr, self.E)), TensorSpec(n["dq_norm"], (self.Qr,), init="norm"),
                TensorSpec(n["uq"], (self.H * (self.d + self.dr), self.Qr)),
                TensorSpec(n["dkv"], (self.R + self.dr, self.E)), TensorSpec(n["dkv_norm"], (self.R,), init="norm"),
                TensorSpec(n["uk"], (self.H * self.d, self.R)), TensorSpec(n["uv"], (self.H * self.dv, self.R)),
                TensorSpec(n["o"], (self.E, self.H * self.dv))]

    def bind(self, tensors, run_dtype, device):
        n = self.names
        # both down projections are one product: rows [query latent | key/value latent | rotated key part]
        self.w_down = fused_rows(tensors, [n["dq"], n["dkv"]], device)
        w_uq = tensors[n["uq"]].contiguous()
        if self.reorder:
            # "half" pairing: the rotated parts' rows into the order the kernels rotate in
            half = self.dr // 2
            order = torch.stack([torch.arange(half), torch.arange(half) + half], dim=1).reshape(-1).to(self.w_down.device)
            tail = self.w_down[self.Qr + self.R:].clone()
            self.w_down[self.Qr + self.R:] = tail[order]
            per_head = w_uq.reshape(self.H, self.d + self.dr, self.Qr).clone()
            per_head[:, self.d:] = per_head[:, self.d:][:, order.to(per_head.device)]
            w_uq = per_head.reshape(self.H * (self.d + self.dr), self.Qr).contiguous()
        self.norm_q = tensors[n["dq_norm"]].to(torch.float32).contiguous()
        self.norm_kv = tensors[n["dkv_norm"]].to(torch.float32).contiguous()
        self.w_uq = w_uq
        # a head's key expansion [d, kv_rank] is applied transposed, to the query: kept as [H, kv_rank, d]
        self.w_ukt = tensors[n["uk"]].reshape(self.H, self.d, self.R).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].reshape(self.H, self.dv, self.R).contiguous()
        self.w_o = tensors[n["o"]].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_down, self.w_uq, self.w_ukt, self.w_uv, self.w_o))

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        seen = 0
        for n, m in zip(q_lens, kv_lens):
            for i in range(n):
                pos = m - n + i
                seen += min(self.window, pos + 1) if self.window > 0 else pos + 1
        products = self.w_down.numel() + self.w_uq.numel() + self.w_ukt.numel() + self.w_uv.numel() + self.w_o.numel()
        return 2.0 * T * products + 2.0 * self.H * (self.row + self.R) * seen

    def _attend(self, ctx, xn, cache, write_cache):
        if not write_cache:
            raise ValueError("latent attention keeps its own cache")
        T, dt = xn.shape[0], xn.dtype
        meta = ctx.group_meta(cache.group)
        cos_sin = self.rotary.cos_sin if self.rotary is not None else None
        cq = ctx.buf("lat_cq", (T, self.Qr), dt)
        q_plain = ctx.buf("lat_q_plain", (T, self.H * self.d), dt)
        q_att = ctx.buf("lat_q", (T, self.H * self.row), dt)
        with kernels.phase("qkv"):
            down = ctx.buf("lat_down32", (T, self.Qr + self.row), torch.float32)
            kernels.linear_latent_split(xn, self.w_down, down, self.norm_q, self.norm_kv, self.eps, cos_sin, ctx.positions,
                                        meta.slots, cq, cache.k, self.Qr, self.R, self.dr)
            q32 = ctx.buf("lat_q32", (T, self.H * (self.d + self.dr)), torch.float32)
            kernels.linear_latent_query_absorb(cq, self.w_uq, q32, cos_sin, ctx.positions, self.w_ukt, q_plain, q_att, self.H,
                                               self.d, self.dr)
        whole_row = kernels.tiled_attention_takes(dt, self.row, meta.block_size)
        out_row = self.row if whole_row else self.R
        lat = ctx.buf("lat_out", (T, self.H * out_row), dt)
        with kernels.phase("attn"):
            if whole_row:
                kernels.paged_attention(q_att, cache.k, cache.k, meta, ctx, self.H, 1, self.row, kernels.mask_code(self.window),
                                        self.scale, lat, tiles=ctx.arrays(self.step_arrays_key()))
            else:
                kernels.paged_attention(q_att, cache.k, None, meta, ctx, self.H, 1, self.row, kernels.mask_code(self.window),
                                        self.scale, lat, dv=self.R, values_in_keys=True)
        att = ctx.buf("lat_heads", (T, self.H * self.dv), dt)
        with kernels.phase("attn"):
            kernels.headwise_linear(lat, self.w_uv, att, self.H, out_row, self.dv)
        return att


register_part("mixer", "latent_attention", LatentAttention)
