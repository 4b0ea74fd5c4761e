"""Mixers that keep state of fixed size per request instead of keys and values per token: a matrix per head (the two
gated linear recurrences below) or a vector (``mingru``, at the end).

Both run the gated linear recurrence per head, with a state S [d, dv] that starts at zero for a new request, lives in
float32 in the request's state slot and is carried from token to token:

* ``gated_linear_attention``: ``S <- diag(a) S + k v^T``, ``o = S^T q``, with ``q = Wq h * d^(-1/2)``, ``k = Wk h``,
  ``v = Wv h`` and a decay per head and key channel ``a = sigmoid(Wa2 (Wa1 h) + b)^(1 / tau)``; every head's o is
  divided by its root mean square, multiplied by one weight vector shared by the heads and by ``silu(Wg h)``, and
  projected by ``Wo``.
* ``gated_delta_rule``: ``S <- diag(a) S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q`` (the read-out sees the
  token's own write), with q, k, v each through a short causal convolution over time per channel and silu, q and k then
  of unit length per head (``x / sqrt(sum x^2 + unit_eps)``) and q times ``d^(-1/2)``; ``beta = sigmoid(Wb h)`` per head;
  ``a = exp(-exp(A_h) softplus(Wa2 (Wa1 h) + dt_bias))`` per head and key channel; grouped heads (value head h reads
  query/key head ``h // (H / G)``); o normed as above and multiplied by ``sigmoid(Wg2 (Wg1 h))``, then ``Wo``.  The
  convolution's last ``taps - 1`` inputs are part of the request's state.

Everything between the products' float32 sums and the output product's input is float32: decays, softplus and
exponentials, gates, unit lengths, the state and the norm.  (The reference has neither; its design notes name recurrent
layer state as a per-sequence block of fixed size, docs/DESIGN-SPACE.md:105.)
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .attention import OutputProduct
from .base import Mixer, StateSpec, register_part


class _Recurrent(OutputProduct, Mixer):
    graph_safe = True
    # A prompt's walk runs for milliseconds on a few blocks.  With launches that overlap, a warmed-up process stopped
    # making progress in the prompt steps of layers of width 2,048 (queued back to back); without the overlap it does not.
    launch_overlap_safe = False
    b_o = None

    def _t(self, name):
        return f"{self.prefix}.{self.nm[name]}"

    def forward(self, ctx, xn, residual, cache, state, write_cache, accumulate=True):
        att = self._attend(ctx, xn, cache, write_cache, state)
        with kernels.phase("wo"):
            kernels.linear(att, self.w_o, None, residual, accumulate=accumulate)

    def forward_into_norm(self, ctx, xn, cache, state, write_cache, y_buf, residual, post, next_norm, out):
        att = self._attend(ctx, xn, cache, write_cache, state)
        with kernels.phase("wo"):
            return post.add_product_into(att, self.w_o, None, y_buf, residual, next_norm, out)

    def forward_then_norm(self, ctx, xn, residual, cache, state, write_cache, norm, out):
        args = norm.fused_args()
        if args is None:
            self.forward(ctx, xn, residual, cache, state, write_cache)
            return False
        att = self._attend(ctx, xn, cache, write_cache, state)
        with kernels.phase("wo"):
            kernels.linear_residual_norm(att, self.w_o, None, residual, args[0], args[1], out, **(args[2] if len(args) > 2 else {}))
        return True

    def _low_rank_sums(self, ctx, xn, w1, w2, tag):
        """float32 sums of ``w2 (w1 xn)``: (planes, splits).  The inner result passes in the run's type."""
        T = xn.shape[0]
        low = ctx.buf(f"rec_low_{tag}", (T, w1.shape[0]), xn.dtype)
        kernels.linear(xn, w1, None, low, accumulate=False)
        return kernels.product_sums(low, w2, ctx.buf(f"rec_z_{tag}", (T, w2.shape[0]), torch.float32))


class GatedLinearAttention(_Recurrent):
    def __init__(self, hidden_size: int, num_heads: int, head_dim: int, v_head_dim: int, tau: float, norm_eps: float, prefix: str,
                 decay_rank: int = -1, names=None, **_):
        self.E, self.H, self.d, self.dv = int(hidden_size), int(num_heads), int(head_dim), int(v_head_dim)
        self.tau, self.eps, self.prefix = float(tau), float(norm_eps), prefix
        self.decay_rank = int(decay_rank)          # -1: the inner size of the decay's two products is the stored tensors'
        if not self.tau > 0:
            raise UnsupportedError("gated linear attention: tau must be positive")
        if self.d > kernels.SCAN_MAX_HEAD:
            raise UnsupportedError(f"gated linear attention: key heads above {kernels.SCAN_MAX_HEAD} are not supported")
        n = {"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a_bias": "a2.b"}
        n.update(names or {})
        self.nm = n
        self.w_in = self.w_o = self.w_a1 = self.w_a2 = self.a_bias = self.norm_w = self.rate = None

    def state_spec(self):
        return StateSpec((self.H * self.dv * self.d,))

    def tensor_specs(self):
        KD, VD = self.H * self.d, self.H * self.dv
        s = [TensorSpec(self._t("q"), (KD, self.E)), TensorSpec(self._t("k"), (KD, self.E)), TensorSpec(self._t("v"), (VD, self.E)),
             TensorSpec(self._t("g"), (VD, self.E)), TensorSpec(self._t("o"), (self.E, VD)),
             TensorSpec(self._t("norm"), (self.dv,), init="norm"), TensorSpec(self._t("a_bias"), (KD,))]
        s += [TensorSpec(self._t("a1"), (self.decay_rank, self.E)), TensorSpec(self._t("a2"), (KD, self.decay_rank))]
        return s

    def bind(self, tensors, run_dtype, device):
        self.w_in = fused_rows(tensors, [self._t(x) for x in ("q", "k", "v", "g")], device)
        self.w_o = tensors[self._t("o")].contiguous()
        self.w_a1, self.w_a2 = tensors[self._t("a1")].contiguous(), tensors[self._t("a2")].contiguous()
        self.a_bias, self.norm_w = tensors[self._t("a_bias")].contiguous(), tensors[self._t("norm")].contiguous()
        self.rate = torch.full((self.H,), 1.0 / self.tau, dtype=torch.float32, device=device)

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o, self.w_a1, self.w_a2))

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        return 2.0 * T * (self.w_in.numel() + self.w_o.numel() + self.w_a1.numel() + self.w_a2.numel()) + 6.0 * T * self.H * self.d * self.dv

    def _attend(self, ctx, xn, cache, write_cache, state):
        T = xn.shape[0]
        KD, VD = self.H * self.d, self.H * self.dv
        C = 2 * KD + 2 * VD
        with kernels.phase("qkv"):
            z, z_splits = self._low_rank_sums(ctx, xn, self.w_a1, self.w_a2, "a")
            a = ctx.buf("rec_decay", (T, KD), torch.float32)
            # sigmoid(z)^(1 / tau) = exp(-(1 / tau) softplus(-z))
            kernels.decay(z, z_splits, self.a_bias, self.rate, -1.0, a, self.H, self.d)
            row, _ = kernels.product_sums(xn, self.w_in, ctx.buf("rec_in", (T, C), torch.float32), finished=True)
        o = ctx.buf("rec_o", (T, VD), torch.float32)
        with kernels.phase("attn"):
            kernels.linear_scan(row[:, :KD], row[:, KD:2 * KD], row[:, 2 * KD:2 * KD + VD], a, None, self.d ** -0.5,
                                state.view(-1, self.H, self.dv, self.d), ctx, o, self.H, self.H, self.d, self.dv)
            att = ctx.buf("rec_att", (T, VD), xn.dtype)
            kernels.gate_norm(o, self.norm_w, self.eps, row, 1, C, 2 * KD + VD, "silu", att, self.H, self.dv)
        return att


class GatedDeltaRule(_Recurrent):
    def __init__(self, hidden_size: int, num_heads: int, num_kv_heads: int, head_dim: int, v_head_dim: int, conv_taps: int,
                 norm_eps: float, prefix: str, unit_eps: float = 1e-6, decay_rank: int = -1, gate_rank: int = -1, names=None, **_):
        self.E, self.H, self.G = int(hidden_size), int(num_heads), int(num_kv_heads)
        self.d, self.dv, self.taps = int(head_dim), int(v_head_dim), int(conv_taps)
        self.eps, self.unit_eps, self.prefix = float(norm_eps), float(unit_eps), prefix
        # -1: the inner sizes of the decay's and the gate's two products are the stored tensors'
        self.decay_rank, self.gate_rank = int(decay_rank), int(gate_rank)
        if self.H % self.G:
            raise UnsupportedError(f"gated delta rule: {self.H} heads over {self.G} query/key heads")
        if not 1 <= self.taps <= kernels.CONV_MAX_TAPS:
            raise UnsupportedError(f"gated delta rule: {self.taps} convolution taps (1 to {kernels.CONV_MAX_TAPS})")
        if self.d > kernels.SCAN_MAX_HEAD:
            raise UnsupportedError(f"gated delta rule: key heads above {kernels.SCAN_MAX_HEAD} are not supported")
        n = {"q": "q", "k": "k", "v": "v", "conv": ".conv", "beta": "b", "A": "A_log", "norm": "norm", "a1": "a1", "a2": "a2",
             "a_bias": "dt_bias", "g1": "g1", "g2": "g2", "o": "o"}
        n.update(names or {})
        self.nm = n
        self.w_in = self.w_conv = self.w_beta = self.w_o = self.w_a1 = self.w_a2 = self.w_g1 = self.w_g2 = None
        self.a_bias = self.norm_w = self.rate = None

    @property
    def C(self):
        """Channels of the convolution: query, key and value heads side by side."""
        return 2 * self.G * self.d + self.H * self.dv

    @property
    def n_matrix(self):
        return self.H * self.dv * self.d

    def state_spec(self):
        return StateSpec((self.n_matrix + max(self.taps - 1, 1) * self.C,))

    def tensor_specs(self):
        KD, VD, HD = self.G * self.d, self.H * self.dv, self.H * self.d
        s = []
        for x, n in (("q", KD), ("k", KD), ("v", VD)):
            s += [TensorSpec(self._t(x), (n, self.E)), TensorSpec(self._t(x) + self.nm["conv"], (n, self.taps))]
        s += [TensorSpec(self._t("beta"), (self.H, self.E)), TensorSpec(self._t("A"), (self.H,)),
              TensorSpec(self._t("norm"), (self.dv,), init="norm"), TensorSpec(self._t("a_bias"), (HD,)),
              TensorSpec(self._t("a1"), (self.decay_rank, self.E)), TensorSpec(self._t("a2"), (HD, self.decay_rank)),
              TensorSpec(self._t("g1"), (self.gate_rank, self.E)), TensorSpec(self._t("g2"), (VD, self.gate_rank)),
              TensorSpec(self._t("o"), (self.E, VD))]
        return s

    def bind(self, tensors, run_dtype, device):
        self.w_in = fused_rows(tensors, [self._t(x) for x in ("q", "k", "v")], device)
        self.w_conv = fused_rows(tensors, [self._t(x) + self.nm["conv"] for x in ("q", "k", "v")], device)
        self.w_beta = tensors[self._t("beta")].contiguous()
        self.w_o = tensors[self._t("o")].contiguous()
        self.w_a1, self.w_a2 = tensors[self._t("a1")].contiguous(), tensors[self._t("a2")].contiguous()
        self.w_g1, self.w_g2 = tensors[self._t("g1")].contiguous(), tensors[self._t("g2")].contiguous()
        self.a_bias, self.norm_w = tensors[self._t("a_bias")].contiguous(), tensors[self._t("norm")].contiguous()
        self.rate = torch.exp(tensors[self._t("A")].to(torch.float32)).contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_beta, self.w_o, self.w_a1, self.w_a2, self.w_g1, self.w_g2))

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        products = sum(w.numel() for w in (self.w_in, self.w_beta, self.w_o, self.w_a1, self.w_a2, self.w_g1, self.w_g2))
        return 2.0 * T * products + 8.0 * T * self.H * self.d * self.dv

    def _attend(self, ctx, xn, cache, write_cache, state):
        T = xn.shape[0]
        KD, VD, HD, C = self.G * self.d, self.H * self.dv, self.H * self.d, self.C
        matrix = state[:, :self.n_matrix].view(-1, self.H, self.dv, self.d)
        carried = state[:, self.n_matrix:].view(state.shape[0], -1, C)
        with kernels.phase("qkv"):
            x, splits = kernels.product_sums(xn, self.w_in, ctx.buf("rec_in", (T, C), torch.float32))
            qkv = ctx.buf("rec_conv", (T, C), torch.float32)
            # query and key heads come first: 2 G heads of unit length, the G query heads of them also times d^(-1/2)
            kernels.short_conv(x, splits, self.w_conv, carried, ctx, qkv, 2 * self.G, self.d, self.H, self.dv, n_unit=2 * self.G,
                               n_scaled=self.G, scale=self.d ** -0.5, unit_eps=self.unit_eps)
            beta, _ = kernels.product_sums(xn, self.w_beta, ctx.buf("rec_beta", (T, self.H), torch.float32), finished=True)
            z, z_splits = self._low_rank_sums(ctx, xn, self.w_a1, self.w_a2, "a")
            a = ctx.buf("rec_decay", (T, HD), torch.float32)
            kernels.decay(z, z_splits, self.a_bias, self.rate, 1.0, a, self.H, self.d)
        o = ctx.buf("rec_o", (T, VD), torch.float32)
        with kernels.phase("attn"):
            kernels.linear_scan(qkv[:, :KD], qkv[:, KD:2 * KD], qkv[:, 2 * KD:], a, beta, 1.0, matrix, ctx, o, self.H, self.G,
                                self.d, self.dv)
        with kernels.phase("qkv"):
            g, g_splits = self._low_rank_sums(ctx, xn, self.w_g1, self.w_g2, "g")
        with kernels.phase("attn"):
            att = ctx.buf("rec_att", (T, VD), xn.dtype)
            kernels.gate_norm(o, self.norm_w, self.eps, g, g_splits, VD, 0, "sigmoid", att, self.H, self.dv)
        return att


class MinGru(_Recurrent):
    """minGRU: a gated recurrence per channel whose gates read the current token only.  With h the mixer's input,

        z = sigmoid(Wz h + bz);  u = Wx h + bx;  candidate = u + 1/2 where u >= 0, sigmoid(u) where u < 0;
        S_t = (1 - z) S_(t-1) + z candidate;      out = Wo (S_t * silu(Wg h))

    all of size ``width``.  S starts at zero, is float32 and lives in the request's state slot.  The three products that
    read h are one product [z | x | g] whose float32 sums the scan kernel takes as they are (the gates, the candidate
    and the state are float32 in both run types); the kernel stores the output product's operand."""

    def __init__(self, hidden_size: int, width: int, prefix: str, names=None, **_):
        self.E, self.W, self.prefix = int(hidden_size), int(width), prefix
        if self.W < 1:
            raise UnsupportedError("minGRU: the width must be positive")
        n = {"z": "z", "x": "x", "g": "g", "o": "o", "z_bias": "z.b", "x_bias": "x.b"}
        n.update(names or {})
        self.nm = n
        self.w_in = self.w_o = self.b_z = self.b_x = None

    def state_spec(self):
        return StateSpec((self.W,))

    def tensor_specs(self):
        return [TensorSpec(self._t("z"), (self.W, self.E)), TensorSpec(self._t("x"), (self.W, self.E)),
                TensorSpec(self._t("g"), (self.W, self.E)), TensorSpec(self._t("o"), (self.E, self.W)),
                TensorSpec(self._t("z_bias"), (self.W,)), TensorSpec(self._t("x_bias"), (self.W,))]

    def bind(self, tensors, run_dtype, device):
        self.w_in = fused_rows(tensors, [self._t(x) for x in ("z", "x", "g")], device)
        self.w_o = tensors[self._t("o")].contiguous()
        self.b_z, self.b_x = tensors[self._t("z_bias")].contiguous(), tensors[self._t("x_bias")].contiguous()

    def weight_bytes(self):
        return sum(w.numel() * w.element_size() for w in (self.w_in, self.w_o))

    def flops(self, q_lens, kv_lens):
        T = sum(q_lens)
        return 2.0 * T * (self.w_in.numel() + self.w_o.numel()) + 6.0 * T * self.W

    def _attend(self, ctx, xn, cache, write_cache, state):
        T = xn.shape[0]
        with kernels.phase("qkv"):
            row, splits = kernels.product_sums(xn, self.w_in, ctx.buf("rec_in", (T, 3 * self.W), torch.float32))
        att = ctx.buf("rec_att", (T, self.W), xn.dtype)
        with kernels.phase("attn"):
            kernels.mingru_scan(row, splits, self.b_z, self.b_x, state, ctx, att, self.W)
        return att


register_part("mixer", "gated_linear_attention", GatedLinearAttention)
register_part("mixer", "mingru", MinGru)
register_part("mixer", "gated_delta_rule", GatedDeltaRule)
