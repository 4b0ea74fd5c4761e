"""Mixture-of-experts feed-forward: a router picks ``top`` of ``experts`` small feed-forwards per token.

Router: ``z = x Wr^T + br`` in float32; the ``top`` largest logits choose the experts and their weights are the
softmax over the chosen logits only.  Expert: ``Wd act(Wu x)`` (not gated, no biases).  Output: the weighted sum of the
chosen experts, plus, when the layer has one, a shared expert of the same form (with a width of its own) that every
token runs.  (The reference has dense layers only.)

Options: ``gated`` experts, ``Wd (act(Wg x) * (Wu x))``.  ``router`` "softmax_all": the scores are a softmax over all
router outputs; an output is chosen by its score plus a stored ``correction`` (the weights use the score without it);
the outputs form ``groups`` = (count, keep) equal groups of neighbours and only outputs of the ``keep`` groups with the
largest choice score can be chosen; weights = scores of the chosen times ``route_scale``, not renormalised.  The last
``identity`` router outputs are identity experts without tensors: their output is the layer's input itself.

Nothing comes back to the host: the router's choices are grouped by expert on the device, the experts run as one
grouped product over the groups' tiles (launch sizes are upper bounds), and each token's choices are summed in
the router's order, so a token's output does not depend on what else is in the step, and steps of single tokens
replay as a graph.
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec, fused_rows
from .base import FeedForward, register_part


class MoeFfn(FeedForward):
    graph_safe = True

    def __init__(self, hidden_size: int, experts: int, top: int, expert_size: int, prefix: str, activation: str = "relu2",
                 router_bias: bool = True, shared_size: int = 0, names=None, gated: bool = False, router: str = "topk_softmax",
                 correction=None, groups=None, identity: int = 0, route_scale: float = 1.0, **_):
        self.E, self.n, self.top, self.F, self.FS = int(hidden_size), int(experts), int(top), int(expert_size), int(shared_size or 0)
        self.gated, self.router, self.identity, self.route_scale = bool(gated), router, int(identity or 0), float(route_scale)
        if router not in ("topk_softmax", "softmax_all"):
            raise UnsupportedError(f"mixture of experts: router '{router}' is not known (topk_softmax, softmax_all)")
        self.n_out = self.n + self.identity                 # router outputs: experts, then identity experts
        self.groups = (int(groups[0]), int(groups[1])) if groups else (1, 1)
        if router == "topk_softmax" and (self.identity or groups or correction or self.route_scale != 1.0):
            raise UnsupportedError("mixture of experts: identity experts, groups, a correction and a scale belong to the softmax_all router")
        if self.identity < 0 or self.n < 0 or self.n_out < 1:
            raise UnsupportedError(f"mixture of experts: {self.n} experts and {self.identity} identity experts")
        count, keep = self.groups
        if count < 1 or self.n_out % count or not 1 <= keep <= count or keep * (self.n_out // count) < self.top:
            raise UnsupportedError(f"mixture of experts: {count} groups of which {keep} are kept do not fit {self.n_out} router "
                                   f"outputs with top {self.top}")
        if router_bias and router == "softmax_all":
            raise UnsupportedError("mixture of experts: the softmax_all router has no bias")
        self.correction_name = correction
        self.correction = None
        if not 1 <= self.top <= self.n_out:
            raise UnsupportedError(f"mixture of experts: top {self.top} of {self.n_out} experts")
        if activation not in kernels.ACTIVATIONS:
            raise UnsupportedError(f"mixture of experts: activation '{activation}' is not supported")
        self.activation, self.router_bias = activation, bool(router_bias)
        n = {"router": "router", "router_bias": "router.b", "expert": "e{}", "shared": "shared", "up": "up", "down": "down",
             "gate": "gate"}
        n.update(names or {})
        self.prefix, self.nm = prefix, n
        self.w_router = self.b_router = self.w_up = self.w_down = self.ws_up = self.ws_down = None

    def _expert(self, i, which):
        return f"{self.prefix}.{self.nm['expert'].format(i)}.{self.nm[which]}"

    def tensor_specs(self):
        s = [TensorSpec(f"{self.prefix}.{self.nm['router']}", (self.n_out, self.E))]
        if self.router_bias:
            s.append(TensorSpec(f"{self.prefix}.{self.nm['router_bias']}", (self.n,)))
        if self.correction_name:
            s.append(TensorSpec(f"{self.prefix}.{self.correction_name}", (self.n_out,)))
        for i in range(self.n):
            if self.gated:
                s.append(TensorSpec(self._expert(i, "gate"), (self.F, self.E)))
            s += [TensorSpec(self._expert(i, "up"), (self.F, self.E)), TensorSpec(self._expert(i, "down"), (self.E, self.F))]
        if self.FS:
            p = f"{self.prefix}.{self.nm['shared']}"
            s += [TensorSpec(f"{p}.{self.nm['up']}", (self.FS, self.E)), TensorSpec(f"{p}.{self.nm['down']}", (self.E, self.FS))]
        return s

    def bind(self, tensors, run_dtype, device):
        self.w_router = tensors[f"{self.prefix}.{self.nm['router']}"].contiguous()
        if self.router_bias:
            self.b_router = tensors[f"{self.prefix}.{self.nm['router_bias']}"].to(self.w_router.dtype).contiguous()
        # all experts' matrices in one array each, [experts, out, in], filled a tensor at a time
        if self.correction_name:
            self.correction = tensors[f"{self.prefix}.{self.correction_name}"].contiguous()
        if self.gated and self.n:
            # an expert's gate and up rows alternate, so that a tile of the grouped product holds both halves of a feature
            first = tensors[self._expert(0, "up")]
            self.w_up = torch.empty((self.n, 2 * self.F, self.E), dtype=first.dtype, device=device)
            for i in range(self.n):
                pair = self.w_up[i].view(self.F, 2, self.E)
                pair[:, 0].copy_(tensors[self._expert(i, "gate")])
                pair[:, 1].copy_(first if i == 0 else tensors[self._expert(i, "up")])
            del first
        else:
            self.w_up = fused_rows(tensors, [self._expert(i, "up") for i in range(self.n)], device).view(self.n, self.F, self.E)
        self.w_down = fused_rows(tensors, [self._expert(i, "down") for i in range(self.n)], device).view(self.n, self.E, self.F)
        if self.FS:
            p = f"{self.prefix}.{self.nm['shared']}"
            self.ws_up = tensors[f"{p}.{self.nm['up']}"].contiguous()
            self.ws_down = tensors[f"{p}.{self.nm['down']}"].contiguous()

    def weight_bytes(self):
        """What a step of one token reads: the router, ``top`` experts and the shared expert."""
        per = lambda w: w.numel() * w.element_size()
        b = per(self.w_router) + (per(self.w_up) + per(self.w_down)) * self.top // self.n_out
        return b + (per(self.ws_up) + per(self.ws_down) if self.FS else 0)

    def flops(self, rows):
        real = self.top * self.n / self.n_out             # chosen experts that are not identity experts, on average
        return 2.0 * rows * (self.n_out * self.E + (3 if self.gated else 2) * real * self.E * self.F + 2 * self.E * self.FS)

    def _experts(self, ctx, xn):
        """Router, grouping and the routed experts: (outputs of every (token, choice) [T * top, E] float32, weights [T, top])."""
        T, P = xn.shape[0], xn.shape[0] * self.top
        i32 = torch.int32
        ids = ctx.buf("moe_ids", (T, self.top), i32)
        wts = ctx.buf("moe_weights", (T, self.top), torch.float32)
        z = ctx.buf("moe_logits", (T, self.n_out), torch.float32)
        with kernels.phase("glue"):
            if self.router == "softmax_all":
                kernels.moe_route_softmax(xn, self.w_router, self.correction, self.top, self.groups[0], self.groups[1],
                                          self.route_scale, ids, wts, z)
            else:
                kernels.moe_route(xn, self.w_router, self.b_router, self.top, ids, wts, z)
            mt = kernels.moe_max_tiles(P, self.n)
            order = ctx.buf("moe_order", (P,), i32)
            tiles = [ctx.buf(f"moe_tile{k}", (mt,), i32) for k in range(3)]
            n_tiles = ctx.buf("moe_n_tiles", (1,), i32)
            kernels.moe_group(ids, self.n, order, *tiles, n_tiles)
        h = ctx.buf("moe_h", (P, self.F), xn.dtype)
        y = ctx.buf("moe_y", (P, self.E), xn.dtype if xn.dtype == torch.float32 else torch.float32)
        with kernels.phase("gate_up"):
            kernels.moe_gemm(xn, self.w_up, h, self.activation, order, self.top, False, *tiles, n_tiles, P, glu=self.gated)
        with kernels.phase("down"):
            kernels.moe_gemm(h, self.w_down, y, "none", order, 0, True, *tiles, n_tiles, P)
        if self.identity:
            return y, wts, ids, self.n, xn
        return y, wts

    def forward_mix(self, ctx, xn):
        """The routed output in pieces, for a block that sums it in a pass of its own: (rows float32 [T * top, E], weights
        [T, top], ids [T, top] or None, number of real experts, the layer's input): a choice whose id is at or above the
        number of real experts stands for the input itself.  None when the layer also has a shared expert."""
        if self.FS:
            return None
        m = self._experts(ctx, xn)
        return m if len(m) == 5 else (m[0], m[1], None, self.n, None)

    def _ones(self, device):
        if getattr(self, "_one", None) is None or self._one.device != device:
            self._one = torch.ones(1, dtype=torch.float32, device=device)
        return self._one

    def _shared_hidden(self, ctx, xn):
        hs = ctx.buf("moe_hs", (xn.shape[0], self.FS), xn.dtype)
        with kernels.phase("gate_up"):
            kernels.linear_act(xn, self.ws_up, hs, self.activation)
        return hs

    def forward_into_norm(self, ctx, xn, y_buf, residual, post, next_norm, out):
        """residual += post(feed-forward output): the weighted sum of the chosen experts, the shared expert's down
        product and its partial sums are all summed by the norm's own pass."""
        if self.identity:
            raise UnsupportedError("identity experts are not summed by a norm's pass")
        mix = self._experts(ctx, xn)
        if not self.FS:
            return post.add_into(None, residual, next_norm, out, mix=mix)
        hs = self._shared_hidden(ctx, xn)
        with kernels.phase("down"):
            return post.add_product_into(hs, self.ws_down, None, y_buf, residual, next_norm, out, mix=mix)

    def forward(self, ctx, xn, residual, accumulate=True):
        T = xn.shape[0]
        if self.identity:
            # the write-back pass of a stream in one copy sums the choices, identity experts among them
            if self.FS:
                raise UnsupportedError("identity experts beside a shared expert are not supported")
            one = self._ones(xn.device)
            if not accumulate:
                residual.zero_()
            with kernels.phase("glue"):
                kernels.hc_update(residual, 1, [], self._experts(ctx, xn), None, one.view(1, 1), one)
            return
        y, wts = self._experts(ctx, xn)
        out = residual
        if accumulate:
            out = ctx.buf("moe_out", residual.shape, torch.float32)
        with kernels.phase("glue"):
            kernels.moe_combine(y, wts, out)
        if self.FS:
            hs = self._shared_hidden(ctx, xn)
            with kernels.phase("down"):
                kernels.linear(hs, self.ws_down, None, out, accumulate=True)
        if accumulate:
            residual.add_(out)


register_part("ffn", "moe", MoeFfn)
