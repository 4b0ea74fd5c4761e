"""Residual arrangements.  Pre-norm: ``x += mixer(norm1(x)); x += ffn(norm2(x))`` (src/model.c:580-623); with a token
shift, the mixer reads ``h_t + (h_(t-1) - h_t) * mu`` instead of ``h_t = norm1(x_t)``.
Norm on both sides of each sublayer: ``x += post1(mixer(norm1(x))); x += post2(ffn(norm2(x)))``, where a layer may
have no feed-forward at all.  Hyper-connections: the stream is kept in several copies; a sublayer reads a weighted
sum of them, and its output is written back into every copy while the copies are mixed among themselves."""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import UnsupportedError
from ..weights.loader import TensorSpec
from .base import Block, StateSpec, register_part
from .norm import ShiftedNorm


class PreNormResidual(Block):
    """``token_shift``: the name of a stored vector mu [hidden_size]; what the mixer reads is then moved towards the previous
    token's normed input, ``h_t + (h_(t-1) - h_t) * mu`` (zeros before a request's first token; the previous token's h as
    it was before its own shift).  The last h of a request is per-request state of the block, one float32 row per
    schedule entry, so that a step may bring only the next token of a request.  The feed-forward reads ``norm2(x)`` as
    it is."""
    graph_safe = True
    wants_next_block = True          # the model hands the following block over, for its shift
    fuses_next_shift = True          # ... and may be given the following block's first norm although that block shifts

    def __init__(self, token_shift=None, hidden_size: int = 0, **_):
        self.shift_tensor, self.E = token_shift, int(hidden_size)
        if self.shift_tensor and self.E < 1:
            raise UnsupportedError("a block with a token shift needs the width of the stream")
        self.mu = None

    def tensor_specs(self):
        return [TensorSpec(self.shift_tensor, (self.E,), init="half")] if self.shift_tensor else []

    def bind(self, tensors, run_dtype, device):
        if self.shift_tensor:
            self.mu = tensors[self.shift_tensor].to(torch.float32).contiguous()

    def state_spec(self):
        return StateSpec((self.E,)) if self.shift_tensor else None

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None, block_state=None,
                next_block=None, next_block_state=None):
        if xn_ready is not None:
            xn = xn_ready                 # (from a block that knew of this block's shift, if it has one)
        elif self.shift_tensor:
            args = getattr(norm1, "shift_args", None)
            if args is None or block_state is None:
                raise UnsupportedError("the token shift needs a norm that offers it and the block's per-request state")
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            with kernels.phase("glue"):
                kernels.norm_shift(x, *args(), self.mu, block_state, ctx, xn)
        else:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        if next_norm is not None and getattr(next_block, "shift_tensor", None):
            # the following block shifts its normed input.  In a step of single tokens the previous row of every request
            # is in its slot, and the tail of this block's last product can do norm, shift and the slot's update; in any
            # other step that block does it itself, in the kernel that sees a request's rows side by side
            if ctx.max_q_len == 1 and next_block_state is not None and hasattr(next_norm, "shift_args"):
                next_norm = ShiftedNorm(next_norm, next_block.mu, next_block_state, ctx)
            else:
                next_norm = None
        if ffn is None:
            # a layer that is a mixer only: the norm behind its product is the next block's first
            fused = getattr(mixer, "forward_then_norm", None) if next_norm is not None else None
            if not fused:
                mixer.forward(ctx, xn, x, cache, state, write_cache)
                return None
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)       # (xn may live there: the mixer has read it by then)
            if not fused(ctx, xn, x, cache, state, write_cache, next_norm, nxt):
                next_norm.forward(x, nxt)
            return nxt
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        fused = getattr(mixer, "forward_then_norm", None)
        if not (fused and fused(ctx, xn, x, cache, state, write_cache, norm2, xn2)):
            if not fused:
                mixer.forward(ctx, xn, x, cache, state, write_cache)
            norm2.forward(x, xn2)
        fused = getattr(ffn, "forward_then_norm", None) if next_norm is not None else None
        if fused:
            nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            if not fused(ctx, xn2, x, next_norm, nxt):
                next_norm.forward(x, nxt)
            return nxt
        ffn.forward(ctx, xn2, x)
        return None


class SandwichResidual(Block):
    """``x += post1(mixer(norm1(x)))``, then, if the layer has a feed-forward, ``x += post2(ffn(norm2(x)))``.  The
    sublayers write their output to a float32 buffer (``accumulate=False``) instead of adding it to the stream; the
    post-norm adds it, and where it can it hands back the following norm of the new stream from the same pass."""
    graph_safe = True

    def __init__(self, **_):
        pass

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None,
                post1=None, post2=None):
        if post1 is None or (ffn is not None and post2 is None):
            raise ValueError("this block needs a norm behind each sublayer")
        if xn_ready is None:
            xn = ctx.buf("block_xn", x.shape, ctx.run_dtype)
            norm1.forward(x, xn)
        else:
            xn = xn_ready
        y = ctx.buf("block_y", x.shape, torch.float32)
        # A part whose output is a product may hand that product to the norm behind it (``forward_into_norm``), which
        # then sums the product's partial sums in its own pass; else the part stores its output in y and the norm adds it.
        # Either way the norm returns whether the following norm of the new stream came out of the same pass.
        fused_norms = hasattr(post1, "add_product_into")

        def mix(following, out):
            into = getattr(mixer, "forward_into_norm", None) if fused_norms else None
            if into is not None:
                return into(ctx, xn, cache, state, write_cache, y, x, post1, following, out)
            mixer.forward(ctx, xn, y, cache, state, write_cache, accumulate=False)
            return post1.add_into(y, x, following, out)

        def feed_forward(xin, following, out):
            into = getattr(ffn, "forward_into_norm", None) if fused_norms else None
            if into is not None:
                return into(ctx, xin, y, x, post2, following, out)
            ffn.forward(ctx, xin, y, accumulate=False)
            return post2.add_into(y, x, following, out)

        nxt = ctx.buf("block_xn", x.shape, ctx.run_dtype) if next_norm is not None else None
        if ffn is None:
            return nxt if mix(next_norm, nxt) else None
        xn2 = ctx.buf("block_xn2", x.shape, ctx.run_dtype)
        if not mix(norm2, xn2):
            norm2.forward(x, xn2)
        return nxt if feed_forward(xn2, next_norm, nxt) else None


class HyperResidual(Block):
    """The stream in ``streams`` copies x_1 .. x_S ([T, S * E] float32, a token's copies side by side).  Sublayer q (1: the
    mixer, 2: the feed-forward) with its tensors ``<prefix>.hc<q>.{in [S], mix [S, S], out [S]}`` and, with ``layer_scale``,
    ``<prefix>.ls<q>`` [E]:

        u = sum_s in[s] x_s;   y = ls .* sublayer(norm(u));   x'_t = sum_s mix[s, t] x_s + out[t] y    (all t from the old x)

    The write-back pass sums the sublayer's output from its pieces (the output products' partial sums, each branch of a
    parallel mixer with its factor; a routed feed-forward's chosen experts with their weights, identity experts among
    them) and hands out the next sublayer's normed input from the new copies, so a sublayer costs one pass over the
    stream.  The norms are Dynamic Tanh norms (element-wise: the pass applies them itself)."""
    graph_safe = True
    wants_next_block = True          # the model hands the following block over, for its read weights

    def __init__(self, streams: int, hidden_size: int, prefix: str, layer_scale: bool = True, has_ffn: bool = True,
                 names=None, **_):
        self.S, self.E, self.prefix, self.layer_scale, self.has_ffn = int(streams), int(hidden_size), prefix, bool(layer_scale), bool(has_ffn)
        if not 1 <= self.S <= kernels.HC_MAX_STREAMS:
            raise UnsupportedError(f"hyper-connections: {self.S} copies of the stream (1 to {kernels.HC_MAX_STREAMS})")
        n = {"hc": "hc{}", "in": "in", "mix": "mix", "out": "out", "scale": "ls{}"}
        n.update(names or {})
        self.nm = n
        self.w = {}                  # (q, "in" | "mix" | "out") -> float32 tensor; (q, "scale") -> [E] or None

    def _name(self, q, which):
        if which == "scale":
            return f"{self.prefix}.{self.nm['scale'].format(q)}"
        return f"{self.prefix}.{self.nm['hc'].format(q)}.{self.nm[which]}"

    def _sublayers(self):
        return (1, 2) if self.has_ffn else (1,)

    def tensor_specs(self):
        s = []
        for q in self._sublayers():
            s += [TensorSpec(self._name(q, "in"), (self.S,), init="half"), TensorSpec(self._name(q, "out"), (self.S,), init="norm"),
                  TensorSpec(self._name(q, "mix"), (self.S, self.S), init="half")]
            if self.layer_scale:
                s.append(TensorSpec(self._name(q, "scale"), (self.E,), init="norm"))
        return s

    def bind(self, tensors, run_dtype, device):
        for q in self._sublayers():
            for which in ("in", "mix", "out"):
                self.w[(q, which)] = tensors[self._name(q, which)].to(torch.float32).contiguous()
            self.w[(q, "scale")] = tensors[self._name(q, "scale")].contiguous() if self.layer_scale else None

    def read_weights(self):
        """The weights with which this block's first sublayer reads the copies."""
        return self.w[(1, "in")]

    @staticmethod
    def _params(norm):
        p = getattr(norm, "params", None)
        if p is None:
            raise UnsupportedError("hyper-connections take Dynamic Tanh norms")
        return p

    def _write_back(self, x, q, sources, mix, next_in, next_norm, out):
        with kernels.phase("glue"):
            kernels.hc_update(x, self.S, sources, mix, self.w[(q, "scale")], self.w[(q, "mix")], self.w[(q, "out")],
                              next_in, self._params(next_norm) if next_norm is not None else None, out)

    def forward(self, ctx, x, norm1, mixer, norm2, ffn, cache, state, write_cache, xn_ready=None, next_norm=None, next_block=None):
        T = x.shape[0]
        shape = (T, self.E)
        if xn_ready is None:
            xn = ctx.buf("block_xn", shape, ctx.run_dtype)
            with kernels.phase("glue"):
                kernels.hc_in_norm(x, self.S, self.w[(1, "in")], None, self._params(norm1), xn)
        else:
            xn = xn_ready
        # what follows this block: the next block's read of the copies with its first norm, or, before the head, the
        # plain sum of the copies with the final norm
        nxt, nxt_in = None, None
        if next_norm is not None and getattr(next_norm, "params", None) is not None:
            if next_block is None or hasattr(next_block, "read_weights"):
                nxt = ctx.buf("block_xn", shape, ctx.run_dtype)
                nxt_in = next_block.read_weights() if next_block is not None else None
        y = ctx.buf("block_y", shape, torch.float32)
        fs = getattr(mixer, "forward_sources", None)
        if fs is not None:
            sources = [(s[0], s[1], s[2] if len(s) > 2 else 1.0) for s in fs(ctx, xn, cache, state, write_cache, y)]
        else:
            mixer.forward(ctx, xn, y, cache, state, write_cache, accumulate=False)
            sources = [(y, 1, 1.0)]
        if len(sources) > 2:
            raise UnsupportedError("the write-back pass sums the output of at most two branches")
        if ffn is None:
            self._write_back(x, 1, sources, None, nxt_in, next_norm if nxt is not None else None, nxt)
            return nxt
        xn2 = ctx.buf("block_xn2", shape, ctx.run_dtype)
        self._write_back(x, 1, sources, None, self.w[(2, "in")], norm2, xn2)
        mix = ffn.forward_mix(ctx, xn2) if hasattr(ffn, "forward_mix") else None
        if mix is not None:
            self._write_back(x, 2, [], mix, nxt_in, next_norm if nxt is not None else None, nxt)
        else:
            ffn.forward(ctx, xn2, y, accumulate=False)
            self._write_back(x, 2, [(y, 1, 1.0)], None, nxt_in, next_norm if nxt is not None else None, nxt)
        return nxt


register_part("block", "hyper_residual", HyperResidual)
register_part("block", "prenorm_residual", PreNormResidual)
register_part("block", "sandwich_residual", SandwichResidual)
