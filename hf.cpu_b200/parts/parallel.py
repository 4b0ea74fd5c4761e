"""Mixers side by side: every branch reads the same input and the result is the weighted sum of their outputs,
``sum_i scale_i * branch_i(h)``.  Branches are mixers of any registered kind, built from their own specs; at most one of
them may keep a paged cache and at most one a state of fixed size per request (the schedule entry has one of each),
which the combination then declares as its own.  (The reference's layer has one mixer, src/model.c:581-609.)
"""
from __future__ import annotations

import torch

from .. import kernels
from ..config.base import PartSpec, UnsupportedError
from .base import Mixer, make_part, register_part


class ParallelMixer(Mixer):
    def __init__(self, branches, positions=None, **_):
        """``branches``: [(PartSpec or {"kind", "args"}, scale), ...]."""
        self.branches, self.scales = [], []
        for spec, scale in branches:
            if not isinstance(spec, PartSpec):
                spec = PartSpec(spec["kind"], dict(spec["args"]))
            self.branches.append(make_part("mixer", spec, positions=positions))
            self.scales.append(float(scale))
        if not self.branches:
            raise UnsupportedError("a parallel mixer needs at least one branch")
        if sum(b.cache_spec() is not None for b in self.branches) > 1:
            raise UnsupportedError("a parallel mixer takes one branch with a paged cache")
        if sum(b.state_spec() is not None for b in self.branches) > 1:
            raise UnsupportedError("a parallel mixer takes one branch with per-request state")

    @property
    def graph_safe(self):
        return all(getattr(b, "graph_safe", False) for b in self.branches)

    @property
    def launch_overlap_safe(self):
        return all(getattr(b, "launch_overlap_safe", True) for b in self.branches)

    def cache_spec(self):
        return next((b.cache_spec() for b in self.branches if b.cache_spec() is not None), None)

    def state_spec(self):
        return next((b.state_spec() for b in self.branches if b.state_spec() is not None), None)

    def step_arrays_key(self):
        keys = [b.step_arrays_key() for b in self.branches if b.step_arrays_key() is not None]
        if len(keys) > 1:
            raise UnsupportedError("a parallel mixer takes one branch with step arrays of its own")
        return keys[0] if keys else None

    def step_arrays(self, batch):
        return next(b.step_arrays(batch) for b in self.branches if b.step_arrays_key() is not None)

    def tensor_specs(self):
        return [s for b in self.branches for s in b.tensor_specs()]

    def bind(self, tensors, run_dtype, device):
        for b in self.branches:
            b.bind(tensors, run_dtype, device)

    def weight_bytes(self):
        return sum(b.weight_bytes() for b in self.branches)

    def flops(self, q_lens, kv_lens):
        return sum(b.flops(q_lens, kv_lens) for b in self.branches)

    def _args(self, b, cache, state):
        return (cache if b.cache_spec() is not None else None), (state if b.state_spec() is not None else None)

    def forward_sources(self, ctx, xn, cache, state, write_cache, y_buf, finished=False):
        """[(planes, splits, factor)] per branch.  Split products share one scratch area, so only the last branch may
        leave its output product in pieces; the others finish theirs in buffers of their own."""
        out = []
        for i, (b, scale) in enumerate(zip(self.branches, self.scales)):
            last = i == len(self.branches) - 1
            c, s = self._args(b, cache, state)
            buf = y_buf if last else ctx.buf(f"parallel_y{i}", y_buf.shape, torch.float32)
            fs = getattr(b, "forward_sources", None)
            if fs is not None:
                for src in fs(ctx, xn, c, s, write_cache, buf, finished=finished or not last):
                    out.append((src[0], src[1], scale * (src[2] if len(src) > 2 else 1.0)))
            else:
                b.forward(ctx, xn, buf, c, s, write_cache, accumulate=False)
                out.append((buf, 1, scale))
        return out

    def forward(self, ctx, xn, residual, cache, state, write_cache, accumulate=True):
        y = ctx.buf("parallel_sum", residual.shape, torch.float32)
        for i, (b, scale) in enumerate(zip(self.branches, self.scales)):
            c, s = self._args(b, cache, state)
            b.forward(ctx, xn, y, c, s, write_cache, accumulate=False)
            with kernels.phase("glue"):
                kernels.scale_(y, scale)
                if i == 0 and not accumulate:
                    residual.copy_(y)
                else:
                    residual.add_(y)


register_part("mixer", "parallel", ParallelMixer)
