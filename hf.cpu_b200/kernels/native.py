"""ctypes binding of the CUDA library: the only kernel backend of the product.

Every method takes torch tensors on the GPU, checks what the C entry point cannot (devices,
contiguity), passes raw pointers and the current torch stream, and raises on a non-zero status.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from . import build as _build

HFB_ENOTSUP = 2          # status of csrc/hfb200.h: not a case for this kernel, nothing was launched

_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)
_current_device = getattr(torch._C, "_cuda_getDevice", None)
if _raw_stream is None or _current_device is None:            # (another torch: the documented way)
    _raw_stream = lambda index: torch.cuda.current_stream(index).cuda_stream
    _current_device = torch.cuda.current_device


class KernelError(RuntimeError):
    pass


F32, BF16 = 0, 1


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16 tensors, got {t.dtype}")


def _p(t):
    return c_void_p(t.data_ptr()) if t is not None else c_void_p(0)


class NativeBackend:
    name = "native"

    def __init__(self):
        if not torch.cuda.is_available():
            raise KernelError("no CUDA device is visible: this engine has no CPU path")
        path = _build.build()
        try:
            self.lib = ctypes.CDLL(path)
        except OSError as e:
            raise KernelError(f"the CUDA library {path} could not be loaded: {e}") from None
        self.lib.hfb_last_error.restype = ctypes.c_char_p
        self.lib.hfb_linear_tc_workspace.restype = ctypes.c_size_t
        self.lib.hfb_attention_fast_scratch.restype = ctypes.c_size_t
        # "fast": tiled tensor-core attention where the sizes allow; "plain": one block per (token, head) always
        self.attention = os.environ.get("HFB_ATTENTION", "fast")
        self.attention_tc = os.environ.get("HFB_ATTN_TC", "1") != "0"     # tcgen05 attention for prompt portions
        self.attention_tc2 = os.environ.get("HFB_ATTN_TC2", "1") != "0"   # its form with two query tiles per CTA
        # the two-tile form takes over once there is a work item for every SM this many times over (tests set 0)
        self.tc2_min_rounds = 0.55                # items per SM from which head size 128 takes the two-tile attention kernel
        self.decode_ctas_per_sm = 2               # CTAs of the decode attention kernel per SM, over all requests' splits
        self.decode_stages = 3                    # tiles of 64 keys in flight per CTA (measured again: 1 or 3 CTAs, 2 or 4 stages lose 0.4-7 %)
        self.sm_count = torch.cuda.get_device_properties(0).multi_processor_count
        # "tc": tensor-core products where the operands allow; "plain": the float32-accumulating SIMT kernel always
        self.gemm = os.environ.get("HFB_GEMM", "tc")
        self._ws = None
        self._argmax_ws = None
        # decode attention: the CTA that stores a tile's last split merges the splits (False: a second kernel does)
        self.merge_in_kernel = True
        self.rope_in_epilogue = os.environ.get("HFB_ROPE_EPILOGUE", "1") != "0"     # prompts: q|k|v product rotates and writes the cache
        self._counters = None
        self.lib.hfb_linear_tc_partials_workspace.restype = ctypes.c_size_t
        self.lib.hfb_argmax2_scratch.restype = ctypes.c_size_t
        self.path = path
        self.launches = 0          # kernels launched through this binding (one per successful call)

    def _stream(self):
        # the raw handle of torch's current stream on the current device; asked for at every launch (a few hundred
        # a step when steps run kernel by kernel), so by the two C calls behind torch.cuda.current_stream(), which
        # itself costs 14 us a call
        return c_void_p(_raw_stream(_current_device()))

    def _check(self, rc: int, what: str):
        if rc != 0:
            raise KernelError(f"{what}: {self.lib.hfb_last_error().decode()} (status {rc})")
        self.launches += 1

    @staticmethod
    def _on_gpu(*ts):
        for t in ts:
            if t is not None and (not t.is_cuda or not t.is_contiguous()):
                raise KernelError("kernel arguments must be contiguous CUDA tensors")

    # ---- entry points -------------------------------------------------------------------------
    def embed(self, ids, table, out):
        self._on_gpu(ids, table, out)
        T, (V, E) = ids.shape[0], table.shape
        self._check(self.lib.hfb_embed(_p(ids), _p(table), c_int(_dt(table)), _p(out), c_int(T), c_int(V), c_int(E),
                                       self._stream()), "embed")

    def embed_pair(self, ids, table, scale, pair, buckets, mul_prev, mul_cur, ctx, prev_state, out):
        self._on_gpu(ids, table, pair, prev_state, out)
        T, (V, E) = ids.shape[0], table.shape
        has = pair is not None
        self._check(self.lib.hfb_embed_pair(
            _p(ids), _p(table), c_int(_dt(table)), c_float(scale), _p(pair), c_int(_dt(pair) if has else 0), c_int(buckets),
            c_int64(mul_prev), c_int64(mul_cur), _p(ctx.token_seq if has else None), _p(ctx.cu_tokens if has else None),
            _p(ctx.seq_slots if has else None), _p(prev_state if has else None), c_int(prev_state.shape[0] if has else 0),
            _p(out), c_int(T), c_int(V), c_int(E), self._stream()), "embed_pair")

    def rmsnorm(self, x, w, eps, out, rows):
        self._on_gpu(x, w, out, rows)
        M, E = out.shape
        self._check(self.lib.hfb_rmsnorm(_p(x), _p(w), c_int(_dt(w)), c_float(eps), _p(out), c_int(_dt(out)), _p(rows),
                                         c_int(M), c_int(E), self._stream()), "rmsnorm")

    def linear(self, a, w, bias, out, accumulate):
        self._on_gpu(a, w, bias, out)
        M, K = a.shape
        N = w.shape[0]
        if (self.gemm == "tc" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and K % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and out.data_ptr() % 16 == 0
                and (bias is None or bias.data_ptr() % 16 == 0)):
            need = self.lib.hfb_linear_tc_workspace(c_int(M), c_int(N), c_int(K))
            if need:
                self._workspace(a.device)
                if need > self._ws.numel():
                    need = 0                                        # runs unsplit
            self._check(self.lib.hfb_linear_tc(_p(a), _p(w), _p(bias), c_int(_dt(bias) if bias is not None else 0),
                                               _p(out), c_int(_dt(out)), c_int(1 if accumulate else 0), c_int(M),
                                               c_int(N), c_int(K), _p(self._ws if need else None),
                                               ctypes.c_size_t(self._ws.numel() if need else 0), self._stream()),
                        "linear_tc")
            return
        self._check(self.lib.hfb_linear_plain(_p(a), c_int(_dt(a)), _p(w), c_int(_dt(w)), _p(bias),
                                              c_int(_dt(bias) if bias is not None else 0), _p(out), c_int(_dt(out)),
                                              c_int(1 if accumulate else 0), c_int(M), c_int(N), c_int(K),
                                              self._stream()), "linear")

    def rope_kv_write(self, qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self._on_gpu(qkv, cos_sin, positions, slots, q_out, k_cache, v_cache)
        T = qkv.shape[0]
        cache_slots = k_cache.shape[0] * k_cache.shape[1]
        npos = cos_sin.shape[0] if cos_sin is not None else 0
        self._check(self.lib.hfb_rope_kv_write(_p(qkv), c_int(_dt(qkv)), _p(cos_sin), c_int(n_rot), c_int(npos),
                                               _p(positions), _p(slots), _p(q_out), _p(k_cache), _p(v_cache),
                                               c_int64(cache_slots), c_int(T), c_int(H), c_int(G), c_int(d),
                                               self._stream()), "rope_kv_write")

    def set_launch_overlap(self, on):
        self.lib.hfb_set_launch_overlap(c_int(1 if on else 0))

    def paged_attention(self, q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tile_arrays, dv=None, sinks=None,
                        zero_sink=False, slopes=None, head_scales=None, softcap=0.0):
        self._on_gpu(q, k_cache, v_cache, meta.block_table, ctx.token_seq, ctx.positions, out, sinks, slopes, head_scales)
        # a sink or a distance bias: the two-tile tensor-core kernel (prompt portions of 64 tokens and more), the decode
        # kernel and the plain kernel have them
        # ... and a factor per head on the scores and a tanh cap
        opts = sinks is not None or zero_sink or slopes is not None or head_scales is not None or softcap > 0
        opt_args = (_p(sinks), c_int(1 if zero_sink else 0), _p(slopes), _p(head_scales), c_float(softcap))
        T = q.shape[0]
        dv = d if dv is None else dv
        v_row = dv
        if v_cache is None:                   # a value is the first dv elements of its key
            v_cache, v_row = k_cache, d
        if (self.attention == "fast" and tile_arrays and q.dtype == torch.bfloat16 and d in (64, 128) and dv == d
                and v_row == dv and 64 % meta.block_size == 0):
            decode = ctx.max_q_len == 1

            def tiles(ratio, height):
                """(seq, t0, nt, count) of the tile list of that height, or None when the step brought none."""
                h = str(height)
                if h + ".seq" not in tile_arrays and decode and height == 4 and 64 // ratio >= 1:
                    h = "1"                                   # one token a tile fits the wider kernel too
                seq = tile_arrays.get(h + ".seq")
                if seq is None:
                    return None
                return seq, tile_arrays[h + ".t0"], tile_arrays[h + ".nt"], seq.shape[0]
            if (not decode and self.attention_tc and meta.block_size >= 8 and 128 % meta.block_size == 0
                    and H // G <= 128):
                # two 128-row tiles per CTA once there are items for more than half of the SMs: it does more per key
                # fetched and overlaps softmax and products, but has half as many items to spread (28 heads over 4: 60
                # items 22.7 against 17.9 us, 116 items 32.3 against 37.9 us; 40 over 8: 88 items 23.0 against 26.7 us).
                # Head size 64 has this form only and always takes it (16 items: 14.6 us against 17.7 us of mma.sync)
                tiling = tiles(H // G, 16) if self.attention_tc2 else None
                enough = self.tc2_min_rounds * self.sm_count if d == 128 and not opts else 0
                if tiling is not None and tiling[3] * G >= enough:
                    tile_seq, tile_t0, tile_nt, n_tiles = tiling
                    self._check(self.lib.hfb_attention_tc2_opt(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(meta.block_size),
                        c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out), c_int(T), c_int(H), c_int(G),
                        c_int(d), *opt_args, self._stream()), "attention_tc2")
                    return
                tiling = tiles(H // G, 8) if d == 128 and not opts else None      # tiles of 128 rows, as the 8-warp kernel's
                if tiling is not None:
                    tile_seq, tile_t0, tile_nt, n_tiles = tiling
                    self._check(self.lib.hfb_attention_tc(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(meta.block_size),
                        c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out), c_int(T), c_int(H), c_int(G),
                        c_int(d), self._stream()), "attention_tc")
                    return
            # single tokens: the decode kernel (16 rows a tile, keys and values by TMA) where the pages are at least 8
            # tokens; smaller pages take the 4-warp kernel with one token a tile
            decode_tma = decode and meta.block_size >= 8
            warps = 4
            tiling = tiles(H // G, 1 if decode_tma else warps) if decode_tma or not opts else None
            if tiling is None and not decode and not opts:
                warps = 8
                tiling = tiles(H // G, 8)
            if tiling is not None:
                tile_seq, tile_t0, tile_nt, n_tiles = tiling
                splits, stages = 1, 2
                if decode:
                    # about `decode_ctas_per_sm` CTAs per SM in all; with one per SM the deep pipeline fits
                    hint = getattr(ctx, "decode_split_hint", max(1, ((ctx.max_kv_len + 63) // 64) // 2))
                    splits = max(1, min(self.decode_ctas_per_sm * self.sm_count // max(1, n_tiles * G), hint))
                    stages = self.decode_stages
                else:
                    # short portions over a long context (the end of a prompt, a prompt behind a shared prefix): few
                    # tiles would each walk all the keys alone; their keys are split too, 256 to a CTA at least
                    splits = max(1, min(2 * self.sm_count // max(1, n_tiles * G), ((ctx.max_kv_len + 63) // 64) // 4, 64))
                need = self.lib.hfb_attention_fast_scratch(c_int(T), c_int(H), c_int(d), c_int(splits))
                scratch = ctx.buf("attn_scratch", (need,), torch.uint8) if need else None
                if decode_tma:
                    # the keys and values come by TMA, a warp of their own keeps them coming; the CTA that stores a
                    # tile's last split merges the splits (merge_in_kernel off: a second kernel does)
                    counters = None
                    if self.merge_in_kernel and splits > 1 and n_tiles * G <= 4096:
                        if self._counters is None or self._counters.device != q.device:
                            self._counters = torch.zeros(4096, dtype=torch.int32, device=q.device)
                        counters = self._counters
                    self._check(self.lib.hfb_attention_decode_opt(
                        _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                        _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(stages), c_int(splits),
                        c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out),
                        _p(scratch), ctypes.c_size_t(need), c_int(T), c_int(H), c_int(G), c_int(d), _p(counters),
                        c_int(counters.numel() if counters is not None else 0), *opt_args, self._stream()), "attention_decode")
                    if splits > 1 and counters is None:
                        self.launches += 1
                    return
                self._check(self.lib.hfb_attention_fast(
                    _p(q), _p(k_cache), _p(v_cache), _p(meta.block_table), c_int(meta.max_blocks), _p(ctx.positions),
                    _p(tile_seq), _p(tile_t0), _p(tile_nt), c_int(n_tiles), c_int(warps), c_int(stages), c_int(splits),
                    c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window), c_float(scale), _p(out),
                    _p(scratch), ctypes.c_size_t(need), c_int(T), c_int(H), c_int(G), c_int(d), self._stream()),
                    "attention_fast")
                if splits > 1:
                    self.launches += 1
                return
        self._check(self.lib.hfb_attention_plain(_p(q), _p(k_cache), _p(v_cache), c_int(_dt(q)), _p(meta.block_table),
                                                 c_int(meta.max_blocks), _p(ctx.token_seq), _p(ctx.positions),
                                                 c_int(meta.block_size), c_int64(k_cache.shape[0]), c_int(window),
                                                 c_float(scale), _p(out), c_int(T), c_int(H), c_int(G), c_int(d), c_int(dv),
                                                 c_int(v_row), *opt_args, self._stream()), "attention")

    def swiglu(self, gu, out, interleaved):
        self._on_gpu(gu, out)
        T, F = out.shape
        self._check(self.lib.hfb_swiglu(_p(gu), _p(out), c_int(_dt(gu)), c_int(T), c_int(F), c_int(1 if interleaved else 0),
                                        self._stream()), "swiglu")

    def argmax(self, logits, out):
        self._on_gpu(logits, out)
        M, V = logits.shape
        need = self.lib.hfb_argmax2_scratch(c_int(M), c_int(V))
        if self._argmax_ws is None or self._argmax_ws.numel() < need:
            self._argmax_ws = torch.empty(max(need, 1 << 20), dtype=torch.uint8, device=logits.device)
        self._check(self.lib.hfb_argmax2(_p(logits), _p(out), c_int(M), c_int(V), _p(self._argmax_ws),
                                         ctypes.c_size_t(self._argmax_ws.numel()), self._stream()), "argmax")
        self.launches += 1

    # ---- fused forms: the tensor-core product with the next memory-bound step in its tail ------------------
    def _tc_ok(self, a, w, out=None):
        return (self.gemm == "tc" and a.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and a.shape[1] % 8 == 0
                and a.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and (out is None or out.data_ptr() % 16 == 0))

    def _workspace(self, device):
        if self._ws is None or self._ws.device != device:
            self._ws = torch.empty(64 << 20, dtype=torch.uint8, device=device)     # split-K partials never need more
        return self._ws

    def _partials(self, a, w):
        """Split-K partial sums of a @ w.T in the workspace; returns (workspace, splits)."""
        M, K = a.shape
        N = w.shape[0]
        ws = self._workspace(a.device)
        need = self.lib.hfb_linear_tc_partials_workspace(c_int(M), c_int(N), c_int(K))
        if need == 0 or need > ws.numel():                      # 0: above 128 rows, and not a product that is split
            return None
        splits = c_int(0)
        self._check(self.lib.hfb_linear_tc_partials(_p(a), _p(w), c_int(M), c_int(N), c_int(K), _p(ws),
                                                    ctypes.c_size_t(ws.numel()), ctypes.byref(splits), self._stream()),
                    "linear_tc_partials")
        return ws, splits.value

    def linear_swiglu(self, a, w, gu_buf, out):
        self._on_gpu(a, w, out)
        M, K = a.shape
        N = w.shape[0]
        if self._tc_ok(a, w, out):
            self._check(self.lib.hfb_linear_tc_swiglu(_p(a), _p(w), _p(out), c_int(_dt(out)), c_int(M), c_int(N), c_int(K),
                                                      self._stream()), "linear_tc_swiglu")
            return
        self.linear(a, w, None, gu_buf, False)
        self.swiglu(gu_buf, out, True)

    def linear_residual_norm(self, a, w, bias, residual, norm_w, eps, xn_out, center=False, shift=None):
        self._on_gpu(a, w, bias, residual, norm_w, xn_out)
        M, K = a.shape
        N = w.shape[0]
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if center or shift is not None:
            # layer norm and the token shift of single-token steps: a tail of their own; where the product is not split
            # it is added to the stream first and the tail only norms
            ws, splits = part if part is not None else (None, 0)
            if part is None:
                self.linear(a, w, bias, residual, True)
                bias = None
            mu, state, seq_slots = shift if shift is not None else (None, None, None)
            self._on_gpu(mu, state, seq_slots)
            self._check(self.lib.hfb_reduce_residual_layernorm(
                _p(ws), c_int(splits), c_int(M), c_int(N), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(residual),
                _p(norm_w), c_float(eps), c_int(1 if center else 0), _p(mu), _p(state),
                c_int64(state.stride(0) if state is not None else 0), _p(seq_slots), c_int(state.shape[0] if state is not None else 0),
                _p(xn_out), c_int(_dt(xn_out)), self._stream()), "reduce_residual_layernorm")
            return
        if part is None:
            self.linear(a, w, bias, residual, True)
            if xn_out is not None:
                self.rmsnorm(residual, norm_w, eps, xn_out, None)
            return
        ws, splits = part
        self._check(self.lib.hfb_reduce_residual_norm(
            _p(ws), c_int(splits), c_int(M), c_int(N), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(residual),
            _p(norm_w), c_int(_dt(norm_w) if norm_w is not None else 0), c_float(eps), _p(xn_out),
            c_int(_dt(xn_out) if xn_out is not None else 0), self._stream()), "reduce_residual_norm")

    def linear_rope_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self._on_gpu(a, w, bias, cos_sin, positions, slots, q_out, k_cache, v_cache)
        M, K = a.shape
        if (self.rope_in_epilogue and M >= 256 and self._tc_ok(a, w, q_out) and q_out.dtype == torch.bfloat16
                and k_cache.dtype == torch.bfloat16 and d in (64, 128) and n_rot == d and cos_sin is not None
                and (bias is None or (bias.dtype == torch.bfloat16 and bias.data_ptr() % 16 == 0))):
            # many tokens: rotation and the cache write run in the product's epilogue
            rc = self.lib.hfb_linear_tc_rope_kv(
                _p(a), _p(w), _p(bias), _p(cos_sin), c_int(cos_sin.shape[0]), _p(positions), _p(slots), _p(q_out),
                _p(k_cache), _p(v_cache), c_int64(k_cache.shape[0] * k_cache.shape[1]), c_int(M), c_int(K), c_int(H),
                c_int(G), c_int(d), self._stream())
            if rc != HFB_ENOTSUP:
                self._check(rc, "linear_tc_rope_kv")
                return
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if part is None:
            self.linear(a, w, bias, qkv_buf, False)
            self.rope_kv_write(qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d)
            return
        ws, splits = part
        cache_slots = k_cache.shape[0] * k_cache.shape[1]
        npos = cos_sin.shape[0] if cos_sin is not None else 0
        self._check(self.lib.hfb_reduce_rope_kv(
            _p(ws), c_int(splits), c_int(_dt(q_out)), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(cos_sin),
            c_int(n_rot), c_int(npos), _p(positions), _p(slots), _p(q_out), _p(k_cache), _p(v_cache), c_int64(cache_slots),
            c_int(M), c_int(H), c_int(G), c_int(d), self._stream()), "reduce_rope_kv")

    # ---- Dynamic Tanh norms, unit-rms heads, gated and routed feed-forwards --------------------------------
    def dyt(self, x, params, out, rows):
        alpha, w, b = params
        self._on_gpu(x, alpha, w, b, out, rows)
        M, E = out.shape
        self._check(self.lib.hfb_dyt(_p(x), c_int(_dt(x)), _p(rows), _p(alpha), _p(w), _p(b), c_int(_dt(w)), _p(out),
                                     c_int(_dt(out)), c_int(M), c_int(E), self._stream()), "dyt")

    def linear_dyt_residual(self, a, w, bias, y_buf, post, residual, nxt, out, mix=None):
        """residual += dyt(a @ w.T + bias (+ mix)): the product's split-K partial sums are summed by the norm's own
        pass where the product is split, else it stores float32 to ``y_buf`` first."""
        self._on_gpu(a, w, bias, y_buf)
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if part is None:
            self.linear(a, w, bias, y_buf, False)
            self.dyt_residual(y_buf, post, residual, nxt, out, mix=mix)
        else:
            self.dyt_residual(part[0], post, residual, nxt, out, splits=part[1], bias=bias, as_f32=True, mix=mix)

    def dyt_residual(self, y, post, residual, nxt, out, splits=1, bias=None, as_f32=False, mix=None):
        self._on_gpu(*post, residual, out, *(nxt or ()), *(mix or ()))
        M, E = residual.shape
        n = nxt or (None, None, None)
        if y is None:
            splits = 0
        mix_y, mix_w = mix or (None, None)
        self._check(self.lib.hfb_dyt_residual(
            _p(y), c_int(F32 if as_f32 or y is None else _dt(y)), c_int(splits), _p(bias), c_int(_dt(bias) if bias is not None else 0),
            _p(mix_y), _p(mix_w), c_int(mix_w.shape[1] if mix_w is not None else 0), _p(post[0]), _p(post[1]), _p(post[2]), c_int(_dt(post[1])), _p(residual), _p(n[0]), _p(n[1]),
            _p(n[2]), c_int(_dt(n[1]) if nxt else 0), _p(out), c_int(_dt(out) if out is not None else 0), c_int(M), c_int(E),
            self._stream()), "dyt_residual")

    def linear_rope_norm_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d, dv,
                            norm_eps, norm_weights=None, value_mix=None, pairing="half"):
        self._on_gpu(a, w, bias, cos_sin, positions, slots, q_out, k_cache, v_cache)
        T = a.shape[0]
        part = self._partials(a, w) if self._tc_ok(a, w) else None
        if part is None:
            self.linear(a, w, bias, qkv_buf, False)
            src, splits, bias = qkv_buf, 1, None
        else:
            src, splits = part
        cache_slots = k_cache.shape[0] * k_cache.shape[1] if G else 0
        q_w, k_w = norm_weights or (None, None)
        v_first, v_mode, v_lambda = value_mix or (None, 0, 0.0)
        self._on_gpu(q_w, k_w, v_first)
        self._check(self.lib.hfb_rope_norm_kv_write(
            _p(src), c_int(splits), _p(bias), c_int(_dt(bias) if bias is not None else 0), _p(cos_sin), c_int(n_rot),
            c_int(cos_sin.shape[0] if cos_sin is not None else 0), _p(positions), _p(slots if G else None), _p(q_out),
            _p(k_cache if G else None), _p(v_cache if G and dv else None), c_int(_dt(q_out)), c_int64(cache_slots), c_int(T), c_int(H),
            c_int(G), c_int(d), c_int(dv), c_int(0 if norm_eps is None else 1), c_float(norm_eps or 0.0), _p(q_w), _p(k_w),
            _p(v_first), c_int(v_mode), c_float(v_lambda), c_int(1 if pairing == "interleaved" else 0), self._stream()),
            "rope_norm_kv_write")

    def product_sums(self, a, w, buf, finished=False):
        self._on_gpu(a, w, buf)
        src, splits = self._product_sums(a, w, buf, finished)
        return (src if src.dtype == torch.float32 else src.view(torch.float32)), splits

    def _product_sums(self, a, w, buf, finished=False):
        """float32 sums of a @ w.T for a tail kernel: (partial sums, splits) where the tensor-core product is split over
        k (the tail then sums the pieces itself), else the finished product in ``buf`` with splits = 1."""
        part = self._partials(a, w) if self._tc_ok(a, w) and not finished else None
        if part is not None:
            return part
        self.linear(a, w, None, buf, False)
        return buf, 1

    def linear_latent_split(self, a, w, buf, q_norm_w, kv_norm_w, eps, cos_sin, positions, slots, cq_out, cache, q_rank, kv_rank, rot):
        self._on_gpu(a, w, buf, q_norm_w, kv_norm_w, cos_sin, positions, slots, cq_out, cache)
        src, splits = self._product_sums(a, w, buf)
        self._check(self.lib.hfb_latent_split(
            _p(src), c_int(splits), _p(q_norm_w), _p(kv_norm_w), c_float(eps), _p(cos_sin),
            c_int(cos_sin.shape[0] if cos_sin is not None else 0), _p(positions), _p(slots), _p(cq_out), _p(cache), c_int(_dt(cq_out)),
            c_int64(cache.shape[0] * cache.shape[1]), c_int(a.shape[0]), c_int(q_rank), c_int(kv_rank), c_int(rot), self._stream()),
            "latent_split")

    def linear_latent_query(self, a, w, buf, cos_sin, positions, q_plain, q_att, H, d, rot, att_col):
        self._on_gpu(a, w, buf, cos_sin, positions, q_plain, q_att)
        src, splits = self._product_sums(a, w, buf)
        self._check(self.lib.hfb_latent_query_rope(
            _p(src), c_int(splits), _p(cos_sin), c_int(cos_sin.shape[0] if cos_sin is not None else 0), _p(positions), _p(q_plain),
            _p(q_att), c_int(_dt(q_att)), c_int(a.shape[0]), c_int(H), c_int(d), c_int(rot), c_int(q_att.shape[1] // H), c_int(att_col),
            self._stream()), "latent_query_rope")

    def linear_latent_query_absorb(self, a, w_uq, buf, cos_sin, positions, w_ukt, q_att, H, d, rot):
        self._on_gpu(a, w_uq, buf, cos_sin, positions, w_ukt, q_att)
        src, splits = self._product_sums(a, w_uq, buf)
        self._check(self.lib.hfb_latent_query_absorb(
            _p(src), c_int(splits), _p(cos_sin), c_int(cos_sin.shape[0] if cos_sin is not None else 0), _p(positions), _p(w_ukt),
            _p(q_att), c_int(a.shape[0]), c_int(H), c_int(d), c_int(rot), c_int(w_ukt.shape[1]), self._stream()), "latent_query_absorb")

    def headwise_linear(self, x, w, out, H, in_row, out_row):
        self._on_gpu(x, w, out)
        self._check(self.lib.hfb_headwise_linear(_p(x), c_int(_dt(x)), _p(w), c_int(_dt(w)), _p(out), c_int(_dt(out)), c_int(x.shape[0]),
                                                 c_int(H), c_int(w.shape[1]), c_int(w.shape[2]), c_int(in_row), c_int(out_row),
                                                 self._stream()), "headwise_linear")

    def linear_glu(self, a, w, gu_buf, out, act):
        self._on_gpu(a, w, gu_buf, out)
        if self._tc_ok(a, w, out):
            M, K = a.shape
            self._check(self.lib.hfb_linear_tc_glu(_p(a), _p(w), _p(out), c_int(_dt(out)), c_int(M), c_int(w.shape[0]), c_int(K),
                                                   c_int(act), self._stream()), "linear_tc_glu")
            return
        self.linear(a, w, None, gu_buf, False)
        T, F = out.shape
        self._check(self.lib.hfb_glu(_p(gu_buf), _p(out), c_int(_dt(out)), c_int(T), c_int(F), c_int(1), c_int(act),
                                     self._stream()), "glu")

    def linear_act(self, a, w, out, act):
        self._on_gpu(a, w, out)
        if self._tc_ok(a, w, out) and 0 < act < 4:
            M, K = a.shape
            self._check(self.lib.hfb_linear_tc_act(_p(a), _p(w), _p(out), c_int(_dt(out)), c_int(M), c_int(w.shape[0]), c_int(K),
                                                   c_int(act), self._stream()), "linear_tc_act")
            return
        self.linear(a, w, None, out, False)
        self._check(self.lib.hfb_act(_p(out), _p(out), c_int(_dt(out)), c_int64(out.numel()), c_int(act), self._stream()), "act")

    def scale_(self, x, s):
        self._on_gpu(x)
        self._check(self.lib.hfb_scale(_p(x), c_int64(x.numel()), c_float(s), self._stream()), "scale")

    def moe_route(self, h, w, b, top, ids, weights, logits):
        self._on_gpu(h, w, b, ids, weights, logits)
        T, E = logits.shape
        part = self._partials(h, w) if self._tc_ok(h, w) else None
        if part is None:
            self.linear(h, w, b, logits, False)
            src, splits, b = logits, 1, None
        else:                                   # the top-k kernel sums the product's partial sums itself
            src, splits = part
        self._check(self.lib.hfb_moe_topk(_p(src), c_int(splits), _p(b), c_int(_dt(b) if b is not None else 0), c_int(T), c_int(E),
                                          c_int(top), _p(ids), _p(weights), self._stream()), "moe_topk")

    def moe_route_softmax(self, h, w, correction, top, n_groups, keep, scale, ids, weights, logits):
        self._on_gpu(h, w, correction, ids, weights, logits)
        T, E = logits.shape
        src, splits = self._product_sums(h, w, logits)
        self._check(self.lib.hfb_moe_route_softmax(_p(src), c_int(splits), _p(correction), c_int(_dt(correction) if correction is not None else 0),
                                                   c_int(T), c_int(E), c_int(top), c_int(n_groups), c_int(keep), c_float(scale), _p(ids),
                                                   _p(weights), self._stream()), "moe_route_softmax")

    # ---- hyper-connections ----------------------------------------------------------------------------------
    def hc_spread(self, emb, x, S):
        self._on_gpu(emb, x)
        T, E = emb.shape
        self._check(self.lib.hfb_hc_spread(_p(emb), _p(x), c_int(S), c_int(T), c_int(E), self._stream()), "hc_spread")

    def hc_in_norm(self, x, S, in_w, rows, norm, out):
        n = norm or (None, None, None)
        self._on_gpu(x, in_w, rows, out, *n)
        M, E = out.shape
        self._check(self.lib.hfb_hc_in_norm(_p(x), c_int(S), _p(in_w), _p(rows), _p(n[0]), _p(n[1]), _p(n[2]),
                                            c_int(_dt(n[1]) if norm else 0), _p(out), c_int(_dt(out)), c_int(M), c_int(E),
                                            self._stream()), "hc_in_norm")

    def hc_update(self, x, S, sources, mix, scale, hc_mix, hc_out, next_in, next_norm, out):
        n = next_norm or (None, None, None)
        my, mw, mids, n_real, mh = mix or (None, None, None, 0, None)
        self._on_gpu(x, my, mw, mids, mh, scale, hc_mix, hc_out, next_in, out, *n)
        src = list(sources) + [(None, 0, 0.0)] * (2 - len(sources))
        T, E = x.shape[0], x.shape[1] // S
        self._check(self.lib.hfb_hc_update(
            _p(x), c_int(S), _p(src[0][0]), c_int(src[0][1]), c_float(src[0][2]), _p(src[1][0]), c_int(src[1][1]), c_float(src[1][2]),
            _p(my), _p(mw), _p(mids), c_int(mw.shape[1] if mw is not None else 0), c_int(n_real), _p(mh),
            c_int(_dt(mh) if mh is not None else 0), _p(scale), c_int(_dt(scale) if scale is not None else 0), _p(hc_mix), _p(hc_out),
            _p(next_in), _p(n[0]), _p(n[1]), _p(n[2]), c_int(_dt(n[1]) if next_norm else 0), _p(out),
            c_int(_dt(out) if out is not None else 0), c_int(T), c_int(E), self._stream()), "hc_update")

    # ---- recurrent mixers -----------------------------------------------------------------------------------
    def decay(self, z, splits, bias, rate, sign, out, H, d, z_stride, z_col0):
        self._on_gpu(bias, rate, out)
        self._check(self.lib.hfb_decay(_p(z), c_int(splits), c_int(z_stride), c_int(z_col0), _p(bias),
                                       c_int(_dt(bias) if bias is not None else 0), _p(rate), c_float(sign), _p(out),
                                       c_int(out.shape[0]), c_int(H), c_int(d), self._stream()), "decay")

    def short_conv(self, x, splits, w, carried, ctx, out, n_a, d_a, n_b, d_b, n_unit, n_scaled, scale, unit_eps):
        self._on_gpu(w, out, ctx.token_seq, ctx.cu_tokens, ctx.seq_slots)
        taps = w.shape[1]
        self._check(self.lib.hfb_short_conv(
            _p(x), c_int(splits), _p(w), c_int(_dt(w)), c_int(taps), _p(carried), c_int64(carried.stride(0)), _p(ctx.token_seq),
            _p(ctx.cu_tokens), _p(ctx.seq_slots), c_int(carried.shape[0]), c_int(ctx.num_seqs), _p(out), c_int(out.shape[0]),
            c_int(n_a), c_int(d_a), c_int(n_b), c_int(d_b), c_int(n_unit), c_int(n_scaled), c_float(scale), c_float(unit_eps),
            self._stream()), "short_conv")
        if taps > 1:
            self.launches += 1

    def linear_scan(self, q, k, v, a, beta_logit, q_scale, state, ctx, o, H, Hq, d, dv):
        self._on_gpu(ctx.cu_tokens, ctx.seq_slots)
        for t in (q, k, v, a, beta_logit, o):
            if t is not None and not t.is_cuda:
                raise KernelError("kernel arguments must be CUDA tensors")
        self._check(self.lib.hfb_linear_scan(
            _p(q), c_int(q.stride(0)), _p(k), c_int(k.stride(0)), _p(v), c_int(v.stride(0)), _p(a), c_int(a.stride(0)),
            _p(beta_logit), c_int(beta_logit.stride(0) if beta_logit is not None else 0), c_float(q_scale), _p(state),
            c_int64(state.stride(0)), _p(ctx.cu_tokens), _p(ctx.seq_slots), c_int(state.shape[0]), c_int(ctx.num_seqs), _p(o),
            c_int(o.stride(0)), c_int(H), c_int(Hq), c_int(d), c_int(dv), self._stream()), "linear_scan")

    def gate_norm(self, o, w, eps, g, g_splits, g_stride, g_col0, gate, out, H, dv):
        self._on_gpu(o, w, out)
        self._check(self.lib.hfb_gate_norm(_p(o), _p(w), c_int(_dt(w)), c_float(eps), _p(g), c_int(g_splits), c_int(g_stride),
                                           c_int(g_col0), c_int(gate), _p(out), c_int(_dt(out)), c_int(o.shape[0]), c_int(H), c_int(dv),
                                           self._stream()), "gate_norm")

    def layernorm(self, x, w, eps, center, out, rows):
        self._on_gpu(x, w, out, rows)
        self._check(self.lib.hfb_layernorm(_p(x), _p(w), c_float(eps), c_int(1 if center else 0), _p(rows), c_int(x.shape[0]), _p(out),
                                           c_int(_dt(out)), c_int(out.shape[0]), c_int(x.shape[1]), self._stream()), "layernorm")

    def norm_shift(self, x, w, eps, center, mu, state, ctx, out):
        self._on_gpu(x, w, mu, out, ctx.token_seq, ctx.cu_tokens, ctx.seq_slots)
        self._check(self.lib.hfb_layernorm_shift(
            _p(x), _p(w), _p(mu), c_float(eps), c_int(1 if center else 0), _p(state), c_int64(state.stride(0)), _p(ctx.token_seq),
            _p(ctx.cu_tokens), _p(ctx.seq_slots), c_int(state.shape[0]), _p(out), c_int(_dt(out)), c_int(x.shape[0]), c_int(x.shape[1]),
            self._stream()), "layernorm_shift")

    def gate_mul(self, a, g, g_splits, g_stride, g_col0, bias, gate, out):
        self._on_gpu(a, bias, out)
        self._check(self.lib.hfb_gate_mul(_p(a), c_int(_dt(a)), _p(g), c_int(g_splits), c_int(g_stride), c_int(g_col0), _p(bias),
                                          c_int(1 if gate == "sigmoid" else 0), _p(out), c_int(a.shape[0]), c_int(a.shape[1]),
                                          self._stream()), "gate_mul")

    def mingru_scan(self, row, splits, bias_z, bias_x, state, ctx, out, W):
        self._on_gpu(bias_z, bias_x, out, ctx.cu_tokens, ctx.seq_slots)
        b_dt = _dt(bias_z) if bias_z is not None else (_dt(bias_x) if bias_x is not None else 0)
        if bias_z is not None and bias_x is not None and bias_z.dtype != bias_x.dtype:
            raise KernelError("mingru_scan: the two biases must have one type")
        self._check(self.lib.hfb_mingru_scan(_p(row), c_int(splits), _p(bias_z), _p(bias_x), c_int(b_dt), _p(state),
                                             c_int64(state.stride(0)), _p(ctx.cu_tokens), _p(ctx.seq_slots), c_int(state.shape[0]),
                                             c_int(ctx.num_seqs), _p(out), c_int(_dt(out)), c_int(out.shape[0]), c_int(W),
                                             self._stream()), "mingru_scan")

    def moe_group(self, ids, experts, order, tile_expert, tile_p0, tile_n, n_tiles, tile):
        self._on_gpu(ids, order, tile_expert, tile_p0, tile_n, n_tiles)
        self._check(self.lib.hfb_moe_sort(_p(ids), c_int(ids.numel()), c_int(experts), c_int(tile), _p(order), _p(tile_expert),
                                          _p(tile_p0), _p(tile_n), _p(n_tiles), self._stream()), "moe_sort")

    def moe_gemm(self, a, w, out, act, order, src_div, scatter, tile_expert, tile_p0, tile_n, n_tiles, max_tiles, tile):
        self._on_gpu(a, w, out, order, tile_expert, tile_p0, tile_n, n_tiles)
        MOE_TILE = tile
        self._check(self.lib.hfb_moe_gemm(_p(a), c_int(_dt(a)), _p(w), c_int(_dt(w)), _p(out), c_int(_dt(out)), c_int(act),
                                          c_int(w.shape[1]), c_int(w.shape[2]), _p(order), c_int(src_div), c_int(1 if scatter else 0),
                                          _p(tile_expert), _p(tile_p0), _p(tile_n), _p(n_tiles), c_int(max_tiles), c_int(MOE_TILE),
                                          self._stream()), "moe_gemm")

    def moe_combine(self, y, weights, out):
        self._on_gpu(y, weights, out)
        T, top = weights.shape
        self._check(self.lib.hfb_moe_combine(_p(y), c_int(_dt(y)), _p(weights), _p(out), c_int(T), c_int(top),
                                             c_int(out.shape[1]), self._stream()), "moe_combine")

    def sample(self, logits, temps, top_ks, top_ps, min_ps, uniforms, out):
        self._on_gpu(logits, temps, top_ks, top_ps, min_ps, uniforms, out)
        M, V = logits.shape
        self._check(self.lib.hfb_sample(_p(logits), c_int(M), c_int(V), _p(temps), _p(top_ks), _p(top_ps), _p(min_ps),
                                        _p(uniforms), _p(out), self._stream()), "sample")

    def error_word_async(self, host_word: torch.Tensor) -> None:
        """Queues a copy of the error word into ``host_word`` (pinned int32[1]); valid once the stream got there."""
        rc = self.lib.hfb_error_word_peek_async(c_void_p(host_word.data_ptr()), self._stream())
        if rc != 0:
            raise KernelError(f"error word: {self.lib.hfb_last_error().decode()} (status {rc})")

    def error_word(self) -> int:
        w = ctypes.c_int32(0)
        self._check(self.lib.hfb_error_word_take(ctypes.byref(w), self._stream()), "error word")
        if w.value and self._counters is not None:
            self._counters.zero_()             # a kernel that gave up may have left tile counts behind
        return w.value
