"""A stand-in for the CUDA library, written with torch ops, for tests only.

It implements each kernel entry point's contract on whatever device the tensors live on, so the
host-side logic (batch building, block tables, page reuse, scheduling, trace replay) can be run on a
machine without a GPU, and so each CUDA kernel has a plain reference to be compared with on the
GPU.  It is never used by the product.
"""
import torch


class EmuBackend:
    name = "emu"

    def embed(self, ids, table, out):
        out.copy_(table[ids.long()].float())

    def embed_pair(self, ids, table, scale, pair, buckets, mul_prev, mul_cur, ctx, prev_state, out):
        x = table[ids.long()].float() * scale
        if pair is not None:
            toks, cu, slots = ids.tolist(), ctx.cu_tokens.tolist(), ctx.seq_slots.tolist()
            rows = []
            for s in range(len(slots)):
                prev = int(prev_state[slots[s]]) - 1
                for t in range(cu[s], cu[s + 1]):
                    rows.append(buckets if prev < 0 else (prev * mul_prev + toks[t] * mul_cur) % buckets)
                    prev = toks[t]
                prev_state[slots[s]] = prev + 1
            x = x + pair[torch.tensor(rows, device=ids.device)].float()
        out.copy_(x)

    def rmsnorm(self, x, w, eps, out, rows):
        xr = x if rows is None else x[rows.long()]
        r = 1.0 / torch.sqrt((xr * xr).sum(-1, keepdim=True) / xr.shape[-1] + eps)
        out.copy_(((xr * r) * w.float()).to(out.dtype))

    def linear(self, a, w, bias, out, accumulate):
        y = a.float() @ w.float().T
        if bias is not None:
            y = y + bias.float()
        if accumulate:
            out.add_(y)
        else:
            out.copy_(y.to(out.dtype))

    def rope_kv_write(self, qkv, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        T = qkv.shape[0]
        x = qkv.float().view(T, H + 2 * G, d)

        def rot(v):
            if n_rot == 0:
                return v
            half = n_rot // 2
            cs = cos_sin[positions.long()]
            c, s = cs[:, None, :, 0], cs[:, None, :, 1]
            a, b = v[..., :half], v[..., half:n_rot]
            return torch.cat([a * c - b * s, a * s + b * c, v[..., n_rot:]], -1)
        q_out.copy_(rot(x[:, :H]).reshape(T, H * d).to(q_out.dtype))
        if slots is None:
            return
        ok = slots >= 0
        kf, vf = k_cache.view(-1, G, d), v_cache.view(-1, G, d)
        kf[slots[ok].long()] = rot(x[:, H:H + G])[ok].to(k_cache.dtype)
        vf[slots[ok].long()] = x[:, H + G:][ok].to(v_cache.dtype)

    def paged_attention(self, q, k_cache, v_cache, meta, ctx, H, G, d, window, scale, out, tiles=None, dv=None, sinks=None,
                        zero_sink=False, slopes=None, head_scales=None, softcap=0.0):
        T = q.shape[0]
        bs = meta.block_size
        dv = d if dv is None else dv
        kf = k_cache.reshape(-1, G, d).float()
        vf = v_cache.reshape(-1, G, dv).float() if v_cache is not None else kf[..., :dv]      # a value inside its key
        seqs, poss, table = ctx.token_seq.tolist(), ctx.positions.tolist(), meta.block_table.tolist()
        qf = q.float().view(T, H, d)
        res = torch.zeros(T, H, dv, dtype=torch.float32, device=q.device)
        for t in range(T):
            pos, row = poss[t], table[seqs[t]]
            lo = max(0, pos - window + 1) if window > 0 else (pos // -window * -window if window < 0 else 0)
            idx = []
            for j in range(lo, pos + 1):
                page = row[j // bs]
                assert page >= 0, f"token {t}: key {j} lies in an unmapped block"
                idx.append(page * bs + j % bs)
            idx = torch.tensor(idx, device=q.device)
            k, v = kf[idx], vf[idx]                       # [n, G, d]
            for h in range(H):
                g = h // (H // G)
                s = (k[:, g] @ qf[t, h]) * scale
                if head_scales is not None:
                    s = s * head_scales[h]
                if softcap > 0:
                    s = softcap * torch.tanh(s / softcap)
                if slopes is not None:
                    s = s - slopes[h] * (pos - torch.arange(lo, pos + 1, device=q.device)).float()
                if sinks is not None or zero_sink:
                    sk = sinks[h].reshape(1) if sinks is not None else torch.zeros(1, device=q.device)
                    p = torch.softmax(torch.cat([s, sk]), 0)[:-1]
                else:
                    p = torch.softmax(s, 0)
                res[t, h] = p @ v[:, g]
        out.copy_(res.view(T, H * dv).to(out.dtype))

    def swiglu(self, gu, out, interleaved):
        F = out.shape[1]
        if interleaved:
            g, u = gu[:, 0::2].float(), gu[:, 1::2].float()
        else:
            g, u = gu[:, :F].float(), gu[:, F:].float()
        out.copy_(((g / (1.0 + torch.exp(-g))) * u).to(out.dtype))

    def linear_swiglu(self, a, w, gu_buf, out):
        self.linear(a, w, None, gu_buf, False)
        self.swiglu(gu_buf, out, True)

    def linear_residual_norm(self, a, w, bias, residual, norm_w, eps, xn_out, center=False, shift=None):
        self.linear(a, w, bias, residual, True)
        if xn_out is None:
            return
        if not center and shift is None:
            self.rmsnorm(residual, norm_w, eps, xn_out, None)
            return
        h = self._norm_rows(residual, norm_w, eps, center)
        if shift is not None:                   # a step of single tokens: row m is request m
            mu, state, seq_slots = shift
            slots = seq_slots.long()
            before = state[slots].clone()
            state[slots] = h
            h = h + (before - h) * mu
        xn_out.copy_(h.to(xn_out.dtype))

    def linear_rope_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d):
        self.linear(a, w, bias, qkv_buf, False)
        self.rope_kv_write(qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d)

    # ---- Dynamic Tanh norms, unit-rms heads, gated and routed feed-forwards ----
    @staticmethod
    def _dyt(x, p):
        alpha, w, b = p
        return torch.tanh(alpha.float() * x.float()) * w.float() + b.float()

    def dyt(self, x, params, out, rows):
        xr = x if rows is None else x[rows.long()]
        out.copy_(self._dyt(xr, params).to(out.dtype))

    def dyt_residual(self, y, post, residual, nxt, out, mix=None):
        v = y.float() if y is not None else torch.zeros_like(residual)
        if mix is not None:
            rows, w = mix
            v = v + (w[:, :, None] * rows.view(w.shape[0], w.shape[1], -1)).sum(1)
        residual.add_(self._dyt(v, post))
        if nxt is not None:
            out.copy_(self._dyt(residual, nxt).to(out.dtype))

    def linear_dyt_residual(self, a, w, bias, y_buf, post, residual, nxt, out, mix=None):
        self.linear(a, w, bias, y_buf, False)
        self.dyt_residual(y_buf, post, residual, nxt, out, mix=mix)

    def linear_rope_norm_kv(self, a, w, bias, qkv_buf, cos_sin, n_rot, positions, slots, q_out, k_cache, v_cache, H, G, d, dv,
                            norm_eps, norm_weights=None, value_mix=None, pairing="half"):
        self.linear(a, w, bias, qkv_buf, False)
        T = a.shape[0]

        def finish(v, weight=None):                    # [T, heads, d]
            if n_rot and pairing == "interleaved":
                v = torch.cat([self._rotate_pairs(v[..., :n_rot], cos_sin, positions), v[..., n_rot:]], -1)
            elif n_rot:
                half = n_rot // 2
                cs = cos_sin[positions.long()]
                c, s = cs[:, None, :, 0], cs[:, None, :, 1]
                x, y = v[..., :half], v[..., half:n_rot]
                v = torch.cat([x * c - y * s, x * s + y * c, v[..., n_rot:]], -1)
            if norm_eps is not None:
                v = v / torch.sqrt((v * v).mean(-1, keepdim=True) + norm_eps)
                if weight is not None:
                    v = v * weight
            return v
        qw, kw = norm_weights or (None, None)
        q_out.copy_(finish(qkv_buf[:, :H * d].view(T, H, d), qw).reshape(T, H * d).to(q_out.dtype))
        if not G or slots is None:
            return
        ok = slots >= 0
        k = finish(qkv_buf[:, H * d:(H + G) * d].view(T, G, d), kw)
        v = qkv_buf[:, (H + G) * d:].view(T, G, dv)
        if value_mix is not None:
            first, mode, lam = value_mix
            if mode == 1:
                first.copy_(v.reshape(T, G * dv))
            else:
                v = (1.0 - lam) * v + lam * first.view(T, G, dv)
        k_cache.view(-1, G, d)[slots[ok].long()] = k[ok].to(k_cache.dtype)
        if dv:
            v_cache.view(-1, G, dv)[slots[ok].long()] = v[ok].to(v_cache.dtype)

    @staticmethod
    def _rotate_pairs(v, cos_sin, positions):
        """Pairs (2i, 2i + 1) of the last axis, all of it."""
        cs = cos_sin[positions.long()]
        c, s = cs[..., 0], cs[..., 1]
        while c.dim() < v.dim():
            c, s = c.unsqueeze(1), s.unsqueeze(1)
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * c - b * s, a * s + b * c], -1).flatten(-2)

    def linear_latent_split(self, a, w, buf, q_norm_w, kv_norm_w, eps, cos_sin, positions, slots, cq_out, cache, q_rank, kv_rank, rot):
        self.linear(a, w, None, buf, False)
        unit = lambda v: v / torch.sqrt((v * v).mean(-1, keepdim=True) + eps)
        cq_out.copy_((unit(buf[:, :q_rank]) * q_norm_w).to(cq_out.dtype))
        c = unit(buf[:, q_rank:q_rank + kv_rank]) * kv_norm_w
        r = buf[:, q_rank + kv_rank:]
        if rot:
            r = self._rotate_pairs(r, cos_sin, positions)
        if slots is None:
            return
        ok = slots >= 0
        cache.view(-1, kv_rank + rot)[slots[ok].long()] = torch.cat([c, r], -1)[ok].to(cache.dtype)

    def linear_latent_query(self, a, w, buf, cos_sin, positions, q_plain, q_att, H, d, rot, att_col):
        self.linear(a, w, None, buf, False)
        T = a.shape[0]
        q = buf.view(T, H, d + rot)
        q_plain.copy_(q[..., :d].reshape(T, H * d).to(q_plain.dtype))
        if rot:
            q_att.view(T, H, -1)[..., att_col:att_col + rot] = self._rotate_pairs(q[..., d:], cos_sin, positions).to(q_att.dtype)

    def headwise_linear(self, x, w, out, H, in_row, out_row):
        T, (_, N, K) = x.shape[0], w.shape
        y = torch.einsum("thk,hnk->thn", x.view(T, H, in_row)[..., :K].float(), w.float())
        out.view(T, H, out_row)[..., :N] = y.to(out.dtype)

    @staticmethod
    def _activate(z, act):
        if act == 0:
            return z / (1.0 + torch.exp(-z))
        if act == 1:
            return torch.relu(z)
        if act == 2:
            return 0.5 * z * (1.0 + torch.tanh(0.7978845608028654 * (z + 0.044715 * z ** 3)))
        if act == 3:
            return torch.relu(z) ** 2
        return z

    def linear_glu(self, a, w, gu_buf, out, act):
        self.linear(a, w, None, gu_buf, False)
        g, u = gu_buf[:, 0::2].float(), gu_buf[:, 1::2].float()
        out.copy_((self._activate(g, act) * u).to(out.dtype))

    def linear_act(self, a, w, out, act):
        out.copy_(self._activate(a.float() @ w.float().T, act).to(out.dtype))

    def scale_(self, x, s):
        x.mul_(s)

    def moe_route(self, h, w, b, top, ids, weights, logits):
        z = h.float() @ w.float().T
        if b is not None:
            z = z + b.float()
        logits.copy_(z)
        zc, idx = torch.sort(z, dim=-1, descending=True, stable=True)
        ids.copy_(idx[:, :top].int())
        weights.copy_(torch.softmax(zc[:, :top], -1))

    def moe_route_softmax(self, h, w, correction, top, n_groups, keep, scale, ids, weights, logits):
        z = h.float() @ w.float().T
        logits.copy_(z)
        s = torch.softmax(z, -1)
        ch = s + correction.float() if correction is not None else s.clone()
        T, E = s.shape
        if n_groups > 1 and keep < n_groups:
            per = E // n_groups
            best = ch.view(T, n_groups, per).max(-1).values
            kept = torch.sort(best, dim=-1, descending=True, stable=True).indices[:, :keep]
            allow = torch.zeros(T, n_groups, dtype=torch.bool, device=s.device)
            allow.scatter_(1, kept, True)
            ch = torch.where(allow[:, :, None].expand(T, n_groups, per).reshape(T, E), ch, torch.full_like(ch, float("-inf")))
        idx = torch.sort(ch, dim=-1, descending=True, stable=True).indices[:, :top]
        ids.copy_(idx.int())
        weights.copy_(torch.gather(s, 1, idx) * scale)

    def product_sums(self, a, w, buf, finished=False):
        self.linear(a, w, None, buf, False)
        return buf, 1

    # ---- hyper-connections ----
    def hc_spread(self, emb, x, S):
        x.copy_(emb.repeat(1, S))

    def hc_in_norm(self, x, S, in_w, rows, norm, out):
        xr = (x if rows is None else x[rows.long()]).view(-1, S, out.shape[1])
        u = xr.sum(1) if in_w is None else (in_w[None, :, None] * xr).sum(1)
        out.copy_((self._dyt(u, norm) if norm is not None else u).to(out.dtype))

    def hc_update(self, x, S, sources, mix, scale, hc_mix, hc_out, next_in, next_norm, out):
        T = x.shape[0]
        E = x.shape[1] // S
        y = torch.zeros(T, E, dtype=torch.float32, device=x.device)
        for src, splits, factor in sources:
            y = y + factor * src.reshape(-1)[:splits * T * E].view(splits, T, E).sum(0)
        if mix is not None:
            my, mw, mids, n_real, mh = mix
            rows = my.view(T, mw.shape[1], E)
            if mids is not None:
                rows = torch.where((mids >= n_real)[:, :, None], mh.float()[:, None, :], rows)
            y = y + (mw[:, :, None] * rows).sum(1)
        if scale is not None:
            y = y * scale.float()
        old = x.view(T, S, E).clone()
        new = torch.einsum("sd,tse->tde", hc_mix, old) + hc_out[None, :, None] * y[:, None, :]
        x.copy_(new.reshape(T, S * E))
        if out is not None:
            u = new.sum(1) if next_in is None else (next_in[None, :, None] * new).sum(1)
            out.copy_((self._dyt(u, next_norm) if next_norm is not None else u).to(out.dtype))

    # ---- recurrent mixers ----
    def decay(self, z, splits, bias, rate, sign, out, H, d, z_stride, z_col0):
        T = out.shape[0]
        v = z.reshape(-1)[:splits * T * z_stride].view(splits, T, z_stride).sum(0)[:, z_col0:z_col0 + H * d]
        if bias is not None:
            v = v + bias.float()
        sp = torch.nn.functional.softplus(sign * v, threshold=20.0)
        out.copy_(torch.exp(-rate.repeat_interleave(d)[None, :] * sp))

    def short_conv(self, x, splits, w, carried, ctx, out, n_a, d_a, n_b, d_b, n_unit, n_scaled, scale, unit_eps):
        T, C = out.shape
        xs = x.reshape(-1)[:splits * T * C].view(splits, T, C).sum(0)
        taps = w.shape[1]
        K = taps - 1
        wf = w.float()
        cu, slots = ctx.cu_tokens.tolist(), ctx.seq_slots.tolist()
        for s in range(len(slots)):
            a, b = cu[s], cu[s + 1]
            hist = torch.cat([carried[slots[s]][:K], xs[a:b]]) if K else xs[a:b]
            y = sum(hist[i:i + (b - a)] * wf[:, i] for i in range(taps))
            out[a:b] = y * torch.sigmoid(y)
            if K:
                carried[slots[s]][:K] = hist[hist.shape[0] - K:]
        at = 0
        for u in range(n_a + n_b):
            n = d_a if u < n_a else d_b
            if u < n_unit:
                seg = out[:, at:at + n]
                r = 1.0 / torch.sqrt((seg * seg).sum(-1, keepdim=True) + unit_eps)
                out[:, at:at + n] = seg * r * (scale if u < n_scaled else 1.0)
            at += n

    def linear_scan(self, q, k, v, a, beta_logit, q_scale, state, ctx, o, H, Hq, d, dv):
        cu, slots = ctx.cu_tokens.tolist(), ctx.seq_slots.tolist()
        rep = H // Hq
        for s in range(len(slots)):
            S = state[slots[s]].transpose(1, 2).clone()              # [H, d, dv]
            for t in range(cu[s], cu[s + 1]):
                qt = q[t].view(Hq, d).repeat_interleave(rep, 0)
                kt = k[t].view(Hq, d).repeat_interleave(rep, 0)
                vt, at = v[t].view(H, dv), a[t].view(H, d)
                S = at[:, :, None] * S
                u = vt
                if beta_logit is not None:
                    u = torch.sigmoid(beta_logit[t])[:, None] * (vt - torch.einsum("hij,hi->hj", S, kt))
                S = S + kt[:, :, None] * u[:, None, :]
                o[t] = (torch.einsum("hij,hi->hj", S, qt) * q_scale).reshape(-1)
            state[slots[s]] = S.transpose(1, 2)

    def gate_norm(self, o, w, eps, g, g_splits, g_stride, g_col0, gate, out, H, dv):
        T = o.shape[0]
        gz = g.reshape(-1)[:g_splits * T * g_stride].view(g_splits, T, g_stride).sum(0)[:, g_col0:g_col0 + H * dv].reshape(T, H, dv)
        x = o.view(T, H, dv)
        y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w.float()
        y = y * (gz * torch.sigmoid(gz) if gate == 0 else torch.sigmoid(gz))
        out.copy_(y.reshape(T, H * dv).to(out.dtype))

    # ---- layer norm, token shift, gates, minGRU ----
    @staticmethod
    def _norm_rows(x, w, eps, center):
        d = x - x.mean(-1, keepdim=True) if center else x
        return d / torch.sqrt((d * d).mean(-1, keepdim=True) + eps) * w

    def layernorm(self, x, w, eps, center, out, rows):
        src = x if rows is None else x[rows.long()]
        out.copy_(self._norm_rows(src, w, eps, center).to(out.dtype))

    def norm_shift(self, x, w, eps, center, mu, state, ctx, out):
        h = self._norm_rows(x, w, eps, center)
        cu, slots = ctx.cu_tokens.tolist(), ctx.seq_slots.tolist()
        for s in range(len(slots)):
            a, b = cu[s], cu[s + 1]
            before = torch.cat([state[slots[s]][None, :], h[a:b - 1]])
            out[a:b] = (h[a:b] + (before - h[a:b]) * mu).to(out.dtype)
            state[slots[s]] = h[b - 1]

    def gate_mul(self, a, g, g_splits, g_stride, g_col0, bias, gate, out):
        T, C = a.shape
        z = g.reshape(-1)[:g_splits * T * g_stride].view(g_splits, T, g_stride).sum(0)[:, g_col0:g_col0 + C]
        if bias is not None:
            z = z + bias
        out.copy_((a.float() * (torch.sigmoid(z) if gate == "sigmoid" else z * torch.sigmoid(z))).to(out.dtype))

    def mingru_scan(self, row, splits, bias_z, bias_x, state, ctx, out, W):
        T = out.shape[0]
        r = row.reshape(-1)[:splits * T * 3 * W].view(splits, T, 3 * W).sum(0)
        z = torch.sigmoid(r[:, :W] + (bias_z.float() if bias_z is not None else 0))
        u = r[:, W:2 * W] + (bias_x.float() if bias_x is not None else 0)
        cand = torch.where(u >= 0, u + 0.5, torch.sigmoid(u))
        g = r[:, 2 * W:]
        cu, slots = ctx.cu_tokens.tolist(), ctx.seq_slots.tolist()
        for s in range(len(slots)):
            S = state[slots[s]].clone()
            for t in range(cu[s], cu[s + 1]):
                S = (1.0 - z[t]) * S + z[t] * cand[t]
                out[t] = (S * g[t] * torch.sigmoid(g[t])).to(out.dtype)
            state[slots[s]] = S

    def moe_group(self, ids, experts, order, tile_expert, tile_p0, tile_n, n_tiles, tile):
        MOE_TILE = tile
        flat = ids.reshape(-1)
        srt = torch.sort(flat, stable=True).indices.int()
        order[:flat.numel()] = srt
        keep = flat < experts                    # an id beyond the experts takes no place
        srt = srt[keep[srt.long()]]
        order[:srt.numel()] = srt
        counts = torch.bincount(flat[keep].long(), minlength=experts).tolist()
        n = at = 0
        for e, c in enumerate(counts):
            for p0 in range(0, c, MOE_TILE):
                tile_expert[n], tile_p0[n], tile_n[n] = e, at + p0, min(MOE_TILE, c - p0)
                n += 1
            at += c
        n_tiles[0] = n

    def moe_gemm(self, a, w, out, act, order, src_div, scatter, tile_expert, tile_p0, tile_n, n_tiles, max_tiles, tile):
        assert int(n_tiles[0]) <= max_tiles
        for i in range(int(n_tiles[0])):
            e, p0, n = int(tile_expert[i]), int(tile_p0[i]), int(tile_n[i])
            places = torch.arange(p0, p0 + n)
            pairs = order[places].long()
            src = pairs // src_div if src_div else places
            dst = pairs if scatter else places
            z = a[src].float() @ w[e].float().T
            if act >> 8:
                out[dst] = (self._activate(z[:, 0::2], act & 255) * z[:, 1::2]).to(out.dtype)
            else:
                out[dst] = self._activate(z, act).to(out.dtype)

    def moe_combine(self, y, weights, out):
        T, top = weights.shape
        out.copy_((weights[:, :, None] * y.float().view(T, top, -1)).sum(1))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).int())

    def error_word(self):
        return 0

    def sample(self, logits, temps, top_ks, top_ps, min_ps, uniforms, out):
        import plain_qwen2 as plain

        class Fixed:
            def __init__(self, u):
                self.u = u

            def uniform(self):
                return self.u
        rows = logits.float().cpu().numpy()
        for i in range(rows.shape[0]):
            out[i] = plain.sample(rows[i], float(temps[i]), int(top_ks[i]), float(top_ps[i]), float(min_ps[i]),
                                  Fixed(uniforms[i].cpu().numpy()))
