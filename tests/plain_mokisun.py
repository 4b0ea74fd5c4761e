"""Plain, slow implementation of the Mokisun decoder in float64, whole sequences, no cache.

One function per mechanism, written from the design's equations and sharing no code with the
package.  A model is (config dict, {tensor name: float64 numpy array}).

Notation: the stream is kept in ``streams`` copies X[s] ([T, width] each), all equal to the embedding at the start.
A sublayer f with norm n, layer scale c and hyper-connection (a [s], B [s, s], d [s]) does
    u = sum_s a[s] X[s];   y = c * f(n(u));   X'[t] = sum_s B[s, t] X[s] + d[t] * y      (all t from the old X)
and a layer is two of them (mixer, feed-forward).  The model's output is head . n_final(sum_s X[s]).
Every norm of the stream is a Dynamic Tanh  tanh(alpha * x) * w + b.
"""
import json
import os
import struct

import numpy as np


# ---- files ---------------------------------------------------------------------------------------
def read_safetensors(path):
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, m in head.items():
        if name == "__metadata__":
            continue
        a, b = m["data_offsets"]
        raw = data[a:b]
        if m["dtype"] == "BF16":
            v = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32)
        elif m["dtype"] == "F32":
            v = np.frombuffer(raw, dtype="<f4")
        elif m["dtype"] == "I32":
            v = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(m["dtype"])
        out[name] = v.astype(np.float64).reshape(m["shape"])
    return out


def read_folder(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small functions -----------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def dynamic_tanh(x, W, name):
    return np.tanh(W[name + ".alpha"] * x) * W[name] + W[name + ".b"]


def rms_norm(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


# ---- attention -----------------------------------------------------------------------------------
def rotate_interleaved(x, positions, rot):
    """x [T, heads, dim]: dimensions (2i, 2i + 1), i < dims/2, turn by position * base^(-2i/dims)."""
    if not rot or not rot.get("dims"):
        return x
    dims = rot["dims"]
    i = np.arange(dims // 2, dtype=np.float64)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * rot["base"] ** (-2.0 * i / dims)
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    out = x.copy()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def windowed_attention(q, k, v, scale, window, sink, slopes=None, rows=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv].  Token i sees j with 0 <= i - j < window.  ``sink`` [H]: a score per head
    that joins the softmax's denominator and has no value.  ``slopes`` [H]: slope * (i - j) is taken off the score.
    ``rows``: the queries to compute (the others' rows stay zero)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = np.zeros((T, H, v.shape[2]))
    for h in range(H):
        g = h // (H // G)
        for i in (range(T) if rows is None else rows):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            if slopes is not None:
                s = s - slopes[h] * (i - np.arange(lo, i + 1))
            m = max(s.max(), sink[h])
            e = np.exp(s - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(0) / (e.sum() + np.exp(sink[h] - m))
    return out


def mixer_attention(h, W, p, m, positions, cfg):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T).reshape(T, H, d)
    k = (h @ W[p + ".k"].T).reshape(T, G, d)
    v = (h @ W[p + ".v"].T).reshape(T, G, dv)
    q, k = rotate_interleaved(q, positions, m.get("rot")), rotate_interleaved(k, positions, m.get("rot"))
    o = windowed_attention(q, k, v, m["scale"], m["mask"]["size"], W[p + ".sink"])
    return o.reshape(T, H * dv) @ W[p + ".o"].T


def distance_slopes(H):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)])


def mixer_biased_attention(h, W, p, m):
    """The left half of a 'parallel' mixer: values are the keys, no rotation, a bias linear in the distance, a sink of
    score zero."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q = (h @ W[p + ".q"].T).reshape(T, H, d)
    k = (h @ W[p + ".k"].T).reshape(T, G, d)
    o = windowed_attention(q, k, k, m["scale"], m["mask"]["size"], np.zeros(H), distance_slopes(H))
    return o.reshape(T, H * d) @ W[p + ".o"].T


# ---- recurrent mixers ----------------------------------------------------------------------------
def short_convolution(x, w):
    """x [T, C], w [C, taps]: y_t = sum_i w[:, i] x_(t - taps + 1 + i), zeros before the start."""
    T, taps = x.shape[0], w.shape[1]
    pad = np.concatenate([np.zeros((taps - 1, x.shape[1])), x])
    return sum(pad[i:i + T] * w[:, i] for i in range(taps))


def delta_rule(q, k, v, beta, g):
    """q, k [T, H, d]; v [T, H, dv]; beta [T, H]; g [T, H, d].  Per head: S <- g S; u = beta (v - S^T k); S += k u^T;
    o = S^T q."""
    T, H, d = q.shape
    out = np.zeros_like(v)
    for h in range(H):
        S = np.zeros((d, v.shape[2]))
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, h])
            S = S + np.outer(k[t, h], u)
            out[t, h] = S.T @ q[t, h]
    return out


def mixer_gated_delta(h, W, p, m, cfg):
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    proj = {}
    for x in "qkv":
        proj[x] = silu(short_convolution(h @ W[f"{p}.{x}"].T, W[f"{p}.{x}.conv"]))
    unit = lambda x: x / np.sqrt((x * x).sum(-1, keepdims=True) + 1e-6)
    q = unit(proj["q"].reshape(T, G, d)) * d ** -0.5
    k = unit(proj["k"].reshape(T, G, d))
    v = proj["v"].reshape(T, H, dv)
    rep = H // G
    q, k = np.repeat(q, rep, axis=1), np.repeat(k, rep, axis=1)
    beta = sigmoid(h @ W[p + ".b"].T)
    dt = softplus((h @ W[p + ".a1"].T) @ W[p + ".a2"].T + W[p + ".dt_bias"]).reshape(T, H, d)
    g = np.exp(-np.exp(W[p + ".A_log"])[None, :, None] * dt)
    o = delta_rule(q, k, v, beta, g)
    o = rms_norm(o, cfg["norm"]["eps"]) * W[p + ".norm"]
    o = o * sigmoid((h @ W[p + ".g1"].T) @ W[p + ".g2"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ W[p + ".o"].T


def mixer_parallel(h, W, p, m, cfg):
    return (m["left_scale"] * mixer_biased_attention(h, W, p + ".left", m["left"])
            + m["right_scale"] * mixer_gated_delta(h, W, p + ".right", m["right"], cfg))


def mixer_gla(h, W, p, m, cfg):
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T).reshape(T, H, d) * d ** -0.5
    k = (h @ W[p + ".k"].T).reshape(T, H, d)
    v = (h @ W[p + ".v"].T).reshape(T, H, dv)
    z = (h @ W[p + ".a1"].T) @ W[p + ".a2"].T + W[p + ".a2.b"]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, d)
    o = np.zeros((T, H, dv))
    for hh in range(H):
        S = np.zeros((d, dv))
        for t in range(T):
            S = alpha[t, hh][:, None] * S + np.outer(k[t, hh], v[t, hh])
            o[t, hh] = S.T @ q[t, hh]
    o = rms_norm(o, cfg["norm"]["eps"]) * W[p + ".norm"]
    return (o.reshape(T, H * dv) * silu(h @ W[p + ".g"].T)) @ W[p + ".o"].T


# ---- feed-forward --------------------------------------------------------------------------------
def route(h, W, p, r):
    """(chosen ids [T, top], weights [T, top]); ids >= r['experts'] name identity experts."""
    n_all = r["experts"] + r.get("identity", 0)
    z = h @ W[p + ".router"].T
    z = z - z.max(-1, keepdims=True)
    s = np.exp(z) / np.exp(z).sum(-1, keepdims=True)
    choice = s + W[p + ".correction"]
    groups = r.get("groups") or {"count": 1, "keep": 1}
    per = n_all // groups["count"]
    best = choice.reshape(-1, groups["count"], per).max(-1)
    ids = np.zeros((h.shape[0], r["top"]), dtype=np.int64)
    for t in range(h.shape[0]):
        keep = np.argsort(-best[t], kind="stable")[:groups["keep"]]
        c = np.full(n_all, -np.inf)
        for gi in keep:
            c[gi * per:(gi + 1) * per] = choice[t, gi * per:(gi + 1) * per]
        ids[t] = np.argsort(-c, kind="stable")[:r["top"]]
    return ids, np.take_along_axis(s, ids, axis=1) * r["scale"]


def feed_forward_moe(h, W, p, mlp):
    r = mlp["router"]
    ids, wts = route(h, W, p, r)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, w in zip(ids[t], wts[t]):
            if e >= r["experts"]:
                out[t] += w * h[t]
            else:
                q = f"{p}.e{e}"
                out[t] += w * ((silu(h[t] @ W[q + ".gate"].T) * (h[t] @ W[q + ".up"].T)) @ W[q + ".down"].T)
    return out


# ---- the model -----------------------------------------------------------------------------------
def hyper_step(X, W, p, f, norm_name, scale_name):
    """One sublayer under hyper-connections; X [streams, T, width]."""
    u = np.tensordot(W[p + ".in"], X, axes=(0, 0))
    y = W[scale_name] * f(dynamic_tanh(u, W, norm_name))
    return np.tensordot(W[p + ".mix"].T, X, axes=(1, 0)) + W[p + ".out"][:, None, None] * y


def forward(cfg, W, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence; with ``return_layers`` also the sum of the streams after every layer."""
    T = len(tokens)
    positions = np.arange(T)
    x = W["embed"][np.asarray(tokens)]
    X = np.stack([x] * cfg["streams"])
    after = []
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}", L["mixer"]
        if L["type"] == "attention":
            f = lambda h: mixer_attention(h, W, p + ".mix", m, positions, cfg)
        elif L["type"] == "parallel":
            f = lambda h: mixer_parallel(h, W, p + ".mix", m, cfg)
        elif L["type"] == "gla":
            f = lambda h: mixer_gla(h, W, p + ".mix", m, cfg)
        else:
            raise ValueError(L["type"])
        X = hyper_step(X, W, p + ".hc1", f, p + ".norm1", p + ".ls1")
        if L.get("mlp") is not None:
            X = hyper_step(X, W, p + ".hc2", lambda h: feed_forward_moe(h, W, p + ".mlp", L["mlp"]), p + ".norm2", p + ".ls2")
        after.append(X.sum(0))
    logits = dynamic_tanh(X.sum(0), W, "final.norm") @ W["head"].T
    return (logits, np.stack(after)) if return_layers else logits


def greedy(cfg, W, prompt, n):
    """n tokens by arg-max, the whole sequence computed anew for each."""
    ids, out = list(prompt), []
    for _ in range(n):
        t = int(np.argmax(forward(cfg, W, ids)[-1]))
        out.append(t)
        ids.append(t)
    return out
