"""Plain, slow implementation of the Silupel decoder in float64, whole sequences, no cache.

One function per mechanism, written from the design's equations and sharing no code with the
package.  A model is (config dict, {tensor name: float64 numpy array}).

Notation: x is the residual stream [T, width]; a layer run is
    h = shift(layernorm(x));  x += mixer(h);  x += ff(layernorm(x))
with layernorm(x) = (x - mean) / sqrt(var + eps) * w (no bias) and
shift(h)_t = h_t + (h_(t-1) - h_t) * mu (h_(-1) = 0), mu a stored vector per layer.
"""
import json
import math
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


# ---- element-wise --------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softmax_rows(s):
    """Softmax over the last axis; entries of -inf get weight zero."""
    m = s.max(-1, keepdims=True)
    e = np.exp(s - m)
    return e / e.sum(-1, keepdims=True)


# ---- norms ---------------------------------------------------------------------------------------
def layer_norm(x, w, eps):
    d = x - x.mean(-1, keepdims=True)
    return d / np.sqrt((d * d).mean(-1, keepdims=True) + eps) * w


def rms_norm(x, w, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps) * w


# ---- token shift ---------------------------------------------------------------------------------
def token_shift(h, mu):
    """Every row moves towards the row before it (as that row was before the move), by mu per feature."""
    before = np.concatenate([np.zeros_like(h[:1]), h[:-1]], 0)
    return h + (before - h) * mu


# ---- rotation ------------------------------------------------------------------------------------
def rot_frequencies(rot):
    """One frequency per pair; with 'scaling', long wavelengths are stretched: short ones (under original / high) stay,
    long ones (over original / low) are divided by the factor, those between are blended."""
    n = rot["dims"]
    f = np.array([float(rot["base"]) ** (-2.0 * i / n) for i in range(n // 2)])
    sc = rot.get("scaling")
    if not sc:
        return f
    out = f.copy()
    for i, fi in enumerate(f):
        wave = 2.0 * math.pi / fi
        if wave < sc["original"] / sc["high"]:
            continue
        if wave > sc["original"] / sc["low"]:
            out[i] = fi / sc["factor"]
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out[i] = (1.0 - s) * fi / sc["factor"] + s * fi
    return out


def rotate_half_layout(x, positions, rot):
    """x [T, heads, D]: the first rot.dims dimensions of each head turn, dimension i with i + dims/2."""
    n = rot["dims"]
    half = n // 2
    ang = np.asarray(positions, dtype=np.float64)[:, None] * rot_frequencies(rot)[None, :]      # [T, half]
    c, s = np.cos(ang)[:, None, :], np.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:n]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:n] = v * c + u * s
    return out


# ---- mixers --------------------------------------------------------------------------------------
def mingru(m, W, p, h):
    """z = sigmoid(Wz h + bz); u = Wx h + bx; candidate = u + 1/2 (u >= 0) or sigmoid(u) (u < 0);
    S_t = (1 - z_t) S_(t-1) + z_t candidate_t from S = 0; out = Wo (S_t * silu(Wg h))."""
    z = sigmoid(h @ W[p + ".z"].T + W[p + ".z.b"])
    u = h @ W[p + ".x"].T + W[p + ".x.b"]
    cand = np.where(u >= 0, u + 0.5, sigmoid(u))
    S = np.zeros(m["width"])
    states = np.zeros_like(z)
    for t in range(h.shape[0]):
        S = (1.0 - z[t]) * S + z[t] * cand[t]
        states[t] = S
    return (states * silu(h @ W[p + ".g"].T)) @ W[p + ".o"].T


def chunk_mask(T, size):
    """[T, T] True where query i sees key j: j <= i and both in the same chunk counted from position 0."""
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return (j <= i) & (i // size == j // size)


def causal_mask(T):
    i, j = np.arange(T)[:, None], np.arange(T)[None, :]
    return j <= i


def attention(m, W, p, h):
    """Grouped heads with biases, partial rotation, a factor per head on the scores, a tanh cap, a chunked mask and a
    sigmoid gate on the heads' outputs."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ W[p + ".q"].T + W[p + ".q.b"]).reshape(T, H, d)
    k = (h @ W[p + ".k"].T + W[p + ".k.b"]).reshape(T, G, d)
    v = (h @ W[p + ".v"].T + W[p + ".v.b"]).reshape(T, G, dv)
    pos = np.arange(T)
    q, k = rotate_half_layout(q, pos, m["rot"]), rotate_half_layout(k, pos, m["rot"])
    see = chunk_mask(T, m["mask"]["size"])
    cap = m["softcap"]
    out = np.zeros((T, H, dv))
    for a in range(H):
        g = a // (H // G)
        s = (q[:, a] @ k[:, g].T) * m["scale"] * W[p + ".temp"][a]
        s = cap * np.tanh(s / cap)
        s = np.where(see, s, -np.inf)
        out[:, a] = softmax_rows(s) @ v[:, g]
    gate = sigmoid(h @ W[p + ".g"].T)
    return (out.reshape(T, H * dv) * gate) @ W[p + ".o"].T + W[p + ".o.b"]


def latent_attention(m, W, p, h, eps):
    """Queries through a normed latent; keys and values expanded from a normed latent; one rotated key part shared by the
    heads; causal."""
    T = h.shape[0]
    H, d, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ W[p + ".dq"].T, W[p + ".dq.norm"], eps)
    q = (cq @ W[p + ".uq"].T).reshape(T, H, d + dr)
    down = h @ W[p + ".dkv"].T
    c = rms_norm(down[:, :R], W[p + ".dkv.norm"], eps)
    pos = np.arange(T)
    rot = dict(m["rot"], dims=dr)
    k_rot = rotate_half_layout(down[:, None, R:], pos, rot)[:, 0]                  # [T, dr]
    q_rot = rotate_half_layout(q[..., d:], pos, rot)                               # [T, H, dr]
    k_plain = (c @ W[p + ".uk"].T).reshape(T, H, d)
    val = (c @ W[p + ".uv"].T).reshape(T, H, dv)
    see = causal_mask(T)
    out = np.zeros((T, H, dv))
    for a in range(H):
        s = (q[:, a, :d] @ k_plain[:, a].T + q_rot[:, a] @ k_rot.T) * m["scale"]
        s = np.where(see, s, -np.inf)
        out[:, a] = softmax_rows(s) @ val[:, a]
    return out.reshape(T, H * dv) @ W[p + ".o"].T


# ---- feed-forward --------------------------------------------------------------------------------
def dense_ff(W, p, h):
    return (gelu_tanh(h @ W[p + ".gate"].T) * (h @ W[p + ".up"].T)) @ W[p + ".down"].T


# ---- the model -----------------------------------------------------------------------------------
def run_order(cfg):
    """Layer indices in the order they run: layers start .. stop - 1 run `times` times in a row."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, W, ids, layers_out=None):
    """Logits [T, vocab] of one whole sequence.  ``layers_out`` (a list) receives the stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][np.asarray(ids)]
    for i in run_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}"
        h = token_shift(layer_norm(x, W[p + ".norm1"], eps), W[p + ".shift"])
        m = L["mixer"]
        if L["type"] == "mingru":
            y = mingru(m, W, p + ".mix", h)
        elif L["type"] == "attention":
            y = attention(m, W, p + ".mix", h)
        elif L["type"] == "latent_attention":
            y = latent_attention(m, W, p + ".mix", h, eps)
        else:
            raise ValueError(L["type"])
        x = x + y
        if L.get("mlp") is not None:
            x = x + dense_ff(W, p + ".mlp", layer_norm(x, W[p + ".norm2"], eps))
        if layers_out is not None:
            layers_out.append(x.copy())
    return layer_norm(x, W["final.norm"], eps) @ W["head"].T


def greedy(cfg, W, ids, n):
    """n tokens by arg-max, each from a whole forward pass."""
    ids, out = list(ids), []
    for _ in range(n):
        out.append(int(np.argmax(forward(cfg, W, ids)[-1])))
        ids.append(out[-1])
    return out
