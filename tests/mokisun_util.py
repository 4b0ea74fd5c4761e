"""Small Mokisun configurations, model folders with random weights, and the plain implementation's logits."""
import numpy as np
import torch

import plain_mokisun as plain


def gla(heads, dim, vdim, tau, a_rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "a_rank": a_rank}}


def att(heads, kv_heads, dim, vdim, scale, window, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window}}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "attention", "mixer": m}


def par(left, right, left_scale, right_scale):
    """left: (heads, kv_heads, dim, scale, window); right: (heads, kv_heads, dim, vdim, taps, a_rank, g_rank)."""
    lh, lg, ld, ls, lw = left
    rh, rg, rd, rv, taps, ar, gr = right
    return {"type": "parallel", "mixer": {
        "left": {"heads": lh, "kv_heads": lg, "dim": ld, "vdim": ld, "scale": ls, "mask": {"size": lw}},
        "right": {"heads": rh, "kv_heads": rg, "dim": rd, "vdim": rv, "conv": taps, "a_rank": ar, "g_rank": gr},
        "left_scale": left_scale, "right_scale": right_scale}}


def moe(experts, identity, top, ff, scale, groups=None):
    r = {"experts": experts, "identity": identity, "top": top, "scale": scale}
    if groups:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": r}


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


def model(vocab, width, streams, eps, layers):
    return {"architecture": "Mokisun", "vocab": vocab, "width": width, "streams": streams, "norm": {"eps": eps}, "layers": layers}


# Odd sizes throughout: three copies of the stream, value heads wider and narrower than key heads, fewer query/key heads
# than value heads in the delta rule, three and two taps, a router without identity experts and without groups, one
# expert a token, layers without a feed-forward, a window shorter than a page and one longer than most portions,
# attention without rotation.
ODD = model(211, 72, 3, 1e-5, [
    layer(gla(3, 24, 40, 7.0, 5), moe(5, 1, 2, 40, 2.0, (3, 2))),
    layer(att(6, 3, 24, 40, 0.3, 9, (8, 500.0)), None),
    layer(par((4, 2, 16, 0.35, 13), (4, 2, 24, 20, 3, 6, 7), 0.7, 1.3), moe(4, 0, 1, 24, 1.0)),
    layer(gla(2, 40, 24, 3.0, 4), moe(6, 2, 3, 32, 0.8, (4, 2))),
    layer(par((6, 6, 8, 0.5, 50), (3, 3, 16, 16, 2, 4, 4), 1.1, 0.6), None),
    layer(att(4, 4, 16, 16, 0.35, 50), moe(3, 3, 2, 24, 1.2, (2, 1))),
])
# Sizes the tensor-core kernels take: head sizes 64 and 128 with equal value heads, widths that are multiples of 8.
WIDE = model(1032, 256, 2, 1e-6, [
    layer(att(8, 2, 64, 64, 0.15, 48, (32, 10000.0)), moe(16, 4, 4, 64, 1.5, (5, 3))),
    layer(gla(4, 64, 64, 8.0, 16), moe(8, 0, 2, 128, 1.0, (2, 1))),
    layer(par((8, 2, 64, 0.14, 100), (8, 4, 64, 32, 4, 16, 24), 1.2, 0.9), moe(6, 2, 3, 96, 2.5, (4, 3))),
    layer(att(4, 1, 128, 128, 0.1, 208, (128, 50000.0)), None),
    layer(par((4, 1, 128, 0.09, 70), (4, 4, 128, 64, 2, 8, 8), 0.8, 1.0), moe(4, 4, 2, 64, 1.0, (4, 2))),
    layer(gla(2, 128, 128, 4.0, 8), moe(16, 0, 4, 64, 1.0)),
])
# One copy of the stream (the hyper-connection is then a scaled residual sum), a width that is no multiple of 8, windows of
# one position and longer than any request, one tap (no convolution state), one key/value head, one head, a router that
# chooses every output, groups of one.
THIN = model(97, 44, 1, 1e-4, [
    layer(par((2, 1, 20, 0.4, 1), (2, 1, 12, 8, 1, 3, 2), 1.0, 1.0), moe(2, 1, 3, 16, 1.0, (1, 1))),
    layer(gla(1, 12, 20, 1.0, 2), None),
    layer(att(2, 1, 20, 12, 0.5, 200, (20, 77.0)), moe(3, 0, 2, 24, 3.0, (3, 2))),
])
CONFIGS = {"odd": ODD, "wide": WIDE, "thin": THIN}
BLOCKS = {"odd": 8, "wide": 16, "thin": 4}


def make_folder(cfg_dict, folder, seed, dtype=torch.float32, edit=None, sharp=3.0):
    """A model folder with random weights in which every mechanism matters: values that leave the linear part of tanh,
    attention far from uniform, sinks of both signs, routers that decide clearly with corrections that change choices,
    decays spread over (0, 1), copies of the stream that really mix.  Stored in bfloat16 the weights are smaller, so that
    the rounding of large intermediate values does not swamp the comparison."""
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors, write_safetensors, weights_path
    cfg = config_from_dict(cfg_dict)
    cfg.save(folder)
    soft = dtype == torch.bfloat16
    tensors = random_tensors(build_model_specs(cfg), seed, torch.float32, std=0.05 if soft else 0.09)
    g = torch.Generator().manual_seed(seed)
    uni = lambda shape, a, b: torch.empty(shape).uniform_(a, b, generator=g)
    for name in tensors:
        t = tensors[name]
        if t.dim() == 2 and name != "embed" and not name.endswith(".conv") and ".hc" not in name:
            # the same gain whatever the input's width: that of 72 inputs
            t = tensors[name] = t * min(1.0, (72.0 / t.shape[1]) ** 0.5)
        if name == "embed":
            tensors[name] = t * (8 if soft else 10)
        elif name.endswith(".alpha"):
            tensors[name] = uni((), 0.4, 1.6)
        elif name.endswith((".ls1", ".ls2")):
            tensors[name] = uni(t.shape, 0.3, 1.2)
        elif name.endswith((".in", ".out")) and ".hc" in name:
            tensors[name] = uni(t.shape, 0.4, 1.1)
        elif name.endswith(".mix") and ".hc" in name:
            tensors[name] = torch.eye(t.shape[0]) * 0.8 + uni(t.shape, -0.25, 0.25)
        elif name.endswith(".router"):
            tensors[name] = t * 6
        elif name.endswith(".correction"):
            tensors[name] = uni(t.shape, -0.15, 0.15)
        elif name.endswith(".sink"):
            tensors[name] = uni(t.shape, -2.0, 2.0)
        elif name.endswith(".norm") and ".mix" in name:
            tensors[name] = uni(t.shape, 0.5, 1.6)
        elif name.endswith(".conv"):
            tensors[name] = uni(t.shape, -1.0, 1.0)
        elif name.endswith((".A_log", ".dt_bias", ".a2.b")):
            tensors[name] = uni(t.shape, -1.5, 1.5)
        elif name.endswith((".a2", ".g2", ".mix.right.b")):
            tensors[name] = t * 8
        elif name.endswith((".q", ".k")) and ".right" not in name:
            tensors[name] = t * sharp
        elif name.endswith((".o", ".down")):
            tensors[name] = t * 2
    if edit:
        edit(tensors)
    # what is stored is what both sides read: round once to the storage type
    write_safetensors(weights_path(folder), {k: v.to(dtype) for k, v in tensors.items()})
    return folder


_PLAIN = {}


def plain_logits(folder, ids):
    key = (folder, tuple(ids))
    if key not in _PLAIN:
        cfg, W = plain.read_folder(folder)
        _PLAIN[key] = torch.from_numpy(plain.forward(cfg, W, list(ids)))
    return _PLAIN[key]


def requests(vocab, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return {f"r{i}": torch.randint(0, vocab, (n,), generator=g).tolist() for i, n in enumerate(lengths)}
