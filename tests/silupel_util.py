"""Small Silupel configurations, model folders with random weights, and the plain implementation's logits."""
import numpy as np
import torch

import plain_silupel as plain


def gru(width):
    return {"type": "mingru", "mixer": {"width": width}}


def att(heads, kv_heads, dim, vdim, scale, chunk, rot_dims, base, softcap, scaling=None):
    rot = {"dims": rot_dims, "base": base}
    if scaling:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale,
                                           "softcap": softcap, "mask": {"size": chunk}, "rot": rot}}


def lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank,
                                                  "kv_rank": kv_rank, "scale": scale, "rot": {"dims": rot_dim, "base": base}}}


def layer(mixer, ff):
    return dict(mixer, mlp={"kind": "dense", "ff": ff} if ff else None)


def model(vocab, width, eps, layers, loop=None):
    d = {"architecture": "Silupel", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    return d


# Odd sizes throughout: fewer key/value heads than heads, value heads wider than key heads, a chunk shorter than a page
# and one longer than the prompts' portions, a layer without a feed-forward, a recurrence wider than the stream and one
# narrower, rotation of a part of the head and of all of it, one rotation stretched, three layers that run three times.
ODD = model(211, 72, 1e-5, [
    layer(gru(100), 100),
    layer(att(6, 3, 24, 40, 0.3, 12, 8, 500.0, 7.0, scaling=(8.0, 1.0, 4.0, 32)), 64),
    layer(lat(3, 16, 8, 24, 40, 24, 0.25, 300.0), None),
    layer(gru(40), 56),
    layer(att(4, 4, 16, 16, 0.35, 50, 16, 10000.0, 30.0), None),
    layer(lat(5, 8, 12, 20, 16, 36, 0.3, 3000.0), 56),
], loop=(1, 4, 3))
# Sizes the tensor-core kernels take: head sizes 64 and 128 with equal value heads, a latent row of 128 and one of 64,
# widths that are multiples of 8, twenty latent heads over the one cached row, the looped stretch at the very start.
WIDE = model(1032, 256, 1e-6, [
    layer(lat(4, 64, 32, 64, 128, 96, 0.12, 25000.0), 512),
    layer(att(8, 2, 64, 64, 0.15, 48, 32, 50000.0, 15.0, scaling=(4.0, 1.0, 4.0, 64)), 256),
    layer(gru(256), 256),
    layer(att(4, 1, 128, 128, 0.1, 208, 128, 10000.0, 50.0), 512),
    layer(lat(20, 32, 16, 48, 64, 48, 0.15, 10000.0), 256),
    layer(gru(384), None),
], loop=(0, 2, 2))
# A width that is no multiple of 8 (no tensor-core product takes it), one key/value head, a chunk of one position (a
# query sees itself only), a chunk longer than any request, no loop at all.
THIN = model(97, 44, 1e-4, [
    layer(att(2, 1, 20, 12, 0.4, 1, 2, 77.0, 3.0), 24),
    layer(gru(44), 20),
    layer(lat(2, 12, 4, 8, 10, 6, 0.5, 77.0), 20),
    layer(att(3, 3, 12, 20, 0.4, 500, 12, 77.0, 100.0, scaling=(2.0, 0.5, 2.0, 16)), None),
    layer(lat(1, 6, 2, 10, 12, 10, 0.5, 77.0), None),
])
CONFIGS = {"odd": ODD, "wide": WIDE, "thin": THIN}
BLOCKS = {"odd": 8, "wide": 16, "thin": 4}


def make_folder(cfg_dict, folder, seed, dtype=torch.float32, edit=None, sharp=None):
    """A model folder with random weights whose attention is far from uniform (query and key projections scaled up), whose
    norm weights, shifts, score factors and biases are well away from their neutral values, and whose recurrence's gates
    are spread over (0, 1).  Stored in bfloat16 the weights are smaller and the scores less sharp, so that the rounding of
    large intermediate values, amplified by eight and more layer runs, does not swamp the comparison."""
    from hfcpu_b200.config import config_from_dict
    from hfcpu_b200.models import build_model_specs
    from hfcpu_b200.weights import random_tensors, write_safetensors, weights_path
    cfg = config_from_dict(cfg_dict)
    cfg.save(folder)
    soft = dtype == torch.bfloat16
    if sharp is None:
        sharp = 1.5 if soft else 3.0
    tensors = random_tensors(build_model_specs(cfg), seed, torch.float32, std=0.05 if soft else 0.09)
    g = torch.Generator().manual_seed(seed)
    for name in tensors:
        t = tensors[name]
        if name == "embed":
            tensors[name] = t * (6 if soft else 8)
        elif name.endswith(".shift"):
            tensors[name] = torch.empty(t.shape).uniform_(-0.2, 1.1, generator=g)
        elif name.endswith(".temp"):
            tensors[name] = torch.empty(t.shape).uniform_(0.5, 1.8, generator=g) * (torch.arange(t.shape[0]) % 3 - 0.5).sign()
        elif name.endswith(("norm1", "norm2", "final.norm", ".norm")):
            tensors[name] = torch.empty(t.shape).uniform_(0.5, 1.6, generator=g)
        elif name.endswith(".b"):
            tensors[name] = torch.empty(t.shape).uniform_(-0.5, 0.5, generator=g)
        elif name.endswith((".mix.q", ".mix.k", ".mix.uq", ".mix.uk", ".mix.dkv", ".mix.z", ".mix.x")):
            tensors[name] = t * sharp
        elif ".mix.o" in name or name.endswith(".down"):
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
