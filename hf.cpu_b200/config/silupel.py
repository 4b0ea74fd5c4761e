"""Silupel: a pre-norm decoder whose config.json lists its layers one by one, with three kinds of mixer, a token shift in
front of every mixer, and a stretch of layers that runs several times.

Top-level keys: ``architecture`` ("Silupel"), ``vocab``, ``width``, ``norm`` ({``eps``}), ``layers`` and optionally ``loop``
({``start``, ``stop``, ``times``}: layers start .. stop - 1 run ``times`` times in a row with the same weights, each run with a
cache or state of its own, then the rest follow).  A layer entry has ``type`` (the kind of mixer), ``mixer`` (its sizes)
and ``mlp`` (its feed-forward, or null for none):

* mixer "mingru": ``width``.  A gated recurrence per channel (see ``parts/recurrent.py``).
* mixer "attention": ``heads``, ``kv_heads`` (default: ``heads``), ``dim`` (query/key head), ``vdim`` (value head; default:
  ``dim``), ``scale`` (factor on the scores), ``softcap`` (scores pass through ``c tanh(s / c)``; absent: no cap), ``mask``
  ({``size``}: chunks of that many positions; a query sees the earlier keys of its own chunk; absent: causal), ``rot``
  ({``dims``, ``base``, optionally ``scaling``: {``factor``, ``low``, ``high``, ``original``}}: rotation of the first ``dims``
  dimensions of each head, dimension i with i + dims/2, frequencies stretched by wavelength).  Biases on q, k, v and o, a
  stored factor per head on the scores, and a sigmoid gate on the heads' outputs.
* mixer "latent_attention": ``heads``, ``dim`` (plain) and ``rot_dim`` (rotated) dimensions per query/key head, ``vdim``,
  ``q_rank`` and ``kv_rank`` (the latents), ``scale``, ``rot`` ({``dims`` = ``rot_dim``, ``base``}); causal.
* mlp ``kind`` "dense": ``ff``; ``down(gelu_tanh(gate x) * (up x))``.

Every norm of the stream is a layer norm with a weight and no bias.  Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2`` /
``shift``, ``l<i>.mix.{z,x,g,o}`` with ``z.b`` / ``x.b``, or ``l<i>.mix.{q,k,v,g,o}`` with ``q.b`` / ``k.b`` / ``v.b`` / ``o.b`` and
``temp``, or ``l<i>.mix.{dq,uq,dkv,uk,uv,o}`` with ``dq.norm`` / ``dkv.norm``, ``l<i>.mlp.{gate,up,down}``, ``final.norm``, ``head``.

config.json gives no context length: ``max_positions`` (optional key, default below) bounds the rotary tables and a
request's length in this engine.
"""
from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any, Dict, List

from .base import (ConfigError, LayerSpec, ModelConfig, ModelPlan, PartSpec, ScheduleEntry, UnsupportedError,
                   take_float, take_int)
from .manapel import _obj
from .registry import register_architecture

DEFAULT_MAX_POSITIONS = 1 << 16
SCALING_KEYS = ("factor", "low", "high", "original")


def _check_rot(m: Dict[str, Any], w: str, width: int, scaling_allowed: bool) -> None:
    rot = _obj(m, "rot", w)
    dims = take_int(rot, "dims", lo=2)
    if dims % 2 or dims > width:
        raise UnsupportedError(f"config.json: {w}rot.dims {dims} must be even and at most {width}")
    take_float(rot, "base", lo=0.0)
    sc = _obj(rot, "scaling", w, required=False)
    if sc is not None:
        if not scaling_allowed:
            raise UnsupportedError(f"config.json: {w}this mixer's rotation is not scaled")
        for k in SCALING_KEYS:
            take_float(sc, k, lo=0.0)
        if not sc["high"] > sc["low"]:
            raise ConfigError(f"config.json: {w}rot.scaling: 'high' must exceed 'low'")


@dataclass
class SilupelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 1e-6
    max_positions: int = DEFAULT_MAX_POSITIONS
    layers: List[Dict[str, Any]] = field(default_factory=list)
    loop: Dict[str, int] = field(default_factory=dict)          # start, stop, times; empty: every layer runs once
    eos_token_id: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "SilupelConfig":
        V = take_int(d, "vocab", lo=1)
        E = take_int(d, "width", lo=1, hi=1_000_000)
        norm = _obj(d, "norm", "")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, L in enumerate(layers):
            w = f"layers[{i}]: "
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: {w}must be an object")
            kind = L.get("type")
            m = _obj(L, "mixer", w)
            if kind == "mingru":
                take_int(m, "width", lo=1)
            elif kind == "attention":
                H = take_int(m, "heads", lo=1)
                G = take_int(m, "kv_heads", default=H, lo=1)
                if H % G:
                    raise UnsupportedError(f"config.json: {w}unsupported attention geometry: {H} heads over {G} key/value heads")
                dim = take_int(m, "dim", lo=1)
                take_int(m, "vdim", default=dim, lo=1)
                take_float(m, "scale")
                take_float(m, "softcap", default=0.0)
                mask = _obj(m, "mask", w, required=False)
                if mask is not None:
                    take_int(mask, "size", lo=1)
                if m.get("rot") is not None:
                    _check_rot(m, w, dim, True)
            elif kind == "latent_attention":
                take_int(m, "heads", lo=1), take_int(m, "dim", lo=1), take_int(m, "vdim", lo=1)
                take_int(m, "q_rank", lo=1), take_int(m, "kv_rank", lo=1)
                take_float(m, "scale")
                rd = take_int(m, "rot_dim", lo=0)
                if rd % 2:
                    raise UnsupportedError(f"config.json: {w}rot_dim {rd} must be even")
                if rd:
                    _check_rot(m, w, rd, False)
                    if m["rot"]["dims"] != rd:
                        raise UnsupportedError(f"config.json: {w}rot.dims must equal rot_dim (the rotated part is rotated whole)")
            else:
                raise UnsupportedError(f"config.json: {w}mixer type '{kind}' is not supported "
                                       f"(known: attention, latent_attention, mingru)")
            mlp = _obj(L, "mlp", w, required=False)
            if mlp is not None:
                if mlp.get("kind") != "dense":
                    raise UnsupportedError(f"config.json: {w}mlp kind '{mlp.get('kind')}' is not supported (known: dense)")
                take_int(mlp, "ff", lo=1)
            out.append(copy.deepcopy(L))
        loop = _obj(d, "loop", "", required=False)
        lp: Dict[str, int] = {}
        if loop is not None:
            lp = {"start": take_int(loop, "start", lo=0), "stop": take_int(loop, "stop", lo=0), "times": take_int(loop, "times", lo=0)}
            if not lp["start"] <= lp["stop"] <= len(out):
                raise ConfigError(f"config.json: loop: layers {lp['start']} .. {lp['stop']} are not a stretch of the {len(out)} layers")
        eos = d.get("eos_token_id", [])
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        return cls(vocab=V, width=E, norm_eps=take_float(norm, "eps", 1e-6, lo=0.0),
                   max_positions=take_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, lo=1), layers=out, loop=lp,
                   eos_token_id=eos)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture or "Silupel", "vocab": self.vocab, "width": self.width,
             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.loop:
            d["loop"] = dict(self.loop)
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    def run_order(self) -> List[int]:
        """Layer indices in the order they run."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    def plan(self) -> ModelPlan:
        E = self.width
        norm = lambda name, optional=False: PartSpec("layernorm", {"size": E, "eps": self.norm_eps, "tensor": name,
                                                                   "optional": optional})
        positions: Dict[str, PartSpec] = {}

        def rotary(rot, head_dim):
            # layers with the same rotation share one table
            sc = rot.get("scaling")
            name = f"rot{rot['dims']}_{float(rot['base'])!r}_{sorted(sc.items()) if sc else None!r}"
            positions.setdefault(name, PartSpec("rotary", {
                "head_dim": head_dim, "n_rot": rot["dims"], "theta": float(rot["base"]), "pairing": "half",
                "scaling": {k: float(sc[k]) for k in SCALING_KEYS} if sc else None}))
            return name

        layers = []
        for i, L in enumerate(self.layers):
            p, m, mlp = f"l{i}", L["mixer"], L.get("mlp")
            if L["type"] == "mingru":
                mixer = PartSpec("mingru", {"hidden_size": E, "width": m["width"], "prefix": f"{p}.mix"})
            elif L["type"] == "attention":
                rot = m.get("rot")
                mixer = PartSpec("paged_attention", {
                    "hidden_size": E, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
                    "v_head_dim": m.get("vdim", m["dim"]), "scale": float(m["scale"]), "qkv_bias": True, "out_bias": True,
                    "window": 0, "chunk": (m.get("mask") or {}).get("size", 0), "softcap": float(m.get("softcap") or 0.0),
                    "head_scale_tensor": "temp", "out_gate": {"tensor": "g", "kind": "sigmoid"},
                    "position": rotary(rot, m["dim"]) if rot else None, "prefix": f"{p}.mix",
                    "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "bias_suffix": ".b"})
            else:
                mixer = PartSpec("latent_attention", {
                    "hidden_size": E, "num_heads": m["heads"], "head_dim": m["dim"], "rot_dim": m["rot_dim"],
                    "v_head_dim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                    "norm_eps": self.norm_eps, "window": 0,
                    "position": rotary(m["rot"], m["rot_dim"]) if m["rot_dim"] else None, "prefix": f"{p}.mix"})
            ffn = None
            if mlp is not None:
                ffn = PartSpec("gated", {"hidden_size": E, "intermediate_size": mlp["ff"], "prefix": f"{p}.mlp",
                                         "activation": "gelu_tanh", "names": {"gate": "gate", "up": "up", "down": "down"}})
            block = PartSpec("prenorm_residual", {"token_shift": f"{p}.shift", "hidden_size": E})
            layers.append(LayerSpec(prefix=p, block=block, norm1=norm(f"{p}.norm1"), mixer=mixer,
                                    norm2=norm(f"{p}.norm2", optional=ffn is None), ffn=ffn))
        plan = ModelPlan(
            hidden_size=E, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "embed"}),
            positions=positions, layers=layers, schedule=[ScheduleEntry(i) for i in self.run_order()],
            final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "head"}),
            eos_token_ids=list(self.eos_token_id))
        plan.validate()
        return plan


register_architecture("Silupel", SilupelConfig)
register_architecture("silupel", SilupelConfig)
