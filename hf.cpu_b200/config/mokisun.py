"""Mokisun: a pre-norm decoder over a residual stream kept in several copies, with three kinds of mixer.

Top-level keys: ``architecture`` ("Mokisun"), ``vocab``, ``width``, ``streams`` (copies of the stream, mixed by
hyper-connections), ``norm`` ({``eps``}) and ``layers``.  A layer entry has ``type`` (the kind of mixer), ``mixer`` (its
sizes) and ``mlp`` (its feed-forward, or null for none):

* mixer "attention": ``heads``, ``kv_heads`` (default: ``heads``), ``dim``, ``vdim`` (default: ``dim``), ``scale`` (factor
  on the scores), ``mask`` ({``size``}: a sliding window), optionally ``rot`` ({``dims``, ``base``}: rotation of the first
  ``dims`` dimensions of each query and key head, pairs (2i, 2i + 1)).  No biases.  A learned sink per head joins the
  softmax's denominator.
* mixer "gla" (gated linear attention): ``heads``, ``dim``, ``vdim``, ``tau``.
* mixer "parallel": ``left``, ``right`` and their factors ``left_scale``, ``right_scale``.  ``left`` is attention whose
  values are its keys, without rotation, with a bias linear in the distance (slope ``2^(-8 (h + 1) / H)`` for head h) and a
  sink of score zero: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (= ``dim``), ``scale``, ``mask``.  ``right`` is a gated
  delta rule: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``conv`` (taps of the short convolution).
* mlp ``kind`` "moe": ``expert`` ({``ff``}) and ``router`` ({``experts``, ``top``, ``identity``, ``scale``, ``groups``:
  {``count``, ``keep``}}); gated experts with silu.

The inner sizes of the low-rank products (the decays' and the gate's) are those of the stored tensors; the optional mixer
keys ``a_rank`` and ``g_rank`` give them where a model is made at random.  Every norm of the stream is a Dynamic Tanh.
Tensor names: ``embed``, ``l<i>.norm1`` / ``norm2`` (with ``.b`` and ``.alpha``), ``l<i>.ls1`` / ``ls2``, ``l<i>.hc1.{in,mix,out}``
/ ``hc2``, ``l<i>.mix.*``, ``l<i>.mlp.{router,correction,e<j>.{gate,up,down}}``, ``final.norm``, ``head``.

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
DISTANCE_SLOPE_EXP = 8.0        # slope of head h of H: 2^(-8 (h + 1) / H)
UNIT_EPS = 1e-6                 # inside the root of the delta rule's unit-length queries and keys


def _attention_sizes(m: Dict[str, Any], w: str, rot_allowed: bool) -> None:
    H = take_int(m, "heads", lo=1)
    G = take_int(m, "kv_heads", default=H, lo=1)
    if H % G:
        raise UnsupportedError(f"config.json: {w}unsupported attention geometry: {H} heads over {G} key/value heads")
    d = take_int(m, "dim", lo=1)
    take_int(m, "vdim", default=d, lo=1)
    take_float(m, "scale")
    mask = _obj(m, "mask", w, required=False)
    if mask is not None:
        take_int(mask, "size", lo=1)
    rot = _obj(m, "rot", w, required=False)
    if rot is not None:
        if not rot_allowed:
            raise UnsupportedError(f"config.json: {w}this mixer has no rotation")
        dims = take_int(rot, "dims", lo=0, hi=d)
        if dims % 2:
            raise UnsupportedError(f"config.json: {w}rot.dims {dims} must be even")
        take_float(rot, "base", lo=0.0)


def _check_mixer(kind: str, m: Dict[str, Any], w: str) -> None:
    if kind == "attention":
        _attention_sizes(m, w, True)
    elif kind == "gla":
        take_int(m, "heads", lo=1), take_int(m, "dim", lo=1), take_int(m, "vdim", lo=1)
        take_float(m, "tau", lo=0.0)
    elif kind == "parallel":
        left, right = _obj(m, "left", w), _obj(m, "right", w)
        _attention_sizes(left, w + "left: ", False)
        if take_int(left, "vdim", default=left["dim"]) != left["dim"]:
            raise UnsupportedError(f"config.json: {w}left: the values are the keys, so vdim must equal dim")
        H = take_int(right, "heads", lo=1)
        G = take_int(right, "kv_heads", default=H, lo=1)
        if H % G:
            raise UnsupportedError(f"config.json: {w}right: {H} heads over {G} query/key heads")
        take_int(right, "dim", lo=1), take_int(right, "vdim", lo=1), take_int(right, "conv", lo=1)
        take_float(m, "left_scale", 1.0), take_float(m, "right_scale", 1.0)
    else:
        raise UnsupportedError(f"config.json: {w}mixer type '{kind}' is not supported (known: attention, gla, parallel)")


def _check_mlp(mlp: Dict[str, Any], w: str) -> None:
    if mlp.get("kind") != "moe":
        raise UnsupportedError(f"config.json: {w}mlp kind '{mlp.get('kind')}' is not supported (known: moe)")
    take_int(_obj(mlp, "expert", w), "ff", lo=1)
    r = _obj(mlp, "router", w)
    n = take_int(r, "experts", lo=0) + take_int(r, "identity", default=0, lo=0)
    top = take_int(r, "top", lo=1)
    if top > n:
        raise ConfigError(f"config.json: {w}router.top {top} exceeds the {n} router outputs")
    take_float(r, "scale", 1.0)
    g = _obj(r, "groups", w, required=False)
    if g is not None:
        count, keep = take_int(g, "count", lo=1), take_int(g, "keep", lo=1)
        if n % count or keep > count or keep * (n // count) < top:
            raise ConfigError(f"config.json: {w}router.groups: {count} groups of which {keep} are kept do not fit {n} router "
                              f"outputs with top {top}")


@dataclass
class MokisunConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    streams: int = 1
    norm_eps: float = 1e-6
    max_positions: int = DEFAULT_MAX_POSITIONS
    layers: List[Dict[str, Any]] = field(default_factory=list)
    eos_token_id: List[int] = field(default_factory=list)

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "MokisunConfig":
        V = take_int(d, "vocab", lo=1)
        E = take_int(d, "width", lo=1, hi=1_000_000)
        norm = _obj(d, "norm", "", required=False) or {}
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        out = []
        for i, L in enumerate(layers):
            w = f"layers[{i}]: "
            if not isinstance(L, dict):
                raise ConfigError(f"config.json: {w}must be an object")
            _check_mixer(L.get("type"), _obj(L, "mixer", w), w)
            mlp = _obj(L, "mlp", w, required=False)
            if mlp is not None:
                _check_mlp(mlp, w)
            out.append(copy.deepcopy(L))
        eos = d.get("eos_token_id", [])
        eos = [] if eos is None else ([eos] if isinstance(eos, int) else list(eos))
        return cls(vocab=V, width=E, streams=take_int(d, "streams", default=1, lo=1, hi=8),
                   norm_eps=take_float(norm, "eps", 1e-6, lo=0.0),
                   max_positions=take_int(d, "max_positions", default=DEFAULT_MAX_POSITIONS, lo=1), layers=out, eos_token_id=eos)

    def to_dict(self) -> Dict[str, Any]:
        d = {"architecture": self.architecture or "Mokisun", "vocab": self.vocab, "width": self.width, "streams": self.streams,
             "norm": {"eps": self.norm_eps}, "layers": copy.deepcopy(self.layers)}
        if self.max_positions != DEFAULT_MAX_POSITIONS:
            d["max_positions"] = self.max_positions
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d

    # ---- the plan ---------------------------------------------------------------------------------------
    def _attention(self, m, prefix, positions, *, sink, values_are_keys=False, slope_exp=None) -> PartSpec:
        pos_name = None
        rot = m.get("rot")
        if rot and rot.get("dims"):
            pos_name = f"rot{m['dim']}_{rot['dims']}_{float(rot['base'])!r}"        # layers with the same rotation share one table
            positions.setdefault(pos_name, PartSpec("rotary", {
                "head_dim": m["dim"], "n_rot": rot["dims"], "theta": float(rot["base"]), "pairing": "interleaved"}))
        return PartSpec("paged_attention", {
            "hidden_size": self.width, "num_heads": m["heads"], "num_kv_heads": m.get("kv_heads", m["heads"]), "head_dim": m["dim"],
            "v_head_dim": m.get("vdim", m["dim"]), "scale": float(m["scale"]), "qkv_bias": False, "out_bias": False,
            "window": (m.get("mask") or {}).get("size", 0), "position": pos_name, "prefix": prefix,
            "names": {"q": "q", "k": "k", "v": "v", "o": "o"}, "weight_suffix": "", "bias_suffix": ".b", "sink": sink,
            "sink_tensor": "sink", "values_are_keys": values_are_keys, "distance_slope_exp": slope_exp})

    def _mixer(self, L, prefix, positions) -> PartSpec:
        m, kind = L["mixer"], L["type"]
        if kind == "attention":
            return self._attention(m, prefix, positions, sink="learned")
        if kind == "gla":
            return PartSpec("gated_linear_attention", {
                "hidden_size": self.width, "num_heads": m["heads"], "head_dim": m["dim"], "v_head_dim": m["vdim"],
                "tau": float(m["tau"]), "norm_eps": self.norm_eps, "decay_rank": m.get("a_rank", -1), "prefix": prefix})
        left, right = m["left"], m["right"]
        return PartSpec("parallel", {"branches": [
            (self._attention(left, prefix + ".left", positions, sink="zero", values_are_keys=True, slope_exp=DISTANCE_SLOPE_EXP),
             float(m.get("left_scale", 1.0))),
            (PartSpec("gated_delta_rule", {
                "hidden_size": self.width, "num_heads": right["heads"], "num_kv_heads": right.get("kv_heads", right["heads"]),
                "head_dim": right["dim"], "v_head_dim": right["vdim"], "conv_taps": right["conv"], "norm_eps": self.norm_eps,
                "unit_eps": UNIT_EPS, "decay_rank": right.get("a_rank", -1), "gate_rank": right.get("g_rank", -1),
                "prefix": prefix + ".right"}), float(m.get("right_scale", 1.0)))]})

    def plan(self) -> ModelPlan:
        E = self.width
        norm = lambda name: PartSpec("dynamic_tanh", {"size": E, "tensor": name, "bias_suffix": ".b", "alpha_suffix": ".alpha"})
        positions: Dict[str, PartSpec] = {}
        layers, schedule = [], []
        for i, L in enumerate(self.layers):
            p, mlp = f"l{i}", L.get("mlp")
            ffn = None
            if mlp is not None:
                r = mlp["router"]
                g = r.get("groups")
                ffn = PartSpec("moe", {
                    "hidden_size": E, "experts": r["experts"], "top": r["top"], "expert_size": mlp["expert"]["ff"], "prefix": f"{p}.mlp",
                    "activation": "silu", "gated": True, "router_bias": False, "router": "softmax_all", "correction": "correction",
                    "groups": (g["count"], g["keep"]) if g else None, "identity": r.get("identity", 0),
                    "route_scale": float(r.get("scale", 1.0)), "names": {"router": "router", "expert": "e{}", "gate": "gate", "up": "up", "down": "down"}})
            layers.append(LayerSpec(
                prefix=p, block=PartSpec("hyper_residual", {"streams": self.streams, "hidden_size": E, "prefix": p, "layer_scale": True,
                                                            "has_ffn": ffn is not None}),
                norm1=norm(f"{p}.norm1"), mixer=self._mixer(L, f"{p}.mix", positions),
                norm2=norm(f"{p}.norm2") if ffn is not None else None, ffn=ffn))
            schedule.append(ScheduleEntry(i))
        plan = ModelPlan(
            hidden_size=E, vocab_size=self.vocab, max_positions=self.max_positions,
            embedding=PartSpec("embedding", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "embed"}),
            positions=positions, layers=layers, schedule=schedule, final_norm=norm("final.norm"),
            head=PartSpec("linear_head", {"vocab_size": self.vocab, "hidden_size": E, "tensor": "head"}),
            eos_token_ids=list(self.eos_token_id), streams=self.streams)
        plan.validate()
        return plan


register_architecture("Mokisun", MokisunConfig)
register_architecture("mokisun", MokisunConfig)
