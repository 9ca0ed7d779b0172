"""Typed configuration of the Ledinex decoder, read from its own ``config.json`` keys.

    {"architecture": "Ledinex", "vocab": V, "width": H, "norm": {"eps": e}, "embedding": {"scale": s},
     "logit_scale": c, "canon": {"taps": n},
     "layers": [{"type": "parallel" | "parallel_2" | "delta", "mixer": {...},
                 "mlp": {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "top": k},
                         "shared": {"ff": Fs}} | null}, ...]}

Mixer keys.  ``parallel`` and ``parallel_2``: ``left`` (attention: ``heads, kv_heads, dim, vdim, scale``,
``softcap``, ``mask.size``, ``rot.{base, dims, scaling}`` with ``scaling.factor`` alone or with
``original, fast, slow``), ``right`` (``heads, dim``, and for ``parallel`` ``vdim`` and ``decay``, one per head),
``left_scale``, ``right_scale``.  ``delta``: ``heads, kv_heads, dim, vdim, conv``.  What a file may leave out:
``embedding.scale`` (1), ``logit_scale`` (1), ``canon`` (no convolution and no ``canon*`` tensors), ``kv_heads`` (``heads``),
``vdim`` (``dim``), ``scale`` (``dim^-1/2``), ``softcap`` (none), ``mask`` (causal), ``rot`` (no rotation),
``rot.dims`` (``dim``), ``rot.scaling`` (plain frequencies), the two scales (1), ``shared`` (no shared expert).
The low rank of a ``parallel_2`` layer's decay is not in config.json: it is the first extent of the tensor
``l<i>.mix.right.w1`` (``with_tensor_shapes``); a configuration that is to be written with random weights
names it as ``mixer.right.decay_rank``.
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .model_config import ConfigError, ModelConfig, _require, architecture_name
from .notirax_config import _obj, _opt, _positive, _req

LAYER_TYPES = ("parallel", "parallel_2", "delta")


def _finite(v: float, name: str) -> float:
    if not math.isfinite(v):
        raise ConfigError(f"config.json: field '{name}' must be finite")
    return v


def _parse_rot(m: Dict[str, Any], dim: int, where: str):
    rot = _obj(m, "rot", where, required=False)
    if not rot:
        return None
    out = {"base": _opt(rot, "base", float, 10000.0, where + "rot."),
           "dims": _opt(rot, "dims", int, dim, where + "rot."), "scaling": None}
    if not (out["base"] > 1 and math.isfinite(out["base"])):
        raise ConfigError(f"config.json: field '{where}rot.base' must be above 1, got {out['base']}")
    if out["dims"] < 0 or out["dims"] % 2 or out["dims"] > dim:
        raise ConfigError(f"config.json: field '{where}rot.dims' must be even and between 0 and {dim}, got {out['dims']}")
    sc = _obj(rot, "scaling", where + "rot.", required=False)
    if sc:
        w = where + "rot.scaling."
        s = {"factor": _positive(_req(sc, "factor", float, w), w + "factor")}
        if any(k in sc for k in ("original", "fast", "slow")):
            for k in ("original", "fast", "slow"):
                s[k] = _positive(_req(sc, k, float, w), w + k)
        out["scaling"] = s
    return out


def _parse_attention(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(_req(m, "heads", int, where), where + "heads"),
           "dim": _positive(_req(m, "dim", int, where), where + "dim")}
    out["kv_heads"] = _positive(_opt(m, "kv_heads", int, out["heads"], where), where + "kv_heads")
    out["vdim"] = _positive(_opt(m, "vdim", int, out["dim"], where), where + "vdim")
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of {where}kv_heads "
                          f"({out['kv_heads']})")
    out["scale"] = _finite(_opt(m, "scale", float, float(out["dim"]) ** -0.5, where), where + "scale")
    out["softcap"] = _opt(m, "softcap", float, 0.0, where)
    if out["softcap"] < 0 or not math.isfinite(out["softcap"]):
        raise ConfigError(f"config.json: field '{where}softcap' must not be negative, got {out['softcap']}")
    out["window"] = _opt(_obj(m, "mask", where, required=False), "size", int, 0, where + "mask.")
    if out["window"] < 0:
        raise ConfigError(f"config.json: field '{where}mask.size' must not be negative, got {out['window']}")
    out["rot"] = _parse_rot(m, out["dim"], where)
    return out


def _parse_side(kind: str, m: Dict[str, Any], where: str) -> Dict[str, Any]:
    left = _parse_attention(_obj(m, "left", where), where + "left.")
    r, w = _obj(m, "right", where), where + "right."
    right = {"heads": _positive(_req(r, "heads", int, w), w + "heads"),
             "dim": _positive(_req(r, "dim", int, w), w + "dim")}
    if kind == "parallel":
        right["vdim"] = _positive(_opt(r, "vdim", int, right["dim"], w), w + "vdim")
        decay = r.get("decay")
        if not isinstance(decay, list) or len(decay) != right["heads"] or not all(
                isinstance(d, (int, float)) and not isinstance(d, bool) and math.isfinite(d) for d in decay):
            raise ConfigError(f"config.json: field '{w}decay' must be a list of {right['heads']} numbers, one per head")
        right["decay"] = [float(d) for d in decay]
    else:
        if left["vdim"] != left["dim"]:
            raise ConfigError(f"config.json: {where}left: values that are the keys have the keys' size (vdim = dim)")
        right["decay_rank"] = _opt(r, "decay_rank", int, 0, w)
    return {"left": left, "right": right,
            "left_scale": _finite(_opt(m, "left_scale", float, 1.0, where), where + "left_scale"),
            "right_scale": _finite(_opt(m, "right_scale", float, 1.0, where), where + "right_scale")}


def _parse_delta(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(_req(m, "heads", int, where), where + "heads"),
           "dim": _positive(_req(m, "dim", int, where), where + "dim"),
           "conv": _positive(_req(m, "conv", int, where), where + "conv")}
    out["kv_heads"] = _positive(_opt(m, "kv_heads", int, out["heads"], where), where + "kv_heads")
    out["vdim"] = _positive(_opt(m, "vdim", int, out["dim"], where), where + "vdim")
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of {where}kv_heads "
                          f"({out['kv_heads']})")
    return out


def _parse_mlp(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    kind = _req(m, "kind", str, where)
    if kind != "moe":
        raise ConfigError(f"config.json: {where}kind '{kind}' is not supported (supported: moe)")
    expert, router = _obj(m, "expert", where), _obj(m, "router", where)
    out = {"kind": kind, "ff": _positive(_req(expert, "ff", int, where + "expert."), where + "expert.ff"),
           "experts": _positive(_req(router, "experts", int, where + "router."), where + "router.experts"),
           "top": _positive(_req(router, "top", int, where + "router."), where + "router.top"), "shared_ff": 0}
    if out["top"] > out["experts"]:
        raise ConfigError(f"config.json: {where}router: {out['experts']} experts cannot give a token {out['top']}")
    shared = _obj(m, "shared", where, required=False)
    if shared:
        out["shared_ff"] = _positive(_req(shared, "ff", int, where + "shared."), where + "shared.ff")
    return out


@dataclass(frozen=True)
class LedinexConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    taps: int = 0          # 0: the file has no ``canon``: sublayers read the stream as it is
    # per layer: {"type", "mixer": {...}, "mlp": {...} | None}, parsed and checked
    layers: Tuple[Dict[str, Any], ...] = field(default=(), compare=False)

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "LedinexConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json: top level must be an object")
        arch = architecture_name(j)
        vocab = _positive(_require(j, "vocab", int), "vocab")
        width = _positive(_require(j, "width", int), "width")
        eps = _req(_obj(j, "norm", ""), "eps", float, "norm.")
        if not (eps >= 0.0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: field 'norm.eps' must be non-negative, got {eps}")
        scale = _finite(_opt(_obj(j, "embedding", "", required=False), "scale", float, 1.0, "embedding."),
                        "embedding.scale")
        logit_scale = _finite(_opt(j, "logit_scale", float, 1.0, ""), "logit_scale")
        canon = _obj(j, "canon", "", required=False)
        taps = _positive(_req(canon, "taps", int, "canon."), "canon.taps") if canon else 0
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: missing required field 'layers' (a list of layers)")
        layers = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: field 'layers[{i}]' has wrong type: expected object")
            kind = _req(layer, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not supported (supported: "
                                  f"{', '.join(LAYER_TYPES)})")
            m = _obj(layer, "mixer", where)
            mixer = _parse_delta(m, where + "mixer.") if kind == "delta" else _parse_side(kind, m, where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: field '{where}mlp' has wrong type: expected object or null")
            layers.append({"type": kind, "mixer": mixer,
                           "mlp": None if mlp is None else _parse_mlp(mlp, where + "mlp.")})
        return cls(architecture=arch, raw=dict(j), vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   logit_scale=logit_scale, taps=taps, layers=tuple(layers))

    def with_tensor_shapes(self, shapes: Dict[str, tuple]) -> "LedinexConfig":
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            name = f"l{i}.mix.right.w1"
            if layer["type"] == "parallel_2" and name in shapes and len(shapes[name]) == 2:
                layer["mixer"]["right"]["decay_rank"] = int(shapes[name][0])
        return LedinexConfig(architecture=self.architecture, raw=self.raw, vocab=self.vocab, width=self.width,
                             norm_eps=self.norm_eps, embedding_scale=self.embedding_scale,
                             logit_scale=self.logit_scale, taps=self.taps, layers=tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                               "logit_scale": self.logit_scale, "layers": []}
        if self.taps:
            out["canon"] = {"taps": self.taps}
        for layer in self.layers:
            m = layer["mixer"]
            if layer["type"] == "delta":
                mixer: Dict[str, Any] = {k: m[k] for k in ("heads", "kv_heads", "dim", "vdim", "conv")}
            else:
                a = m["left"]
                left: Dict[str, Any] = {k: a[k] for k in ("heads", "kv_heads", "dim", "vdim", "scale")}
                if a["softcap"]:
                    left["softcap"] = a["softcap"]
                if a["window"]:
                    left["mask"] = {"size": a["window"]}
                if a["rot"]:
                    left["rot"] = {"base": a["rot"]["base"], "dims": a["rot"]["dims"]}
                    if a["rot"]["scaling"]:
                        left["rot"]["scaling"] = dict(a["rot"]["scaling"])
                mixer = {"left": left, "right": dict(m["right"]), "left_scale": m["left_scale"],
                         "right_scale": m["right_scale"]}
            mlp = layer["mlp"]
            j = None
            if mlp is not None:
                j = {"kind": "moe", "expert": {"ff": mlp["ff"]}, "router": {"experts": mlp["experts"], "top": mlp["top"]}}
                if mlp["shared_ff"]:
                    j["shared"] = {"ff": mlp["shared_ff"]}
            out["layers"].append({"type": layer["type"], "mixer": mixer, "mlp": j})
        return out
