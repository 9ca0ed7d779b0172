"""Typed configuration of the Rabapel decoder, read from its own ``config.json`` keys.

    {"architecture": "Rabapel", "vocab": V, "width": H, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "latent_attention", "mixer": {...},
                 "mlp": {"kind": "dense", "ff": F}
                      | {"kind": "moe", "expert": {"ff": F}, "router": {"experts": E, "identity": I, "top": k},
                         "shared": {"ff": Fs}}
                      | null}, ...]}

Mixer keys: ``heads, dim, rot_dim, vdim, kv_rank, scale``, ``rot`` (``base``, ``dims``, ``scaling`` with
``factor, original, fast, slow``) and ``mask.size``.  What a file may leave out: ``embedding.scale`` (1),
``vdim`` (``dim``), ``scale`` (the inverse root of ``dim + rot_dim``), ``rot.dims`` (``rot_dim``),
``rot.scaling`` (the plain frequencies), ``mask`` (plain causal), ``router.identity`` (0), ``shared`` (no
shared expert).
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, Tuple

from .model_config import ConfigError, ModelConfig, _require, architecture_name
from .notirax_config import _obj, _opt, _positive, _req

MIXER_TYPES = ("latent_attention",)
MLP_KINDS = ("dense", "moe")


def _parse_scaling(rot: Dict[str, Any], where: str):
    sc = _obj(rot, "scaling", where, required=False)
    if not sc:
        return None
    out = {"factor": _req(sc, "factor", float, where + "scaling."),
           "original": _req(sc, "original", float, where + "scaling."),
           "fast": _req(sc, "fast", float, where + "scaling."),
           "slow": _req(sc, "slow", float, where + "scaling.")}
    for k, v in out.items():
        if not (v > 0 and math.isfinite(v)):
            raise ConfigError(f"config.json: field '{where}scaling.{k}' must be positive, got {v}")
    return out


def _parse_mixer(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    out = {"heads": _positive(_req(m, "heads", int, where), where + "heads"),
           "dim": _positive(_req(m, "dim", int, where), where + "dim"),
           "rot_dim": _req(m, "rot_dim", int, where),
           "kv_rank": _positive(_req(m, "kv_rank", int, where), where + "kv_rank")}
    out["vdim"] = _positive(_opt(m, "vdim", int, out["dim"], where), where + "vdim")
    if out["rot_dim"] < 0 or out["rot_dim"] % 2:
        raise ConfigError(f"config.json: field '{where}rot_dim' must be even and not negative, got {out['rot_dim']}")
    out["scale"] = _opt(m, "scale", float, float(out["dim"] + out["rot_dim"]) ** -0.5, where)
    if not math.isfinite(out["scale"]):
        raise ConfigError(f"config.json: field '{where}scale' must be finite")
    rot = _obj(m, "rot", where, required=out["rot_dim"] > 0)
    out["rot_base"] = _opt(rot, "base", float, 10000.0, where + "rot.")
    out["rot_dims"] = _opt(rot, "dims", int, out["rot_dim"], where + "rot.")
    if not (out["rot_base"] > 1 and math.isfinite(out["rot_base"])):
        raise ConfigError(f"config.json: field '{where}rot.base' must be above 1, got {out['rot_base']}")
    if out["rot_dims"] < 0 or out["rot_dims"] % 2 or out["rot_dims"] > out["rot_dim"]:
        raise ConfigError(f"config.json: field '{where}rot.dims' must be even and between 0 and {out['rot_dim']}, "
                          f"got {out['rot_dims']}")
    out["rot_scaling"] = _parse_scaling(rot, where + "rot.")
    mask = _obj(m, "mask", where, required=False)
    out["window"] = _opt(mask, "size", int, 0, where + "mask.")
    if out["window"] < 0:
        raise ConfigError(f"config.json: field '{where}mask.size' must not be negative, got {out['window']}")
    return out


def _parse_mlp(m: Dict[str, Any], where: str) -> Dict[str, Any]:
    kind = _req(m, "kind", str, where)
    if kind not in MLP_KINDS:
        raise ConfigError(f"config.json: {where}kind '{kind}' is not supported (supported: {', '.join(MLP_KINDS)})")
    if kind == "dense":
        return {"kind": kind, "ff": _positive(_req(m, "ff", int, where), where + "ff")}
    expert = _obj(m, "expert", where)
    router = _obj(m, "router", where)
    out = {"kind": kind,
           "ff": _positive(_req(expert, "ff", int, where + "expert."), where + "expert.ff"),
           "experts": _req(router, "experts", int, where + "router."),
           "identity": _opt(router, "identity", int, 0, where + "router."),
           "top": _positive(_req(router, "top", int, where + "router."), where + "router.top"),
           "shared_ff": 0}
    if out["experts"] < 0 or out["identity"] < 0 or out["experts"] + out["identity"] < out["top"]:
        raise ConfigError(f"config.json: {where}router: {out['experts']} experts and {out['identity']} identity "
                          f"experts cannot give a token {out['top']}")
    shared = _obj(m, "shared", where, required=False)
    if shared:
        out["shared_ff"] = _positive(_req(shared, "ff", int, where + "shared."), where + "shared.ff")
    return out


@dataclass(frozen=True)
class RabapelConfig(ModelConfig):
    vocab: int = 0
    width: int = 0
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    # per layer: {"type", "mixer": {...}, "mlp": {...} | None}, parsed and checked
    layers: Tuple[Dict[str, Any], ...] = field(default=(), compare=False)

    @classmethod
    def from_json(cls, j: Dict[str, Any]) -> "RabapelConfig":
        if not isinstance(j, dict):
            raise ConfigError("config.json: top level must be an object")
        arch = architecture_name(j)
        vocab = _positive(_require(j, "vocab", int), "vocab")
        width = _positive(_require(j, "width", int), "width")
        eps = _req(_obj(j, "norm", ""), "eps", float, "norm.")
        if not (eps >= 0.0 and math.isfinite(eps)):
            raise ConfigError(f"config.json: field 'norm.eps' must be non-negative, got {eps}")
        scale = _opt(_obj(j, "embedding", "", required=False), "scale", float, 1.0, "embedding.")
        if not math.isfinite(scale):
            raise ConfigError("config.json: field 'embedding.scale' must be finite")
        raw_layers = j.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: missing required field 'layers' (a list of layers)")
        layers = []
        for i, layer in enumerate(raw_layers):
            where = f"layers[{i}]."
            if not isinstance(layer, dict):
                raise ConfigError(f"config.json: field 'layers[{i}]' has wrong type: expected object")
            kind = _req(layer, "type", str, where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}type '{kind}' is not supported (supported: "
                                  f"{', '.join(MIXER_TYPES)})")
            mixer = _parse_mixer(_obj(layer, "mixer", where), where + "mixer.")
            mlp = layer.get("mlp")
            if mlp is not None and not isinstance(mlp, dict):
                raise ConfigError(f"config.json: field '{where}mlp' has wrong type: expected object or null")
            layers.append({"type": kind, "mixer": mixer,
                           "mlp": None if mlp is None else _parse_mlp(mlp, where + "mlp.")})
        return cls(architecture=arch, raw=dict(j), vocab=vocab, width=width, norm_eps=eps, embedding_scale=scale,
                   layers=tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        """The config.json this configuration would be read back from."""
        out: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                               "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale},
                               "layers": []}
        for layer in self.layers:
            m = layer["mixer"]
            rot: Dict[str, Any] = {"base": m["rot_base"], "dims": m["rot_dims"]}
            if m["rot_scaling"]:
                rot["scaling"] = dict(m["rot_scaling"])
            mixer: Dict[str, Any] = {"heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"], "vdim": m["vdim"],
                                     "kv_rank": m["kv_rank"], "scale": m["scale"], "rot": rot}
            if m["window"]:
                mixer["mask"] = {"size": m["window"]}
            mlp = layer["mlp"]
            if mlp is None:
                j = None
            elif mlp["kind"] == "dense":
                j = {"kind": "dense", "ff": mlp["ff"]}
            else:
                j = {"kind": "moe", "expert": {"ff": mlp["ff"]},
                     "router": {"experts": mlp["experts"], "identity": mlp["identity"], "top": mlp["top"]}}
                if mlp["shared_ff"]:
                    j["shared"] = {"ff": mlp["shared_ff"]}
            out["layers"].append({"type": layer["type"], "mixer": mixer, "mlp": j})
        return out
