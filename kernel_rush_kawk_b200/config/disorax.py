"""Configuration of the Disorax decoder, read from its own config.json keys.

    {"architecture": "Disorax", "vocab": V, "width": C, "norm": {"eps": e}, "residual_mult": m,
     "layers": [{"type": T, "mixer": {...}, "mlp": {...} | null}, ...]}

Mixer types and their keys:

* ``attention``: ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``, ``rot`` (``dims``, ``base``),
  ``mask`` (``size``, ``keep_first``), ``v_mix`` (bool).
* ``latent_attention``: ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``; causal.
* ``latent_attention_2``: the same with ``mask.size`` (a sliding window) and a sink in the softmax.

Feed-forward (``mlp``): ``kind`` "moe", ``expert.ff``, ``router.experts``, ``router.top``, and ``shared.ff``
(or no ``shared``). Every size and constant comes from the file.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from pathlib import Path

from .base import ConfigError, ModelConfig, positive, require
from .taredra import _int, _number, _section

PRESET_DIR = Path(__file__).parent / "presets" / "disorax"

MIXER_TYPES = ("attention", "latent_attention", "latent_attention_2")


def _read_mixer(kind: str, raw: dict, where: str) -> dict:
    out = {"heads": _int(raw, "heads", where), "dim": _int(raw, "dim", where), "vdim": _int(raw, "vdim", where),
           "scale": _number(raw, "scale", where)}
    if kind == "attention":
        out["kv_heads"] = _int(raw, "kv_heads", where)
        if out["heads"] % out["kv_heads"]:
            raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of kv_heads ({out['kv_heads']})")
        rot = _section(raw, "rot", where)
        out["rot"] = {"dims": _int(rot, "dims", where + "rot."), "base": _number(rot, "base", where + "rot.")}
        if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
            raise ConfigError(f"config.json: {where}rot.dims ({out['rot']['dims']}) must be even and at most dim ({out['dim']})")
        if not out["rot"]["base"] > 0:
            raise ConfigError(f"config.json: {where}rot.base must be positive")
        mask = _section(raw, "mask", where)
        keep = mask.get("keep_first", 0)
        if isinstance(keep, bool) or not isinstance(keep, int) or keep < 0:
            raise ConfigError(f"config.json: {where}mask.keep_first must be a non-negative integer, got {keep!r}")
        out["mask"] = {"size": _int(mask, "size", where + "mask."), "keep_first": keep}
        out["v_mix"] = bool(raw.get("v_mix", False))
    else:
        out["kv_rank"] = _int(raw, "kv_rank", where)
        if kind == "latent_attention_2" or raw.get("mask") is not None:
            out["mask"] = {"size": _int(_section(raw, "mask", where), "size", where + "mask.")}
    return out


def _read_mlp(raw, where: str):
    if raw is None:
        return None
    if not isinstance(raw, dict) or raw.get("kind") != "moe":
        raise ConfigError(f"config.json: {where}mlp must be null or of kind 'moe', got {raw!r}")
    router = _section(raw, "router", where + "mlp.")
    out = {"kind": "moe", "expert": {"ff": _int(_section(raw, "expert", where + "mlp."), "ff", where + "mlp.expert.")},
           "router": {"experts": _int(router, "experts", where + "mlp.router."), "top": _int(router, "top", where + "mlp.router.")}}
    if out["router"]["top"] > out["router"]["experts"]:
        raise ConfigError(f"config.json: {where}mlp.router.top exceeds the number of experts")
    if raw.get("shared") is not None:
        out["shared"] = {"ff": _int(_section(raw, "shared", where + "mlp."), "ff", where + "mlp.shared.")}
    return out


def _read_layer(raw: dict, i: int) -> dict:
    where = f"layers[{i}]."
    kind = raw.get("type")
    if kind not in MIXER_TYPES:
        raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design {MIXER_TYPES}")
    return {"type": kind, "mixer": _read_mixer(kind, _section(raw, "mixer", where), where + "mixer."),
            "mlp": _read_mlp(raw.get("mlp"), where)}


@dataclass(frozen=True)
class DisoraxConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    residual_mult: float
    #: one normalised dict per layer (type, mixer, mlp); treated as read-only
    layers: tuple = field(default_factory=tuple)

    architecture = "Disorax"

    @classmethod
    def from_dict(cls, raw: dict) -> "DisoraxConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=require(raw, "vocab", int), width=require(raw, "width", int),
                  eps=_number(_section(raw, "norm", ""), "eps", "norm."),
                  residual_mult=_number(raw, "residual_mult", "") if "residual_mult" in raw else 1.0,
                  layers=tuple(_read_layer(layer, i) for i, layer in enumerate(layers)))
        positive("vocab", cfg.vocab)
        positive("width", cfg.width)
        if not cfg.eps >= 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {cfg.eps!r}")
        blended = [(l["mixer"]["kv_heads"], l["mixer"]["vdim"]) for l in cfg.layers
                   if l["type"] == "attention" and l["mixer"]["v_mix"]]
        if len(set(blended)) > 1:
            raise ConfigError(f"config.json: layers that blend values need value heads of one number and size, got {blended}")
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "norm": {"eps": self.eps}, "residual_mult": self.residual_mult,
                "layers": copy.deepcopy(list(self.layers))}

    @classmethod
    def preset_names(cls) -> list[str]:
        return sorted(p.stem for p in PRESET_DIR.glob("*.json"))

    @classmethod
    def preset(cls, name: str) -> "DisoraxConfig":
        path = PRESET_DIR / f"{name}.json"
        if not path.is_file():
            raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")
        return cls.from_dict(json.loads(path.read_text()))
