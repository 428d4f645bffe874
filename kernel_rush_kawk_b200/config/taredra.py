"""Configuration of the Taredra decoder, read from its own config.json keys.

The file names the design with one string (``architecture``) and describes the
model as a list of layers, each with a mixer of its own kind and sizes:

    {"architecture": "Taredra", "vocab": V, "width": C,
     "embedding": {"scale": s}, "norm": {"eps": e},
     "layers": [{"type": "parallel" | "wkv", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...]}

``wkv`` mixer: ``heads``, ``dim``. ``parallel`` mixer: ``left`` (``heads``,
``kv_heads``, ``dim``, ``vdim``, ``scale``, ``mask.size``, ``rot.dims``,
``rot.base``), ``right`` (``heads``, ``dim``), ``left_scale``, ``right_scale``.
Every size and constant comes from the file; sizes that the file leaves to the
tensors (the rank of a decay's two small matrices) are read from the checkpoint
(``TaredraConfig.with_tensor_shapes``), or default for random weights.
"""

from __future__ import annotations

import copy
import json
from dataclasses import dataclass, field
from pathlib import Path

from .base import ConfigError, ModelConfig, positive, require

PRESET_DIR = Path(__file__).parent / "presets" / "taredra"

#: rank of the decay's low-rank pair where neither a checkpoint nor the configuration gives one
DEFAULT_DECAY_RANK = 16


def _section(raw: dict, key: str, where: str) -> dict:
    value = raw.get(key)
    if not isinstance(value, dict):
        raise ConfigError(f"config.json: {where}'{key}' must be an object, got {value!r}")
    return value


def _int(raw: dict, key: str, where: str) -> int:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, int) or value <= 0:
        raise ConfigError(f"config.json: {where}'{key}' must be a positive integer, got {value!r}")
    return value


def _number(raw: dict, key: str, where: str) -> float:
    value = raw.get(key)
    if isinstance(value, bool) or not isinstance(value, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {value!r}")
    return float(value)


def _read_window_side(raw: dict, where: str) -> dict:
    out = {"heads": _int(raw, "heads", where), "kv_heads": _int(raw, "kv_heads", where),
           "dim": _int(raw, "dim", where), "vdim": _int(raw, "vdim", where),
           "scale": _number(raw, "scale", where),
           "mask": {"size": _int(_section(raw, "mask", where), "size", where + "mask.")},
           "rot": {"dims": _int(_section(raw, "rot", where), "dims", where + "rot."),
                   "base": _number(_section(raw, "rot", where), "base", where + "rot.")}}
    if out["heads"] % out["kv_heads"]:
        raise ConfigError(f"config.json: {where}heads ({out['heads']}) must be a multiple of kv_heads ({out['kv_heads']})")
    if out["rot"]["dims"] % 2 or out["rot"]["dims"] > out["dim"]:
        raise ConfigError(f"config.json: {where}rot.dims ({out['rot']['dims']}) must be even and at most dim ({out['dim']})")
    if not out["rot"]["base"] > 0:
        raise ConfigError(f"config.json: {where}rot.base must be positive")
    return out


def _read_state_side(raw: dict, where: str) -> dict:
    out = {"heads": _int(raw, "heads", where), "dim": _int(raw, "dim", where)}
    if "rank" in raw:
        out["rank"] = _int(raw, "rank", where)
    return out


def _read_layer(raw: dict, i: int) -> dict:
    where = f"layers[{i}]."
    kind = raw.get("type")
    mixer = _section(raw, "mixer", where)
    if kind == "wkv":
        m = _read_state_side(mixer, where + "mixer.")
    elif kind == "parallel":
        m = {"left": _read_window_side(_section(mixer, "left", where + "mixer."), where + "mixer.left."),
             "right": _read_state_side(_section(mixer, "right", where + "mixer."), where + "mixer.right."),
             "left_scale": _number(mixer, "left_scale", where + "mixer."),
             "right_scale": _number(mixer, "right_scale", where + "mixer.")}
    else:
        raise ConfigError(f"config.json: {where}type '{kind}' is not a mixer of this design (wkv, parallel)")
    mlp = raw.get("mlp")
    if mlp is not None:
        if not isinstance(mlp, dict) or mlp.get("kind") != "dense":
            raise ConfigError(f"config.json: {where}mlp must be null or of kind 'dense', got {mlp!r}")
        mlp = {"kind": "dense", "ff": _int(mlp, "ff", where + "mlp.")}
    return {"type": kind, "mixer": m, "mlp": mlp}


@dataclass(frozen=True)
class TaredraConfig(ModelConfig):
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    #: one normalised dict per layer (type, mixer, mlp); treated as read-only
    layers: tuple = field(default_factory=tuple)

    architecture = "Taredra"

    @classmethod
    def from_dict(cls, raw: dict) -> "TaredraConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        cfg = cls(vocab=require(raw, "vocab", int), width=require(raw, "width", int),
                  eps=_number(_section(raw, "norm", ""), "eps", "norm."),
                  embedding_scale=_number(_section(raw, "embedding", ""), "scale", "embedding."),
                  layers=tuple(_read_layer(layer, i) for i, layer in enumerate(layers)))
        positive("vocab", cfg.vocab)
        positive("width", cfg.width)
        if not cfg.eps >= 0:
            raise ConfigError(f"config.json: norm.eps must not be negative, got {cfg.eps!r}")
        return cfg

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.eps},
                "layers": copy.deepcopy(list(self.layers))}

    def with_tensor_shapes(self, shapes: dict) -> "TaredraConfig":
        """The same configuration with the sizes that only the checkpoint gives: the rank of
        every decay's low-rank pair, from the shape of its first matrix."""
        layers = copy.deepcopy(list(self.layers))
        for i, layer in enumerate(layers):
            for side, prefix in ((layer["mixer"], f"l{i}.mix."), (layer["mixer"].get("right"), f"l{i}.mix.right.")):
                if isinstance(side, dict) and "dim" in side and prefix + "w1" in shapes:
                    side["rank"] = int(shapes[prefix + "w1"][0])
        return TaredraConfig(self.vocab, self.width, self.eps, self.embedding_scale, tuple(layers))

    @classmethod
    def preset_names(cls) -> list[str]:
        return sorted(p.stem for p in PRESET_DIR.glob("*.json"))

    @classmethod
    def preset(cls, name: str) -> "TaredraConfig":
        path = PRESET_DIR / f"{name}.json"
        if not path.is_file():
            raise ConfigError(f"unknown preset '{name}'; known presets: {cls.preset_names()}")
        return cls.from_dict(json.loads(path.read_text()))
