"""Shared by the Taredra tests: small configurations, model folders, comparisons.

The configurations differ from one another in every size and constant, and none of a
model's sizes coincide by accident (key and value heads of different sizes, a rotation
of part of a head, head counts that do not divide the width, ranks other than the
default, sizes that are no multiple of 8 or 32, a layer without a feed-forward in
different places).

  name  width vocab layers
  ta     64   211   wkv(2 x 16, rank 8, ff 80) | parallel(left 4/2 heads dim 16 vdim 32 window 10 rot 8; right 3 x 16, rank 8; no ff)
                    | parallel(left 2/2 heads dim 24 vdim 8 window 37 rot 24; right 1 x 48, rank 12; ff 72)
  tb     96   301   parallel(left 6/1 heads dim 32 vdim 32 window 70 rot 16; right 2 x 32; ff 136) | wkv(3 x 32, no ff)
                    | wkv(1 x 64, ff 40) | parallel(left 3/3 heads dim 8 vdim 40 window 5 rot 2; right 5 x 8; ff 96)
  tc     50    97   parallel(left 3/3 heads dim 6 vdim 5 window 3 rot 4; right 1 x 7, rank 3; ff 33) | wkv(3 x 9, rank 5, no ff)
                    (nothing a multiple of 4 or 8: every kernel's plain path, the products' fallbacks, padded columns)
"""

from __future__ import annotations

import json
from pathlib import Path

import torch

import plain_taredra as plain


def _left(heads, kv, dim, vdim, window, rot, base, scale):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": window},
            "rot": {"dims": rot, "base": base}}


CONFIGS = {
    "ta": {"architecture": "Taredra", "vocab": 211, "width": 64, "embedding": {"scale": 3.0}, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "wkv", "mixer": {"heads": 2, "dim": 16, "rank": 8}, "mlp": {"kind": "dense", "ff": 80}},
               {"type": "parallel", "mlp": None,
                "mixer": {"left": _left(4, 2, 16, 32, 10, 8, 100.0, 0.31), "right": {"heads": 3, "dim": 16, "rank": 8},
                          "left_scale": 0.7, "right_scale": 1.3}},
               {"type": "parallel", "mlp": {"kind": "dense", "ff": 72},
                "mixer": {"left": _left(2, 2, 24, 8, 37, 24, 5000.0, 0.2), "right": {"heads": 1, "dim": 48, "rank": 12},
                          "left_scale": 1.2, "right_scale": 0.6}},
           ]},
    "tb": {"architecture": "Taredra", "vocab": 301, "width": 96, "embedding": {"scale": 5.0}, "norm": {"eps": 1e-6},
           "layers": [
               {"type": "parallel", "mlp": {"kind": "dense", "ff": 136},
                "mixer": {"left": _left(6, 1, 32, 32, 70, 16, 15000.0, 0.18), "right": {"heads": 2, "dim": 32},
                          "left_scale": 0.9, "right_scale": 1.1}},
               {"type": "wkv", "mixer": {"heads": 3, "dim": 32}, "mlp": None},
               {"type": "wkv", "mixer": {"heads": 1, "dim": 64}, "mlp": {"kind": "dense", "ff": 40}},
               {"type": "parallel", "mlp": {"kind": "dense", "ff": 96},
                "mixer": {"left": _left(3, 3, 8, 40, 5, 2, 10.0, 0.5), "right": {"heads": 5, "dim": 8},
                          "left_scale": 0.5, "right_scale": 1.5}},
           ]},
    "tc": {"architecture": "Taredra", "vocab": 97, "width": 50, "embedding": {"scale": 2}, "norm": {"eps": 1e-5},
           "layers": [
               {"type": "parallel", "mlp": {"kind": "dense", "ff": 33},
                "mixer": {"left": _left(3, 3, 6, 5, 3, 4, 7.0, 0.4), "right": {"heads": 1, "dim": 7, "rank": 3},
                          "left_scale": 1, "right_scale": 2}},
               {"type": "wkv", "mixer": {"heads": 3, "dim": 9, "rank": 5}, "mlp": None},
           ]},
}
SEEDS = {"ta": 5, "tb": 6, "tc": 7}


def config(name: str):
    from kernel_rush_kawk_b200 import TaredraConfig

    return TaredraConfig.from_dict(CONFIGS[name])


def write_folder(folder, name: str) -> Path:
    """Random weights, shaped so that every mechanism carries weight in the logits: projections of
    std 0.08, the attention's queries and keys scaled up (sharp softmax: a wrong key shows), sinks near
    the scores' size, decays spread over (0, 1), gains around their neutral value."""
    from kernel_rush_kawk_b200 import write_model_folder
    from kernel_rush_kawk_b200.engine.model import expected_tensors
    from kernel_rush_kawk_b200.config.registry import get_architecture

    cfg = config(name)
    names = expected_tensors(get_architecture(cfg.architecture).plan(cfg))
    scale = {}
    for n in names:
        if n.endswith(".left.q") or n.endswith(".left.k"):
            scale[n] = 3.0
        elif n.endswith(".sink") or n.endswith(".w0") or n.endswith(".a.b") or n.endswith(".mix.u"):
            scale[n] = 10.0
        elif n.endswith(".w2"):
            scale[n] = 8.0
        elif ".mu." in n:
            scale[n] = 6.0
    folder = write_model_folder(folder, cfg, SEEDS[name], std=0.08, gain_std=0.1, scale=scale)
    return folder


def prompts(name: str, lengths, seed=0):
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist() for n in lengths]


_cache: dict = {}


def plain_logits(folder, ids) -> torch.Tensor:
    """float64 logits [T, vocab] of the plain implementation (cached per folder and sequence)."""
    key = (str(folder), tuple(ids))
    if key not in _cache:
        cfg, w = plain.read_folder(folder, torch.float64)
        _cache[key] = plain.forward(cfg, w, ids)
    return _cache[key]


def spread(got: torch.Tensor, ref: torch.Tensor) -> torch.Tensor:
    """Per row: root mean square of the difference with its mean taken off, over the reference's own
    spread. A wrong key, window or state moves this by tenths to ones; rounding by 1e-6 in 32-bit and, with
    the sharp softmax of these test weights, by up to 1.1e-1 in bfloat16 (at a sequence's first positions). The 32-bit comparisons are the
    sharp ones; the bfloat16 ones show that the serving path computes the same model."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    r = ref - ref.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / r.pow(2).mean().sqrt()


TOL = {"float32": 2e-5, "bfloat16": 2e-1}


def assert_logits(got, ref, dtype: str, what: str) -> None:
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    s = spread(got, ref)
    worst = int(s.argmax())
    assert s.max().item() <= TOL[dtype], f"{what}: row {worst} differs by {s.max().item():.3e} of the logits' spread (allowed {TOL[dtype]:.0e})"
