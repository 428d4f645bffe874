"""Shared by the Disorax tests: small configurations, model folders, comparisons.

The configurations differ from one another in every size and constant, and none of a model's sizes
coincide by accident: key and value heads of different sizes, one kv head and as many as query heads,
windows shorter and longer than a page, kept first tokens that fill less than a page and more than
one, a layer multiplier of 1 and others, layers in different orders, layers without a feed-forward,
experts of which a token takes one, some or all, with and without the shared expert, and one model
with nothing a multiple of 4 or 8.

  da  width 64, vocab 211, multiplier 0.5:
      attention 4/2 heads dim 16 vdim 24 window 10 keep 3 rot 8 (blend: first) + 5 experts top 2 ff 40, shared 24
      | latent 3 heads dim 16 vdim 8 rank 24, causal, no feed-forward
      | attention 2/2 heads dim 8 vdim 24 window 37 keep 0 rot 8 (blend) + 4 experts top 1 ff 32, no shared
      | latent 2 heads dim 8 vdim 40 rank 16 window 6 with a sink + 3 experts top 3 ff 16, shared 8
  db  width 96, vocab 301, multiplier 1:
      latent 5 heads dim 12 vdim 12 rank 40 window 70 with a sink + 8 experts top 2 ff 48, shared 64
      | attention 6/1 heads dim 32 vdim 32 window 70 keep 65 rot 16 (no blend), no feed-forward
      | attention 3/3 heads dim 8 vdim 40 window 5 keep 1 rot 2 (blend: the only one) + 2 experts top 1 ff 24, shared 16
      | latent 1 head dim 64 vdim 16 rank 8, causal + 6 experts top 4 ff 16, no shared
  dc  width 50, vocab 97, multiplier 1.7 (nothing a multiple of 4 or 8):
      attention 3/3 heads dim 6 vdim 5 window 3 keep 2 rot 4 + 3 experts top 2 ff 11, shared 7
      | latent 3 heads dim 7 vdim 5 rank 9 window 4 with a sink + 5 experts top 3 ff 9, shared 3
"""

from __future__ import annotations

import torch

import plain_disorax as plain


def _attn(heads, kv, dim, vdim, window, keep, rot, base, scale, v_mix):
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale,
            "mask": {"size": window, "keep_first": keep}, "rot": {"dims": rot, "base": base}, "v_mix": v_mix}


def _latent(heads, dim, vdim, rank, scale, window=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": rank, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def _moe(experts, top, ff, shared=None):
    m = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


CONFIGS = {
    "da": {"architecture": "Disorax", "vocab": 211, "width": 64, "norm": {"eps": 1e-5}, "residual_mult": 0.5, "layers": [
        {"type": "attention", "mixer": _attn(4, 2, 16, 24, 10, 3, 8, 100.0, 0.3, True), "mlp": _moe(5, 2, 40, 24)},
        {"type": "latent_attention", "mixer": _latent(3, 16, 8, 24, 0.25), "mlp": None},
        {"type": "attention", "mixer": _attn(2, 2, 8, 24, 37, 0, 8, 5000.0, 0.35, True), "mlp": _moe(4, 1, 32)},
        {"type": "latent_attention_2", "mixer": _latent(2, 8, 40, 16, 0.4, 6), "mlp": _moe(3, 3, 16, 8)},
    ]},
    "db": {"architecture": "Disorax", "vocab": 301, "width": 96, "norm": {"eps": 1e-6}, "residual_mult": 1.0, "layers": [
        {"type": "latent_attention_2", "mixer": _latent(5, 12, 12, 40, 0.3, 70), "mlp": _moe(8, 2, 48, 64)},
        {"type": "attention", "mixer": _attn(6, 1, 32, 32, 70, 65, 16, 15000.0, 0.18, False), "mlp": None},
        {"type": "attention", "mixer": _attn(3, 3, 8, 40, 5, 1, 2, 10.0, 0.5, True), "mlp": _moe(2, 1, 24, 16)},
        {"type": "latent_attention", "mixer": _latent(1, 64, 16, 8, 0.125), "mlp": _moe(6, 4, 16)},
    ]},
    "dc": {"architecture": "Disorax", "vocab": 97, "width": 50, "norm": {"eps": 1e-5}, "residual_mult": 1.7, "layers": [
        {"type": "attention", "mixer": _attn(3, 3, 6, 5, 3, 2, 4, 7.0, 0.4, False), "mlp": _moe(3, 2, 11, 7)},
        {"type": "latent_attention_2", "mixer": _latent(3, 7, 5, 9, 0.4, 4), "mlp": _moe(5, 3, 9, 3)},
    ]},
}
SEEDS = {"da": 11, "db": 12, "dc": 13}


def config(name: str):
    from kernel_rush_kawk_b200 import DisoraxConfig

    return DisoraxConfig.from_dict(CONFIGS[name])


def write_folder(folder, name: str):
    """Random weights, shaped so that every mechanism carries weight in the logits: projections of std
    0.08, queries and keys scaled up (a sharp softmax: a wrong key shows), sinks near the scores' size,
    gates and routers with logits of order one, blending weights well inside (0, 1)."""
    from kernel_rush_kawk_b200 import write_model_folder
    from kernel_rush_kawk_b200.config.registry import get_architecture
    from kernel_rush_kawk_b200.engine.model import expected_tensors

    cfg = config(name)
    names = expected_tensors(get_architecture(cfg.architecture).plan(cfg))
    scale = {}
    for n in names:
        if n.endswith(".mix.q") or n.endswith(".mix.k") or n.endswith(".mix.uk"):
            scale[n] = 3.0
        elif n.endswith(".sink") or n.endswith(".router.b"):
            scale[n] = 10.0
        elif n.endswith(".mix.g") or n.endswith(".router") or n.endswith(".shared.sg"):
            scale[n] = 4.0
        elif n.endswith(".vmix"):
            scale[n] = 5.0
    return write_model_folder(folder, cfg, SEEDS[name], std=0.08, gain_std=0.1, scale=scale)


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
    """Per row: root mean square of the difference with its mean taken off, over the reference's own spread.
    A wrong key, window, expert or kept token moves this by tenths to ones; rounding by 1e-6 in 32-bit."""
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    d = got - ref
    d = d - d.mean(dim=-1, keepdim=True)
    r = ref - ref.mean(dim=-1, keepdim=True)
    return d.pow(2).mean(dim=-1).sqrt() / r.pow(2).mean().sqrt()


TOL = {"float32": 5e-5, "bfloat16": 1e-1}


def assert_logits(got, ref, dtype: str, what: str) -> None:
    """32-bit: every row within the tolerance. bfloat16: a token whose two best router logits lie closer than
    the rounding of its input may take another expert than the 64-bit implementation does, and the rows after
    it feel that; so nineteen rows in twenty are held to the tolerance and the rest to five times it."""
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} vs {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite logits"
    s = spread(got, ref)
    worst = int(s.argmax())
    if dtype == "float32":
        assert s.max().item() <= TOL[dtype], f"{what}: row {worst} differs by {s.max().item():.3e} of the logits' spread (allowed {TOL[dtype]:.0e})"
        return
    over = int((s > TOL[dtype]).sum())
    assert over <= max(1, s.numel() // 20), f"{what}: {over} of {s.numel()} rows differ by more than {TOL[dtype]:.0e}; worst row {worst}: {s.max().item():.3e}"
    assert s.max().item() <= 5 * TOL[dtype], f"{what}: row {worst} differs by {s.max().item():.3e} of the logits' spread"
