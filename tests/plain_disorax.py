"""A plain, slow restatement of the Disorax decoder, one function per mechanism.

Written from the design's equations for the tests only; it shares no code with
the package. Everything runs in the dtype of the tensors it is given (float64 in
the tests). Notation: x is the residual stream [T, C]; h a sublayer's normalised
input; positions count from 0.

  norm        y = x / sqrt(mean(x^2) + eps) * g
  embedding   x = E[token]
  layer       x <- x + m * (mixer(norm1(x)) + ff(norm2(x)))      (both norms read the same x)
  output      logits = W_head . norm_final(x)

Mixers (all gated on their way out, all read the same h):
  attention           grouped-query heads, rotation of part of each head, a window that also keeps the
                      sequence's first tokens, values blended with an earlier layer's, gate per element
  latent_attention    keys and values made from one normalised low-rank row per token; causal; gate per head
  latent_attention_2  the same over a sliding window, with a sink in the softmax's denominator
Feed-forward: routed SwiGLU experts (softmax over the chosen logits) plus a shared one behind a sigmoid.
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


def read_folder(folder, dtype=torch.float64):
    from safetensors import safe_open

    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    w = {}
    for shard in sorted(folder.glob("*.safetensors")):
        with safe_open(str(shard), framework="pt", device="cpu") as f:
            for name in f.keys():
                t = f.get_tensor(name)
                w[name] = t.to(dtype) if t.dtype.is_floating_point else t
    return cfg, w


# ---------------------------------------------------------------------------
# small pieces
# ---------------------------------------------------------------------------

def rms_norm(x, g, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * g


def silu(z):
    return z * torch.sigmoid(z)


def rotate_part(x, positions, dims, base):
    """x [T, heads, D]: element i < dims/2 of a head is paired with element i + dims/2 and the pair is
    turned by the angle position * base^(-2i/dims); elements from ``dims`` on pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


def visible(T, window=None, keep_first=0):
    """[T, T] bool: query i (row) sees key j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    see = j <= i
    if window is not None:
        see &= (i - j < window) | (j < keep_first)
    return see


def masked_softmax_mix(q, k, v, scale, see, sink=None):
    """q [T, H, D], k [T, G, D], v [T, G, DV] -> [T, H, DV], one query after the other. ``sink`` [H]: one more
    term exp(sink_h) in the denominator, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[-1]), dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = torch.nonzero(see[i]).flatten()
            s = (k[js, g] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            denom = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - m))
            out[i, h] = (e / denom) @ v[js, g]
    return out


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------

def attention(h, w, p, m, shared):
    """The rotated grouped-query mixer. ``shared`` carries the first value-mixing layer's values."""
    T = h.shape[0]
    H, G, D, DV = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, DV)
    q = rotate_part(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_part(k, pos, m["rot"]["dims"], m["rot"]["base"])
    if m.get("v_mix"):
        if "v_first" in shared:
            lam = w[p + "vmix"]
            v = (1.0 - lam) * v + lam * shared["v_first"]
        else:
            shared["v_first"] = v
    see = visible(T, m["mask"]["size"], m["mask"].get("keep_first", 0))
    o = masked_softmax_mix(q, k, v, m["scale"], see).reshape(T, H * DV)
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T


def latent_attention(h, w, p, m, eps, window=None, sink=None):
    T = h.shape[0]
    H, D, DV = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    c = rms_norm(h @ w[p + "dkv"].T, w[p + "dkv.norm"], eps)
    k = (c @ w[p + "uk"].T).view(T, H, D)
    v = (c @ w[p + "uv"].T).view(T, H, DV)
    o = masked_softmax_mix(q, k, v, m["scale"], visible(T, window), sink)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * DV) @ w[p + "o"].T


# ---------------------------------------------------------------------------
# feed-forward
# ---------------------------------------------------------------------------

def expert(h, w, p):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def routed_ff(h, w, p, mlp):
    E, top = mlp["router"]["experts"], mlp["router"]["top"]
    z = h @ w[p + "router"].T + w[p + "router.b"]
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        best = torch.topk(z[t], top).indices
        weight = torch.softmax(z[t, best], dim=0)
        for e, a in zip(best.tolist(), weight):
            out[t] += a * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    assert E == z.shape[1]
    if mlp.get("shared") is not None:
        out = out + torch.sigmoid(h @ w[p + "shared.sg"].T) * expert(h, w, p + "shared.")
    return out


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def forward(cfg, w, ids, keep_layers=False):
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    x = w["embed"][torch.as_tensor(ids)]
    shared = {}
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        m = layer["mixer"]
        h1 = rms_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "attention":
            a = attention(h1, w, p + "mix.", m, shared)
        elif layer["type"] == "latent_attention":
            a = latent_attention(h1, w, p + "mix.", m, eps)
        elif layer["type"] == "latent_attention_2":
            a = latent_attention(h1, w, p + "mix.", m, eps, m["mask"]["size"], w[p + "mix.sink"])
        else:
            raise ValueError(layer["type"])
        b = 0.0
        if layer["mlp"] is not None:
            b = routed_ff(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"])
        x = x + mult * (a + b)
        after.append(x)
    logits = rms_norm(x, w["final.norm"], eps) @ w["head"].T
    return (logits, torch.stack(after)) if keep_layers else logits
