"""A plain, slow restatement of the Taredra decoder, one function per mechanism.

Written from the design's equations for the tests only; it shares no code with
the package. Everything runs in the dtype of the tensors it is given (float64
in the tests), one token or one head after the other where that is the clearest
way to write it. Notation: x is the residual stream [T, C]; h a sublayer's
normalised input; a mixer returns [T, C].

  norm       y = x / sqrt(mean(x^2) + eps) * (1 + g)
  embedding  x = E[token] * s
  layer      x += mixer(norm1(x)); x += ff(norm2(x)) (the second only if the layer has one)
  output     logits = E . norm_final(x)   (E without its scale)
"""

from __future__ import annotations

import json
import math
from pathlib import Path

import torch


# ---------------------------------------------------------------------------
# reading a model folder
# ---------------------------------------------------------------------------

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

def unit_rms(x, eps):
    """x divided by its root mean square over the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def centered_norm(x, g, eps):
    """RMS norm whose stored weight sits around zero."""
    return unit_rms(x, eps) * (1.0 + g)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def gated_ff(h, w_gate, w_up, w_down):
    return (gelu_tanh(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def rotate_part(x, positions, dims, base):
    """x [T, heads, D]; the first ``dims`` elements of each head are rotated, element i with
    element i + dims/2 by the angle position * base^(-2i/dims); the others pass."""
    half = dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    a = positions.to(x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


# ---------------------------------------------------------------------------
# mechanisms
# ---------------------------------------------------------------------------

def sink_window_attention(q, k, v, scale, window, sink):
    """q [T, H, D], k [T, G, D], v [T, G, Dv] of one sequence from position 0. Query i sees keys
    j with 0 <= i - j < window. Each head's softmax has one more term in its denominator,
    exp(sink[h]), which has no value. Returns [T, H, Dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            out[i, h] = (e[:, None] * v[lo:i + 1, g]).sum(dim=0) / (e.sum() + torch.exp(sink[h] - m))
    return out


def windowed_branch(h, w, p, m, eps, positions):
    """The attention side of a 'parallel' mixer. ``w`` maps local names to tensors."""
    T = h.shape[0]
    H, G, D, Dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).view(T, H, D)
    k = (h @ w[p + "k"].T).view(T, G, D)
    v = (h @ w[p + "v"].T).view(T, G, Dv)
    q = rotate_part(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_part(k, positions, m["rot"]["dims"], m["rot"]["base"])
    v = unit_rms(v, eps)
    o = sink_window_attention(q, k, v, m["scale"], m["mask"]["size"], w[p + "sink"])
    return o.reshape(T, H * Dv) @ w[p + "o"].T


def delta_rule_scan(r, k, v, decay, rate, state=None):
    """Generalized delta rule of one sequence, token by token. r, k, v, decay, rate: [T, H, N].
    With u = k / sqrt(sum k^2 + 1e-6): S <- diag(decay) S - (rate * u)(u^T S) + k v^T, both
    first terms from the old S; o = S^T r. S is [H, N(key), N(value)]. Returns (o, S)."""
    T, H, N = r.shape
    S = torch.zeros(H, N, N, dtype=r.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, N, dtype=r.dtype)
    for t in range(T):
        u = k[t] / torch.sqrt((k[t] * k[t]).sum(dim=-1, keepdim=True) + 1e-6)
        uS = torch.einsum("hi,hij->hj", u, S)
        S = decay[t][:, :, None] * S - (rate[t] * u)[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S)
    return out, S


def delta_branch(h, w, p, m, eps):
    """The recurrent side of a 'parallel' mixer."""
    T = h.shape[0]
    H, N = m["heads"], m["dim"]
    r = (h @ w[p + "r"].T).view(T, H, N)
    k = (h @ w[p + "k"].T).view(T, H, N)
    v = (h @ w[p + "v"].T).view(T, H, N)
    lora = torch.tanh(h @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = torch.exp(-math.exp(-0.5) * torch.sigmoid(lora)).view(T, H, N)
    rate = torch.sigmoid(h @ w[p + "a"].T + w[p + "a.b"]).view(T, H, N)
    o, _ = delta_rule_scan(r, k, v, decay, rate)
    o = unit_rms(o, eps).reshape(T, H * N) * w[p + "norm"]
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def parallel_mixer(h, w, p, m, eps, positions):
    left = windowed_branch(h, w, p + "left.", m["left"], eps, positions)
    right = delta_branch(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def wkv_scan(r, k, v, decay, bonus, state=None):
    """r, k, v, decay [T, H, N], bonus [H, N]. o_t = (S + diag(bonus) k v^T)^T r with the old S,
    then S <- diag(decay) S + k v^T. Returns (o, S)."""
    T, H, N = r.shape
    S = torch.zeros(H, N, N, dtype=r.dtype) if state is None else state.clone()
    out = torch.zeros(T, H, N, dtype=r.dtype)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + bonus[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    return out, S


def wkv_mixer(h, w, p, m, eps):
    """Time mixing with a token shift: each projection reads h + (h_prev - h) * mu of its own."""
    T = h.shape[0]
    H, N = m["heads"], m["dim"]
    prev = torch.cat([torch.zeros_like(h[:1]), h[:-1]], dim=0)
    mix = lambda s: h + (prev - h) * w[p + "mu." + s]
    r = (mix("r") @ w[p + "r"].T).view(T, H, N)
    k = (mix("k") @ w[p + "k"].T).view(T, H, N)
    v = (mix("v") @ w[p + "v"].T).view(T, H, N)
    g = mix("g") @ w[p + "g"].T
    gate = g * torch.sigmoid(g)
    lora = torch.tanh(mix("w") @ w[p + "w1"].T) @ w[p + "w2"].T + w[p + "w0"]
    decay = torch.exp(-torch.exp(lora)).view(T, H, N)
    o, _ = wkv_scan(r, k, v, decay, w[p + "u"])
    o = unit_rms(o, eps).reshape(T, H * N) * w[p + "norm"]
    return (o * gate) @ w[p + "o"].T


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------

def forward(cfg, w, ids, keep_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the residual stream after every
    layer if asked)."""
    eps = cfg["norm"]["eps"]
    dtype = w["embed"].dtype
    ids = torch.as_tensor(ids, dtype=torch.long)
    positions = torch.arange(len(ids))
    x = w["embed"][ids] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = centered_norm(x, w[p + "norm1"], eps)
        if layer["type"] == "wkv":
            x = x + wkv_mixer(h, w, p + "mix.", layer["mixer"], eps)
        elif layer["type"] == "parallel":
            x = x + parallel_mixer(h, w, p + "mix.", layer["mixer"], eps, positions)
        else:
            raise ValueError(f"unknown layer type {layer['type']}")
        if layer.get("mlp") is not None:
            h = centered_norm(x, w[p + "norm2"], eps)
            x = x + gated_ff(h, w[p + "mlp.gate"], w[p + "mlp.up"], w[p + "mlp.down"])
        after.append(x)
    logits = centered_norm(x, w["final.norm"], eps) @ w["embed"].T
    if keep_layers:
        return logits.to(dtype), torch.stack(after)
    return logits
