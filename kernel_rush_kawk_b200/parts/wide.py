"""Parts for models whose residual stream is kept in 32-bit on every path.

* ``ScaledEmbedding``: x = table[token] * scale, written as float32 rows.
* ``WideRMSNorm``: y = x / sqrt(mean(x^2) + eps) * (offset + w) with x, the sum
  x + branch and all arithmetic in float32; only y is rounded to the path's
  dtype. ``offset`` 1 serves weights that are stored around zero, 0 the usual
  gain. The stream it leaves behind (``x_new``) is float32.
* ``GatedMLP``: down(act(gate h) * (up h)) with the activation as a parameter
  (``gelu_tanh``: 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), or ``silu``);
  the activation and the product are computed in float32 and rounded once.
"""

from __future__ import annotations

import torch

from .base import Embedding, FeedForward, Norm, Stream, TensorSpec, register_embedding, register_feed_forward, register_norm
from .norm import Normed

ACTIVATIONS = {"silu": 0, "gelu_tanh": 1, "sigmoid": 2}


class ScaledEmbedding(Embedding):
    """params: vocab, hidden, scale."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.scale = float(params.get("scale", 1.0))
        self.table = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.table = tensors["table"]

    def forward(self, ctx):
        return ctx.ops.embed_scaled(self.table, ctx.batch.tokens, ctx.batch.n_rows, self.scale)


class WideRMSNorm(Norm):
    """params: size, eps, gain_offset (default 0)."""

    def __init__(self, params):
        super().__init__(params)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.offset = float(params.get("gain_offset", 0.0))
        self.gain = None
        self.dtype = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.size,), "vector" if self.offset else "gain")}

    def bind(self, tensors, runtime):
        self.gain = tensors["weight"].float().contiguous()
        self.dtype = runtime.dtype

    def forward(self, ctx, stream: Stream) -> Normed:
        x = stream.x
        if x.dtype != torch.float32:
            raise TypeError("a wide norm follows a float32 residual stream (an embedding or norm of the same family)")
        x_new = ctx.ops.empty_like(x) if stream.branch is not None else x
        rows = ctx.ops.rmsnorm_wide(x, stream.branch, self.gain, self.offset, self.eps, x_new, self.dtype)
        normed = Normed(ctx.ops, x, stream.branch, self.gain, self.eps, x_new)
        normed.mark_fused(rows)  # computed here and now: a product never folds this norm into its prologue
        stream.x = x_new
        stream.branch = None
        return normed


class GatedMLP(FeedForward):
    """params: hidden, intermediate, activation."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.intermediate = int(params["intermediate"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ("silu", "gelu_tanh"):
            raise ValueError(f"unknown activation '{self.activation}' for a gated feed-forward")
        self.w_gate_up = self.w_down = None

    def tensor_specs(self):
        return {"gate": TensorSpec((self.intermediate, self.hidden)),
                "up": TensorSpec((self.intermediate, self.hidden)),
                "down": TensorSpec((self.hidden, self.intermediate))}

    def bind(self, tensors, runtime):
        self.w_gate_up = torch.cat([tensors["gate"], tensors["up"]], dim=0).contiguous()
        self.w_down = tensors["down"].contiguous()

    def forward(self, ctx, h):
        act = ctx.ops.gate_up_act(h, self.w_gate_up, self.intermediate, self.activation)
        return ctx.ops.linear(act, self.w_down)


register_embedding("scaled_embedding", ScaledEmbedding)
register_norm("rmsnorm_wide", WideRMSNorm)
register_feed_forward("gated_mlp", GatedMLP)
