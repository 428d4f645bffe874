"""Attention whose keys and values are made from one low-rank row per token.

q = Wq h, per head of ``dim`` elements. c = norm(Wdkv h) * w_norm, a row of ``kv_rank``
elements (RMS norm in 32-bit): the only thing a position leaves in the cache. Per
head h: k = Wuk_h c, v = Wuv_h c; score = (q . k) * scale; a causal or windowed
softmax, optionally with a sink in the denominator; the head's output is multiplied
by sigmoid(Wg h)_h; Wo over the concatenated heads. No positions enter.

Single tokens and portions of prompts never form the keys and values. Since
q_h . (Wuk_h c) = (Wuk_h^T q_h) . c and sum_j p_j Wuv_h c_j = Wuv_h (sum_j p_j c_j), a head's query is carried into the latent
space (one small product per head), attention runs over the cached rows themselves
with every head reading the same row as key and as value (``kv_rank`` wide, one
"kv head"), and the result is carried out through Wuv_h. A step reads kv_rank
numbers per cached position instead of heads * (dim + vdim). The per-head gate is
one number and commutes with Wuv_h, so it is applied where attention writes its rows.

A step in which every sequence starts at its first token (whole prompts) has no cached
rows to read, and there the other order is cheaper: the step's own keys and values
are made from its latent rows by one dense product, [Wuk; Wuv] c, written to scratch
pages that only this call sees, and ordinary attention with heads of ``dim`` (not
``kv_rank``) elements runs over them, on the tensor cores where the head sizes allow.
What the cache keeps is the same either way.
"""

from __future__ import annotations

import copy

import torch

from .base import KVNeed, TensorSpec, register_mixer
from .branches import Branch


class LatentAttention(Branch):
    """params: hidden, heads, dim, vdim, kv_rank, scale, window (None or int), sink (bool), gate (bool), eps."""

    def __init__(self, params):
        super().__init__(params)
        p = params
        self.hidden = int(p["hidden"])
        self.heads = int(p["heads"])
        self.dim = int(p["dim"])
        self.vdim = int(p.get("vdim") or self.dim)
        self.rank = int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.window = None if p.get("window") is None else int(p["window"])
        self.has_sink = bool(p.get("sink", False))
        self.has_gate = bool(p.get("gate", False))
        self.eps = float(p.get("eps", 0.0))

    def tensor_specs(self):
        specs = {"q": TensorSpec((self.heads * self.dim, self.hidden)),
                 "dkv": TensorSpec((self.rank, self.hidden)),
                 "dkv.norm": TensorSpec((self.rank,), "gain"),
                 "uk": TensorSpec((self.heads * self.dim, self.rank)),
                 "uv": TensorSpec((self.heads * self.vdim, self.rank)),
                 "o": TensorSpec((self.hidden, self.heads * self.vdim))}
        if self.has_gate:
            specs["g"] = TensorSpec((self.heads, self.hidden))
        if self.has_sink:
            specs["sink"] = TensorSpec((self.heads,), "vector")
        return specs

    def cache_need(self):
        return KVNeed(1, self.rank, self.window, values=False)

    def attention_head_dims(self):
        """Whole prompts in bfloat16 run on the tensor cores where key and value heads have one size that is a
        multiple of 16: that kernel is compiled per head size."""
        return (self.dim,) if self.dim == self.vdim and self.dim % 16 == 0 and self.dim <= 256 else ()

    def bind(self, tensors, runtime):
        self.w = {k: tensors[k] for k in ("q", "dkv", "o") + (("g",) if self.has_gate else ())}
        self.norm_gain = tensors["dkv.norm"].float().contiguous()
        # per head: Wuk_h^T [kv_rank, dim] carries a query in, Wuv_h [vdim, kv_rank] carries a result out
        self.uk_t = tensors["uk"].view(self.heads, self.dim, self.rank).transpose(1, 2).contiguous()
        self.uv = tensors["uv"].view(self.heads, self.vdim, self.rank).contiguous()
        self.w_expand = torch.cat([tensors["uk"], tensors["uv"]], dim=0).contiguous()  # [heads * (dim + vdim), kv_rank]
        self.no_freq = torch.zeros(0, dtype=torch.float32, device=runtime.device)
        self.sink = tensors["sink"].float().contiguous() if self.has_sink else None
        self.bind_standalone()

    def in_weight(self):
        return torch.cat([self.w["q"], self.w["dkv"]] + ([self.w["g"]] if self.has_gate else []), dim=0)

    def out_weight(self):
        return self.w["o"]

    def middle(self, ctx, proj, cache, out, col0, scale):
        ops = ctx.ops
        H, R = self.heads, self.rank
        c_col = H * self.dim
        gate = (c_col + R, "head") if self.has_gate else None
        batch = ctx.batch
        if not batch.is_decode and not any(batch.starts):
            # whole prompts: keys and values of the step's own rows, in scratch pages of this call
            rows = ops.latent_norm_write(proj, c_col, R, self.norm_gain, self.eps, batch, cache, keep_rows=True)
            kv = ops.linear(rows, self.w_expand)
            scratch_batch, scratch = self._scratch(ctx, kv)
            ops.rotate_norm_write(kv, 0, 0, H * self.dim, 0, H, self.dim, self.vdim, self.no_freq, 0, None, scratch_batch,
                                  scratch)
            ops.sink_attention(proj, 0, H, self.dim, self.vdim, self.sink, self.scale, self.window, scratch_batch, scratch,
                               out, col0, scale, gate=gate)
            return
        ops.latent_norm_write(proj, c_col, R, self.norm_gain, self.eps, batch, cache)
        q_lat = ops.head_linear(proj[:, :c_col], self.uk_t)  # [rows, heads * kv_rank]
        mixed = torch.empty_like(q_lat)
        ops.sink_attention(q_lat, 0, H, R, R, self.sink, self.scale, self.window, ctx.batch, cache, mixed, 0, 1.0,
                           gate=gate, gate_rows=proj if gate else None)
        ops.head_linear(mixed, self.uv, out=out, out_col=col0, out_scale=scale)

    def _scratch(self, ctx, kv):
        """Scratch pages for the keys and values of a step of whole prompts, and the step's description with every
        sequence in a slot of its own of the scratch table. The layout depends on the step alone and is shared by
        the layers of the step."""
        from ..cache.store import PAGE, KVView  # the cache's module imports this package's base

        batch = ctx.batch
        layout = ctx.shared.get("whole_prompt_pages")
        if layout is None:
            pages = [-(-n // PAGE) for n in batch.q_lens]
            width = max(pages)
            table = torch.zeros((len(pages), width), dtype=torch.int32)
            first = 0
            for s, n in enumerate(pages):
                table[s, :n] = torch.arange(first, first + n, dtype=torch.int32)
                first += n
            view = copy.copy(batch)
            view.seq_slot = torch.arange(len(pages), dtype=torch.int32, device=kv.device)
            layout = ctx.shared["whole_prompt_pages"] = (view, table.to(kv.device), first, width)
        view, table, n_pages, width = layout
        # zeroed like the cache itself: a kernel that takes whole pages multiplies what lies beyond a sequence's end
        # by weights of zero, and that must not be a NaN's bit pattern
        k = torch.zeros((n_pages, self.heads, PAGE, self.dim), dtype=kv.dtype, device=kv.device)
        v = torch.zeros((n_pages, self.heads, PAGE, self.vdim), dtype=kv.dtype, device=kv.device)
        return view, KVView(k, v, table, width, self.window, self.heads, self.dim, self.vdim)


register_mixer("latent_attention", LatentAttention)
