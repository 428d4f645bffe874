"""Mixers that can stand alone or side by side, and the mixer that sets them side by side.

A *branch* is a mixer that splits its work in three: a projection of its input
by one matrix of its own (``in_weight``), a middle part that turns the projected
rows into the rows its output projection reads (``middle``), and that output
projection (``out_weight``). Alone, it runs the three in turn. Side by side
(``ParallelMixer``), the branches read the same input, so their input matrices
are stacked into one product, each middle part writes its rows, already
multiplied by the branch's weight in the sum, into its own columns of one
buffer, and one product with the output matrices set side by side gives
sum_b scale_b * branch_b(h).
"""

from __future__ import annotations

import torch

from .base import Mixer, mixer_class, register_mixer


def pad_rows(w: torch.Tensor, multiple: int = 8) -> torch.Tensor:
    """``w`` with zero rows appended up to a multiple (the library product wants 16-byte rows of output)."""
    extra = -w.shape[0] % multiple
    if not extra:
        return w.contiguous()
    return torch.cat([w, w.new_zeros((extra, w.shape[1]))], dim=0).contiguous()


class Branch(Mixer):
    """A mixer in three parts; see the module text."""

    def in_weight(self) -> torch.Tensor:
        """[features, hidden]: every projection of the shared input, stacked."""
        raise NotImplementedError

    def out_weight(self) -> torch.Tensor:
        """[hidden, columns]: the output projection."""
        raise NotImplementedError

    def middle(self, ctx, proj, cache, out, col0: int, scale: float) -> None:
        """proj [rows, features] (a column slice of a wider buffer) -> out[:, col0:col0 + columns],
        multiplied by ``scale``."""
        raise NotImplementedError

    def bind_standalone(self) -> None:
        self._w_in = pad_rows(self.in_weight())
        self._w_out = self.out_weight().contiguous()

    def forward(self, ctx, h, cache):
        ops = ctx.ops
        proj = ops.linear(h, self._w_in)
        out = torch.empty((proj.shape[0], self._w_out.shape[1]), dtype=proj.dtype, device=proj.device)
        self.middle(ctx, proj, cache, out, 0, 1.0)
        return ops.linear(out, self._w_out)


class ParallelMixer(Mixer):
    """params: hidden, branches: a list of {"name", "kind", "params", "scale"}. The result is
    sum_b scale_b * branch_b(h). Tensor keys are "<name>.<the branch's key>"."""

    def __init__(self, params):
        super().__init__(params)
        self.hidden = int(params["hidden"])
        self.names, self.scales, self.branches = [], [], []
        for b in params["branches"]:
            cls = mixer_class(b["kind"])
            if not issubclass(cls, Branch):
                raise TypeError(f"mixer kind '{b['kind']}' cannot stand beside others (it is no Branch)")
            self.names.append(str(b["name"]))
            self.scales.append(float(b.get("scale", 1.0)))
            self.branches.append(cls(b["params"]))
        self.graph_safe = all(b.graph_safe for b in self.branches)

    def tensor_specs(self):
        return {f"{name}.{key}": spec for name, b in zip(self.names, self.branches)
                for key, spec in b.tensor_specs().items()}

    def cache_need(self):
        needs = []
        self._need_slices = []
        for b in self.branches:
            need = b.cache_need()
            many = isinstance(need, (tuple, list))
            group = list(need) if many else ([] if need is None else [need])
            self._need_slices.append((len(needs), len(group), many))
            needs.extend(group)
        return tuple(needs) if needs else None

    def attention_head_dims(self):
        return tuple(d for b in self.branches for d in getattr(b, "attention_head_dims", lambda: ())())

    def bind(self, tensors, runtime):
        for name, b in zip(self.names, self.branches):
            mine = {key[len(name) + 1:]: t for key, t in tensors.items() if key.startswith(name + ".")}
            b.bind(mine, runtime)
        ins = [b.in_weight() for b in self.branches]
        outs = [b.out_weight() for b in self.branches]
        self.in_cols, col = [], 0
        for w in ins:
            self.in_cols.append((col, w.shape[0]))
            col += w.shape[0]
        self.w_in = pad_rows(torch.cat(ins, dim=0))
        self.out_cols, col = [], 0
        for w in outs:
            self.out_cols.append(col)
            col += w.shape[1]
        self.out_width = col + (-col % 8)
        w_out = torch.cat(outs, dim=1)
        if self.out_width != col:
            w_out = torch.cat([w_out, w_out.new_zeros((w_out.shape[0], self.out_width - col))], dim=1)
        self.w_out = w_out.contiguous()
        self.out_used = col
        self.cache_need()

    def forward(self, ctx, h, cache):
        ops = ctx.ops
        proj = ops.linear(h, self.w_in)
        rows = proj.shape[0]
        alloc = torch.empty if self.out_used == self.out_width else torch.zeros
        out = alloc((rows, self.out_width), dtype=proj.dtype, device=proj.device)
        views = cache if isinstance(cache, tuple) else (() if cache is None else (cache,))
        for b, scale, (c0, n), o0, (first, count, many) in zip(self.branches, self.scales, self.in_cols, self.out_cols,
                                                               self._need_slices):
            mine = tuple(views[first:first + count]) if many else (views[first] if count else None)
            b.middle(ctx, proj[:, c0:c0 + n], mine, out, o0, scale)
        return ops.linear(out, self.w_out)


register_mixer("parallel", ParallelMixer)
