"""The Taredra decoder as a plan.

A scaled token embedding feeds a 32-bit residual stream; every layer is
x += mixer(norm1(x)) and, if it has a feed-forward, x += ff(norm2(x)); the norms
are RMS norms whose weights are stored around zero; a final norm and the
embedding table itself (unscaled) give the logits. A layer's mixer is either
RWKV-style time mixing (``wkv``) or two mixers side by side (``parallel``): windowed
grouped-query attention with a softmax sink on the left and a generalized delta rule on
the right, summed with the configuration's two weights. The feed-forward is gated
with the tanh form of GELU.

Tensor names: ``embed``, ``final.norm`` and, for layer i, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.{gate,up,down}``.
"""

from __future__ import annotations

from ..config.registry import register_architecture
from ..config.taredra import DEFAULT_DECAY_RANK, TaredraConfig
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

#: the design gives no longest sequence; tables and caches are sized by what the caller asks for
MAX_POSITIONS = 1 << 20


def _names(prefix: str, keys) -> dict:
    return {k: prefix + k for k in keys}


def taredra_plan(cfg: TaredraConfig) -> ModelPlan:
    C = cfg.width
    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        norm = lambda key: PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps, "gain_offset": 1.0}, {"weight": p + key})
        m = layer["mixer"]
        if layer["type"] == "wkv":
            params = {"hidden": C, "heads": m["heads"], "dim": m["dim"], "rank": m.get("rank", DEFAULT_DECAY_RANK),
                      "eps": cfg.eps}
            keys = ["mu.r", "mu.k", "mu.v", "mu.g", "mu.w", "r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o"]
            mixer = PartSpec("wkv_time_mix", params, _names(p + "mix.", keys))
        else:
            left, right = m["left"], m["right"]
            branches = [
                {"name": "left", "kind": "sink_window_attention", "scale": m["left_scale"],
                 "params": {"hidden": C, "heads": left["heads"], "kv_heads": left["kv_heads"], "dim": left["dim"],
                            "vdim": left["vdim"], "scale": left["scale"], "window": left["mask"]["size"],
                            "rot_dims": left["rot"]["dims"], "rot_base": left["rot"]["base"], "value_norm": True,
                            "sink": True, "eps": cfg.eps}},
                {"name": "right", "kind": "delta_rule", "scale": m["right_scale"],
                 "params": {"hidden": C, "heads": right["heads"], "dim": right["dim"],
                            "rank": right.get("rank", DEFAULT_DECAY_RANK), "eps": cfg.eps}},
            ]
            keys = ["left." + k for k in ("q", "k", "v", "sink", "o")]
            keys += ["right." + k for k in ("r", "k", "v", "g", "a", "a.b", "w1", "w2", "w0", "norm", "o")]
            mixer = PartSpec("parallel", {"hidden": C, "branches": branches}, _names(p + "mix.", keys))
        ffn_norm = ffn = None
        if layer["mlp"] is not None:
            ffn_norm = norm("norm2")
            ffn = PartSpec("gated_mlp", {"hidden": C, "intermediate": layer["mlp"]["ff"], "activation": "gelu_tanh"},
                           _names(p + "mlp.", ("gate", "up", "down")))
        layers.append(LayerSpec("prenorm", norm("norm1"), mixer, ffn_norm, ffn))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=C,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab": cfg.vocab, "hidden": C, "scale": cfg.embedding_scale},
                           {"table": "embed"}),
        position=None,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps, "gain_offset": 1.0}, {"weight": "final.norm"}),
        head=PartSpec("output_head", {"vocab": cfg.vocab, "hidden": C}, {"weight": "embed"}),
        max_positions=MAX_POSITIONS,
    )


register_architecture(TaredraConfig.architecture, TaredraConfig, taredra_plan)
