"""The Disorax decoder as a plan.

A token embedding feeds a 32-bit residual stream. Every layer reads one x twice,
x <- x + m * (mixer(norm1(x)) + ff(norm2(x))), with plain RMS norms and m the
configuration's multiplier; a layer without a feed-forward adds its mixer alone.
A layer's mixer is grouped-query attention with a rotation of part of each head, a
window that also keeps the sequence's first tokens, values blended with those of
the first such layer, and a gate per element; or attention over one cached
low-rank row per token, causal or windowed with a sink, gated per head. The
feed-forward is a set of routed SwiGLU experts with a shared one behind a sigmoid.
A final norm and a head of its own give the logits.

Tensor names: ``embed``, ``final.norm``, ``head`` and, for layer i, ``l<i>.norm1``,
``l<i>.norm2``, ``l<i>.mix.*`` and ``l<i>.mlp.{router,router.b,e<j>.*,shared.*}``.
"""

from __future__ import annotations

from ..config.disorax import DisoraxConfig
from ..config.registry import register_architecture
from ..parts.plan import LayerSpec, ModelPlan, PartSpec, ScheduleEntry

#: the design gives no longest sequence; tables and caches are sized by what the caller asks for
MAX_POSITIONS = 1 << 20


def _names(prefix: str, keys) -> dict:
    return {k: prefix + k for k in keys}


def disorax_plan(cfg: DisoraxConfig) -> ModelPlan:
    C = cfg.width
    norm = lambda name: PartSpec("rmsnorm_wide", {"size": C, "eps": cfg.eps}, {"weight": name})
    layers = []
    blend_seen = False
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        m = layer["mixer"]
        if layer["type"] == "attention":
            params = {"hidden": C, "heads": m["heads"], "kv_heads": m["kv_heads"], "dim": m["dim"], "vdim": m["vdim"],
                      "scale": m["scale"], "window": m["mask"]["size"], "keep_first": m["mask"]["keep_first"],
                      "rot_dims": m["rot"]["dims"], "rot_base": m["rot"]["base"], "gate": "element", "eps": cfg.eps}
            keys = ["q", "k", "v", "g", "o"]
            if m["v_mix"]:
                params["value_mix"] = "blend" if blend_seen else "first"
                blend_seen = True
                keys.append("vmix")
            mixer = PartSpec("sink_window_attention", params, _names(p + "mix.", keys))
        else:
            second = layer["type"] == "latent_attention_2"
            params = {"hidden": C, "heads": m["heads"], "dim": m["dim"], "vdim": m["vdim"], "kv_rank": m["kv_rank"],
                      "scale": m["scale"], "window": m["mask"]["size"] if "mask" in m else None, "sink": second,
                      "gate": True, "eps": cfg.eps}
            keys = ["q", "dkv", "dkv.norm", "uk", "uv", "g", "o"] + (["sink"] if second else [])
            mixer = PartSpec("latent_attention", params, _names(p + "mix.", keys))
        ffn_norm = ffn = None
        mlp = layer["mlp"]
        if mlp is not None:
            shared = mlp.get("shared")
            E = mlp["router"]["experts"]
            keys = ["router", "router.b"] + [f"e{e}.{k}" for e in range(E) for k in ("gate", "up", "down")]
            if shared is not None:
                keys += ["shared.gate", "shared.up", "shared.down", "shared.sg"]
            ffn_norm = norm(p + "norm2")
            ffn = PartSpec("routed_experts",
                           {"hidden": C, "experts": E, "top": mlp["router"]["top"], "intermediate": mlp["expert"]["ff"],
                            "activation": "silu", "shared_intermediate": shared["ff"] if shared is not None else None,
                            "shared_gate": shared is not None}, _names(p + "mlp.", keys))
        layers.append(LayerSpec("parallel_residual", norm(p + "norm1"), mixer, ffn_norm, ffn,
                                block_params={"multiplier": cfg.residual_mult}))
    return ModelPlan(
        architecture=cfg.architecture,
        hidden_size=C,
        vocab_size=cfg.vocab,
        embedding=PartSpec("scaled_embedding", {"vocab": cfg.vocab, "hidden": C, "scale": 1.0}, {"table": "embed"}),
        position=None,
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("output_head", {"vocab": cfg.vocab, "hidden": C}, {"weight": "head"}),
        max_positions=MAX_POSITIONS,
    )


register_architecture(DisoraxConfig.architecture, DisoraxConfig, disorax_plan)
