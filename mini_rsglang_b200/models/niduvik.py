"""Niduvik as a composition of parts: every layer is a "sandwich_norm" block (an RMS norm before and after
each branch) around one mixer, "biased_window_attention" or "mamba2", and, where the layer has one, a
"clamped_glu" feed-forward; the output head reads the embedding table.  Sizes and constants come from the
configuration, layer by layer; the tensor names are the checkpoint's: `embed`, `final.norm`, and below `l<i>.`
the norms `norm1`, `norm1b`, `norm2`, `norm2b` (the tensor is the norm's root), `mix.*` and `mlp.*`.

What the design fixes: the feed-forward's sigmoid slope, the sink in the softmax, biases on q, k and v, one gate
a query head, and that the first layer which blends values is the one whose values the others blend with."""
from __future__ import annotations

from ..config.model_config import NiduvikConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec

GLU_SIGMOID_SLOPE = 1.702

ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                   "bias_table": "rel", "mix": "vmix", "gate": "g"}
SSM_NAMES = {"in": "in", "conv": "conv", "conv_bias": "conv.b", "dt_bias": "dt_bias", "a_log": "A_log", "d": "D",
             "norm": "norm", "out": "o"}
GLU_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def niduvik_spec(config: NiduvikConfig) -> ModelSpec:
    c = config
    norm = PartSpec("rmsnorm", {"width": c.width, "eps": c.norm_eps, "leaf": ""})
    layers = []
    blends = False                       # whether an earlier layer blends values: the first one is the source
    for i, layer in enumerate(c.layers):
        m = layer["mixer"]
        if layer["type"] == "attention":
            mixer = PartSpec("biased_window_attention", {
                "width": c.width, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                "value_dim": m["vdim"], "scale": m["scale"], "softcap": m["softcap"], "window": m["mask"]["size"],
                "keep_first": m["mask"]["keep_first"], "bias_far": m["bias_max"], "bias_rows": m.get("bias_rows") or -1, "sink": True,
                "projection_bias": True, "output_gate": True, "value_mix": "values" if m["v_mix"] else None,
                "value_mix_source": bool(m["v_mix"]) and not blends, "names": ATTENTION_NAMES})
            blends = blends or bool(m["v_mix"])
        else:
            mixer = PartSpec("mamba2", {"width": c.width, "heads": m["heads"], "head_dim": m["vdim"], "state": m["state"],
                                        "groups": m["groups"], "conv": m["conv"], "norm_groups": m["norm_groups"],
                                        "eps": c.norm_eps, "names": SSM_NAMES})
        parts = {"norm1": norm, "mixer": mixer, "norm1b": norm}
        names = {"norm1": "norm1", "mixer": "mix", "norm1b": "norm1b"}
        if layer["mlp"] is not None:
            parts.update(norm2=norm, norm2b=norm, feed_forward=PartSpec("clamped_glu", {
                "width": c.width, "inner": layer["mlp"]["ff"], "limit": layer["mlp"]["limit"], "alpha": GLU_SIGMOID_SLOPE,
                "names": GLU_NAMES}))
            names.update(norm2="norm2", norm2b="norm2b", feed_forward="mlp")
        layers.append(LayerSpec(f"l{i}", "sandwich_norm", parts, names))
    table = {"vocab": c.vocab_size, "width": c.width}
    return ModelSpec(vocab_size=c.vocab_size, width=c.width,
                     embedding=PartSpec("token_embedding", dict(table, leaf="")), embedding_prefix="embed",
                     layers=layers, final_norm=norm, final_norm_prefix="final.norm",
                     head=PartSpec("linear_head", dict(table, tied_to="embed")), head_prefix="head")
