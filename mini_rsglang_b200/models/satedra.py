"""Satedra as a composition of parts: every layer is a "pre_norm" block (layer norms with bias) around a
"latent_attention" mixer and, where the layer has one, a feed-forward: "swiglu" for a dense layer, "routed_experts"
(with a "swiglu" as the shared expert) for a mixture.  Sizes and constants come from the configuration, layer by
layer; the tensor names are the checkpoint's: `embed`, `final.norm` (+ `.b`), `head`, and below `l<i>.` the norms
`norm1`, `norm2` (the weight is the norm's root, the bias its leaf `b`), `mix.*` and `mlp.*`.

A layer with `kv_from` keeps no cache: its run reads the cache of the named layer's run (`RunEntry.cache_of`), and
that layer's cache is kept for the widest window among the layers that read it.

What the design fixes: stretched ("YaRN") rotary positions whose cosines and sines grow by 0.1 ln(factor) + 1,
softmax scores in the router with a correction that steers the choice only, gated heads, a gated shared expert."""
from __future__ import annotations

from ..config.model_config import SatedraConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry

YARN_MAGNITUDE_SLOPE = 0.1

ATTENTION_NAMES = {"q": "q", "down": "dkv", "latent_norm": "dkv.norm", "up_k": "uk", "up_v": "uv", "gate": "g", "o": "o"}
UNIT_NAMES = {"gate": "gate", "up": "up", "down": "down"}
EXPERT_NAMES = dict(UNIT_NAMES, router="router", correction="correction", expert="e{}", shared="shared", shared_gate="shared.sg")


def position_spec(mixer: dict) -> PartSpec | None:
    rot = mixer["rot"]
    if not rot["dims"]:
        return None
    params = {"rotary_dim": rot["dims"], "theta": rot["base"], "magnitude_slope": YARN_MAGNITUDE_SLOPE}
    if "scaling" in rot:
        params.update(rot["scaling"])
    return PartSpec("yarn_rope", params)


def satedra_spec(config: SatedraConfig) -> ModelSpec:
    c = config
    norm = PartSpec("layernorm", {"width": c.width, "eps": c.norm_eps, "leaf": "", "bias_leaf": "b"})
    window = [(layer["mixer"].get("mask") or {}).get("size", 0) for layer in c.layers]
    kept = list(window)                  # the window that each layer's cache is kept for: the widest that reads it
    for i, layer in enumerate(c.layers):
        source = layer["mixer"].get("kv_from")
        if source is not None:
            kept[source] = 0 if not (kept[source] and window[i]) else max(kept[source], window[i])
    layers, order, ignorable = [], [], []
    for i, layer in enumerate(c.layers):
        m = layer["mixer"]
        source = m.get("kv_from")
        mixer = PartSpec("latent_attention", {
            "width": c.width, "num_heads": m["heads"], "head_dim": m["dim"], "rotary_head_dim": m["rot_dim"], "value_dim": m["vdim"],
            "latent_dim": m["kv_rank"], "scale": m["scale"], "eps": c.norm_eps, "position": position_spec(m), "window": window[i],
            "cache_window": kept[i], "shares_cache": source is not None, "output_gate": True, "names": ATTENTION_NAMES})
        parts = {"norm1": norm, "mixer": mixer}
        names = {"norm1": "norm1", "mixer": "mix"}
        mlp = layer["mlp"]
        if mlp is None:
            ignorable += [f"l{i}.norm2", f"l{i}.norm2.b"]
        else:
            if mlp["kind"] == "dense":
                unit = PartSpec("swiglu", {"width": c.width, "inner": mlp["ff"], "names": UNIT_NAMES})
            else:
                r = mlp["router"]
                shared = PartSpec("swiglu", {"width": c.width, "inner": mlp["shared"]["ff"], "names": UNIT_NAMES}) if "shared" in mlp else None
                unit = PartSpec("routed_experts", {
                    "width": c.width, "experts": r["experts"], "identity": r["identity"], "top": r["top"], "scale": r["scale"],
                    "inner": mlp["expert"]["ff"], "score": "softmax", "correction": True, "shared": shared,
                    "shared_gate": shared is not None, "names": EXPERT_NAMES})
            parts.update(norm2=norm, feed_forward=unit)
            names.update(norm2="norm2", feed_forward="mlp")
        layers.append(LayerSpec(f"l{i}", "pre_norm", parts, names))
        order.append(RunEntry(i, cache_of=source))
    table = {"vocab": c.vocab_size, "width": c.width}
    return ModelSpec(vocab_size=c.vocab_size, width=c.width,
                     embedding=PartSpec("token_embedding", dict(table, leaf="")), embedding_prefix="embed",
                     layers=layers, final_norm=norm, final_norm_prefix="final.norm",
                     head=PartSpec("linear_head", dict(table, leaf="", scale=c.logit_scale)), head_prefix="head",
                     run_order=order, ignorable_weights=tuple(ignorable))
