"""The Bolovik decoder as a model description.

A decoder-only model whose layers norm a sub-layer's result, not its input:
``x <- x + N(mixer(x))``, then ``x <- x + N(ff(x))``, with ``N`` an RMS norm over equal
consecutive parts of the vector, and whose stream between layers is a learned
weighted sum of the embedding's output and all layers' results so far.  A
layer's mixer is either ``delta`` - a gated delta rule: a matrix state per head
that is decayed, corrected towards the token's value along its key and read by
its query, behind short causal convolutions - or ``attention``: grouped-query
attention with biased projections, partial rotary positions (frequencies
rescaled in three bands of wavelength), queries, keys and values divided by
their root mean square per head, and a sliding window that also keeps the first
tokens of the sequence.  Feed-forwards are gated GELU layers or mixtures of
SiLU experts routed by sigmoid scores inside the best groups of experts; a layer
may have none.

Checkpoint names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.dwa``, ``l<i>.mix.*``
(delta: ``q, k, v, g, b, a, q.conv, k.conv, v.conv, A_log, dt_bias, norm, o``; attention:
``q, k, v`` with ``.b`` biases, ``o``), ``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.router`` and
``l<i>.mlp.e<j>.{gate, up, down}``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.bolovik import BolovikConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem
from ..registry import register_architecture


def build_bolovik_spec(cfg: BolovikConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("part_rmsnorm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "parts": cfg.norm_groups,
                                         "weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "delta":
            mixer = PartSpec("delta", {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads,
                                       "head_dim": m.dim, "vdim": m.vdim, "conv": m.conv, "eps": cfg.norm_eps,
                                       "prefix": p + "mix."})
        else:
            position = None
            if m.rot is not None and m.rot.dims > 0:
                scaling = None
                if m.rot.scaling is not None:
                    factor, low, high, original = m.rot.scaling
                    scaling = {"rope_type": "llama3", "factor": factor, "low_freq_factor": low,
                               "high_freq_factor": high, "original_max_position_embeddings": original}
                position = {"kind": "rotary", "params": {"head_dim": m.dim, "rotary_dim": m.rot.dims,
                                                         "theta": m.rot.base, "scaling": scaling}}
            mixer = PartSpec("attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "v_head_dim": m.vdim, "window": m.window, "keep_first": m.keep_first, "scale": m.scale,
                "position": position, "prefix": p + "mix.", "names": {"q": "q", "k": "k", "v": "v", "o": "o"},
                "biases": {"q": "q.b", "k": "k.b", "v": "v.b"},
                "unit_norm": {"eps": cfg.norm_eps, "value": True}})
        parts = {"norm1": norm(p + "norm1"), "mixer": mixer}
        if layer.mlp is not None:
            parts["norm2"] = norm(p + "norm2")
            if layer.mlp.kind == "dense":
                parts["ffn"] = PartSpec("swiglu", {
                    "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "prefix": p + "mlp.",
                    "names": {"gate": "gate", "up": "up", "down": "down"}, "activation": "gelu_tanh"})
            else:
                parts["ffn"] = PartSpec("moe", {
                    "hidden_size": cfg.width, "expert_size": layer.mlp.ff, "experts": layer.mlp.experts,
                    "top": layer.mlp.top, "activation": "silu", "prefix": p + "mlp.", "router_bias": None,
                    "scoring": "sigmoid", "renormalize": False,
                    "groups": {"count": layer.mlp.group_count, "keep": layer.mlp.group_keep, "top": 2}})
        layers.append(LayerSpec(block="subnorm", name=p, parts=parts,
                                params={"depth_average": p + "dwa", "depth_index": i}))
    return ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed",
                                               "act": True, "result_slots": len(cfg.layers) + 1}),
        layers=tuple(layers),
        schedule=tuple(ScheduleItem(i) for i in range(len(layers))),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head"}),
        max_position=cfg.max_position,
    )


register_architecture("Bolovik", BolovikConfig.from_dict, build_bolovik_spec)
