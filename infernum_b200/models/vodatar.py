"""The Vodatar decoder as a model description.

A decoder-only model whose layers norm both what a sub-layer reads and what it
returns (RMS norms over equal consecutive parts of the vector), add a short
causal convolution to what it reads, gate what it returns and scale the sum:
``x <- x + m * norm_b(gate(h) * f(h + conv(h)))`` with ``h = norm(x)``.  A layer's mixer
is ``attention`` - differential attention: two score maps per head over shared
values behind short convolutions, rotated in neighbouring pairs, soft-capped -
or ``latent_attention``: attention through a low-rank latent of keys and values
with one rotated key part shared by the heads, frequencies rescaled along a
ramp.  Feed-forwards are mixtures of SiLU experts routed by a softmax over all
router outputs, some of which hand the input on, plus an expert every token
uses behind a sigmoid gate.  A run of layers may be walked several times with
the same weights; each pass re-enters through a product over the stream and the
embedding's output.  The embedding is normed.

Checkpoint names: ``embed``, ``embed.norm``, ``loop.in``, ``loop.step``,
``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.canon1|canon2``, ``l<i>.rg1|rg2`` with ``.b``,
``l<i>.mix.*`` (attention: ``q, k, v, o, q.conv, k.conv, v.conv, lq1, lk1, lq2, lk2``;
latent_attention: ``q, dkv, dkv.norm, uk, uv, o``), ``l<i>.mlp.{router, correction,
e<j>.{gate, up, down}, shared.{gate, up, down, sg}}``, ``final.norm``, ``head``.
"""

from __future__ import annotations

from ..config.vodatar import VodatarConfig
from ..parts.base import LayerSpec, ModelSpec, PartSpec, ScheduleItem
from ..registry import register_architecture


def _scaling(rot):
    if rot.scaling is None:
        return None
    s = rot.scaling
    return {"rope_type": "ramp", "factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}


def build_vodatar_spec(cfg: VodatarConfig) -> ModelSpec:
    def norm(name: str) -> PartSpec:
        return PartSpec("part_rmsnorm", {"hidden_size": cfg.width, "eps": cfg.norm_eps, "parts": cfg.norm_groups,
                                         "weight": name})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        if layer.type == "attention":
            mixer = PartSpec("diff_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "dim": m.dim,
                "vdim": m.vdim, "scale": m.scale, "softcap": m.softcap, "diff": m.diff, "conv": m.conv,
                "eps": cfg.norm_eps, "prefix": p + "mix.",
                "rotary": {"dims": m.rot.dims, "theta": m.rot.base, "scaling": _scaling(m.rot)}})
        else:
            mixer = PartSpec("latent_attention", {
                "hidden_size": cfg.width, "num_heads": m.heads, "dim": m.dim, "rot_dim": m.rot_dim, "vdim": m.vdim,
                "q_rank": 0, "kv_rank": m.kv_rank, "scale": m.scale, "window": 0, "eps": cfg.norm_eps,
                "rotary_dim": m.rot.dims, "theta": m.rot.base, "rotary_scaling": _scaling(m.rot),
                "rotary_pairing": "adjacent", "prefix": p + "mix."})
        parts = {"norm1": norm(p + "norm1"), "norm1b": norm(p + "norm1b"), "mixer": mixer}
        if layer.mlp is not None:
            f = layer.mlp
            parts["norm2"], parts["norm2b"] = norm(p + "norm2"), norm(p + "norm2b")
            parts["ffn"] = PartSpec("moe", {
                "hidden_size": cfg.width, "expert_size": f.ff, "experts": f.experts, "top": f.top,
                "activation": "silu", "prefix": p + "mlp.", "router_bias": None, "scoring": "softmax_all",
                "identity": f.identity, "correction": "correction",
                "shared": {"size": f.shared_ff, "prefix": "shared.", "gate": "sg"} if f.shared_ff else None})
        layers.append(LayerSpec(block="sandwich", name=p, parts=parts, params={
            "hidden_size": cfg.width, "mult": cfg.residual_mult,
            "canon": {"taps": cfg.canon_taps, "names": (p + "canon1", p + "canon2")} if cfg.canon_taps else None,
            "gates": {"names": (p + "rg1", p + "rg2")}}))

    L = len(layers)
    schedule, entry = [ScheduleItem(i) for i in range(L)], None
    if cfg.loop is not None:
        start, stop, times = cfg.loop
        schedule = [ScheduleItem(i) for i in range(start)]
        for t in range(times):
            schedule += [ScheduleItem(i, enter=t if i == start else None) for i in range(start, stop)]
        schedule += [ScheduleItem(i) for i in range(stop, L)]
        entry = PartSpec("concat_reentry", {"hidden_size": cfg.width, "passes": times, "weight": "loop.in",
                                            "step": "loop.step"})
    return ModelSpec(
        hidden_size=cfg.width,
        vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {
            "vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "embed", "keep_origin": entry is not None,
            "norm": {"kind": "part_rmsnorm", "params": {"hidden_size": cfg.width, "eps": cfg.norm_eps,
                                                        "parts": cfg.norm_groups, "weight": "embed.norm"}}}),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=norm("final.norm"),
        lm_head=PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "weight": "head"}),
        max_position=cfg.max_position,
        pass_entry=entry,
    )


register_architecture("Vodatar", VodatarConfig.from_dict, build_vodatar_spec)
