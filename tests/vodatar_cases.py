"""Small Vodatar configurations for the tests and their model folders."""

from __future__ import annotations

import os
from typing import Optional

import torch


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def attention(heads, kv_heads, dim, vdim, scale, softcap=None, diff=0.2, conv=None, rotation=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "diff": diff}
    if softcap is not None:
        m["softcap"] = softcap
    if conv is not None:
        m["conv"] = conv
    if rotation is not None:
        m["rot"] = rotation
    return {"type": "attention", "mixer": m, "mlp": mlp}


def latent(heads, dim, rot_dim, vdim, kv_rank, scale, rotation, mlp=None):
    return {"type": "latent_attention", "mlp": mlp,
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
                      "rot": rotation}}


def moe(ff, experts, top, identity=None, shared=None):
    router = {"experts": experts, "top": top}
    if identity is not None:
        router["identity"] = identity
    m = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        m["shared"] = {"ff": shared}
    return m


# Three norm parts; both mixers; grouped heads; values narrower and wider than a map; rotation over
# a part of a map and over all of it; frequencies on the ramp, before and behind it; outputs that hand
# the input on; a shared expert wider and narrower than an expert; a layer without a feed-forward;
# a loop that begins behind the first layer and runs three times.
CASE_A = {
    "architecture": "Vodatar", "vocab": 211, "width": 96, "residual_mult": 0.6, "norm": {"eps": 1e-5, "groups": 3},
    "canon": {"taps": 3}, "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        attention(4, 2, 16, 24, 0.3, 15.0, 0.25, 4, rot(8, 1000.0), moe(40, 6, 2, 2, 24)),
        latent(3, 16, 8, 20, 32, 0.2, rot(8, 10000.0, (4.0, 64, 8.0, 1.0)), moe(24, 5, 3, 1, 56)),
        attention(6, 3, 8, 12, 0.4, 8.0, 0.3, 3, rot(8, 100.0), None),
        latent(2, 24, 16, 8, 40, 0.15, rot(16, 500.0, (2.0, 32, 4.0, 2.0)), moe(16, 4, 2, 0, None)),
    ],
}
# Values that are 1 or equal, and keys that a model may leave out: one norm part; no loop; no
# convolutions at all; one head; as many key heads as heads; no cap on the scores; no rotation, and
# a rotation without rescaling; one expert of one chosen; every output chosen; no
# shared expert; a difference of 0; sizes that are no multiple of 8; a residual factor left out.
CASE_B = {
    "architecture": "Vodatar", "vocab": 130, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        attention(1, 1, 12, 12, 0.4, None, 0.0, None, None, moe(20, 1, 1)),
        latent(1, 10, 6, 14, 24, 0.3, rot(6, 50.0), moe(12, 3, 4, 1)),
        attention(3, 3, 10, 6, 0.3, 30.0, 0.5, 1, rot(10, 7.0), None),
        latent(3, 12, 4, 12, 20, 0.25, rot(2, 20.0, (8.0, 16, 2.0, 1.0)), moe(28, 2, 2, 2, 20)),
    ],
}
# A loop of one pass over everything, two taps, one key head for all heads, a residual factor above 1.
CASE_C = {
    "architecture": "Vodatar", "vocab": 97, "width": 64, "residual_mult": 1.3, "norm": {"eps": 1e-5, "groups": 4},
    "canon": {"taps": 2}, "loop": {"start": 0, "stop": 2, "times": 1},
    "layers": [
        latent(4, 16, 16, 16, 32, 0.2, rot(16, 10000.0, (3.0, 48, 6.0, 0.5)), moe(32, 4, 2, 1, 32)),
        attention(4, 1, 16, 16, 0.25, 12.0, 0.2, 2, rot(16, 300.0), moe(16, 8, 4, 3, 16)),
    ],
}
# Sizes the tensor-core kernels take (latent rank a multiple of 32, width of the cached vector a
# multiple of 16, expert widths multiples of 64, pages of 16), in a loop of two passes over all layers
# but the last.
CASE_D = {
    "architecture": "Vodatar", "vocab": 384, "width": 128, "residual_mult": 0.7, "norm": {"eps": 1e-6, "groups": 2},
    "canon": {"taps": 4}, "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        latent(4, 32, 32, 48, 64, 0.12, rot(32, 10000.0, (2.0, 128, 32.0, 1.0)), moe(64, 8, 3, 2, 128)),
        attention(6, 2, 48, 64, 0.15, 25.0, 0.2, 4, rot(24, 30000.0), moe(64, 8, 4, 2, 64)),
        attention(8, 2, 16, 32, 0.25, 10.0, 0.1, 3, rot(8, 5000.0), moe(64, 4, 2, 0, 64)),
    ],
}
# One layer of each mixer, no feed-forward at all: what the mixers, the convolutions and the gates do.
CASE_E = {
    "architecture": "Vodatar", "vocab": 89, "width": 48, "residual_mult": 0.8, "norm": {"eps": 1e-5, "groups": 2},
    "canon": {"taps": 5}, "loop": {"start": 0, "stop": 1, "times": 2},
    "layers": [attention(2, 1, 8, 40, 0.35, 6.0, 0.4, 5, rot(4, 40.0), None),
               latent(2, 8, 8, 24, 16, 0.3, rot(8, 90.0), None)],
}

CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 4}


def random_case(seed: int) -> dict:
    """A configuration drawn at random from sizes a small model might have: widths, part counts,
    layer orders, loops, taps, head counts and sizes, rotations with and without a ramp, routers
    with and without outputs that hand the input on, shared experts, layers without a feed-forward."""
    import random
    rng = random.Random(seed)
    width = rng.choice([128, 192, 256, 352, 384])
    parts = rng.choice([g for g in (1, 2, 4, 8) if width % g == 0])
    layers = []
    for _ in range(rng.randint(2, 5)):
        mlp = None
        if rng.random() < 0.85:
            experts = rng.choice([4, 6, 8, 12, 16])
            identity = rng.choice([None, 0, 1, 2, 3])
            mlp = moe(rng.choice([32, 64, 96]), experts, rng.randint(1, min(experts + (identity or 0), 6)), identity,
                      rng.choice([None, 64, 96, 128]))
        if rng.random() < 0.5:
            heads = rng.choice([2, 4, 6, 8])
            kv = rng.choice([h for h in (1, 2, 3, 4, 8) if heads % h == 0])
            dim = rng.choice([16, 32, 48, 64])
            rd = rng.choice([0, dim // 4 * 2, dim // 2, dim])
            layers.append(attention(heads, kv, dim, rng.choice([dim, 32, 64, 80, 128]), rng.choice([dim ** -0.5, 0.1, 0.2]),
                                    rng.choice([None, 10.0, 20.0, 50.0]), rng.choice([0.0, 0.1, 0.3, 0.5]),
                                    rng.choice([None, 1, 2, 3, 4, 5]),
                                    rot(rd, rng.choice([100.0, 10000.0, 20000.0])) if rd else None, mlp))
        else:
            rot_dim = rng.choice([8, 16, 32, 64])
            dim = rng.choice([16, 32, 64, 96])
            scaling = rng.choice([None, (2.0, 512, 32.0, 1.0), (4.0, 256, 16.0, 2.0), (8.0, 64, 8.0, 0.5)])
            layers.append(latent(rng.choice([2, 4, 6, 8]), dim, rot_dim, rng.choice([dim, 32, 80, 128]),
                                 rng.choice([32, 64, 96, 100, 128]), rng.choice([(dim + rot_dim) ** -0.5, 0.1]),
                                 rot(rng.choice([rot_dim, rot_dim // 2]), rng.choice([100.0, 10000.0, 250000.0]), scaling),
                                 mlp))
    cfg = {"architecture": "Vodatar", "vocab": rng.choice([300, 512, 777, 1000]), "width": width,
           "residual_mult": rng.choice([0.5, 0.7, 1.0]), "norm": {"eps": rng.choice([1e-5, 1e-6]), "groups": parts},
           "layers": layers}
    if rng.random() < 0.8:
        cfg["canon"] = {"taps": rng.choice([1, 2, 3, 4])}
    if rng.random() < 0.8:
        start = rng.randint(0, len(layers) - 1)
        cfg["loop"] = {"start": start, "stop": rng.randint(start + 1, len(layers)), "times": rng.randint(1, 3)}
    return cfg


def make_folder(folder: str, config: dict, seed: int, sharpen: float = 0.0, drop: Optional[list] = None,
                gain: float = 1.0, correction: float = 1.0) -> str:
    """A random model through the package's writer, reshaped so that faults show: projections of the
    mixers large enough that scores differ, gates that depend on their input, router logits of order
    one, a difference weight ``lam`` away from its constant.  ``sharpen`` multiplies the mixers' ``scale``
    (and lifts a cap on the scores) so that the softmax is peaked and one wrong key shows in the logits.
    ``gain`` below 1 scales the projections up less (1 + gain (factor - 1)): what rounding does to their
    results is scaled with them.  ``correction`` scales the routers' correction of the choice: large beside
    the scores it settles most choices, so that rounding before the router seldom changes one (a changed
    choice is another, equally valid, result that no tolerance on logits covers)."""
    import json

    from infernum_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file

    if sharpen:
        config = json.loads(json.dumps(config))
        for layer in config["layers"]:
            layer["mixer"]["scale"] = layer["mixer"]["scale"] * sharpen
            if layer["mixer"].get("softcap"):
                layer["mixer"]["softcap"] = layer["mixer"]["softcap"] * sharpen
    write_random_model(folder, config, seed)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith((".mix.q", ".mix.k", ".mix.v", ".mix.dkv", ".mix.uk", ".mix.uv", ".gate", ".up", ".rg1", ".rg2")):
            t = t * (1.0 + gain * 4.0)
        elif name.endswith((".lq1", ".lk1", ".lq2", ".lk2")):
            t = t * (1.0 + gain * 2.0)
        elif name.endswith(".correction") and correction != 1.0:
            t = t * correction
        elif name.endswith(".router"):
            t = t * (2.0 / t.shape[1] ** 0.5)  # logits of order one: scores that are not saturated
        else:
            continue
        tensors[name] = t.to(torch.bfloat16)
    for name in drop or []:
        del tensors[name]
    save_file(tensors, path, metadata={"format": "pt"})
    return folder
