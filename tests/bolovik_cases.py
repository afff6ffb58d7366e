"""Small Bolovik configurations for the tests and their model folders."""

from __future__ import annotations

import os
from typing import Optional

import torch


def delta(heads, kv_heads, dim, vdim, conv, mlp=None):
    return {"type": "delta", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv},
            "mlp": mlp}


def attention(heads, kv_heads, dim, vdim, scale, window=None, keep_first=None, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


DENSE = lambda ff: {"kind": "dense", "ff": ff}  # noqa: E731


def moe(ff, experts, top, groups=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    return {"kind": "moe", "expert": {"ff": ff}, "router": router}


# Three norm parts; every mixer and feed-forward kind; grouped heads; values narrower and wider
# than keys; a window that is no multiple of a page, with kept first tokens that end inside a
# page; all three bands of the frequency scaling; a layer without a feed-forward.
CASE_A = {
    "architecture": "Bolovik", "vocab": 211, "width": 96, "norm": {"eps": 1e-5, "groups": 3},
    "layers": [
        delta(4, 2, 16, 24, 4, DENSE(72)),
        attention(6, 2, 16, 8, 0.35, 21, 5, rot(8, 10000.0, (8.0, 1.0, 4.0, 64)), moe(40, 8, 3, (4, 2))),
        delta(2, 2, 20, 12, 3, None),
        attention(4, 4, 8, 20, 0.5, 10, 3, rot(8, 100.0), moe(24, 6, 2, (2, 1))),
        delta(6, 3, 8, 16, 2, moe(16, 5, 2)),
    ],
}
# Values that are 1 or equal, and keys that a model may leave out: one norm part; one head; as
# many key heads as heads; convolutions of one tap and none; a window of one token; kept first
# tokens that outnumber the window; no mask; no rotation, and one over the whole head; one expert
# of one chosen, all experts chosen, one group; sizes that are no multiple of 8.
CASE_B = {
    "architecture": "Bolovik", "vocab": 130, "width": 72, "norm": {"eps": 1e-6},
    "layers": [
        attention(1, 1, 12, 12, 0.4, 1, 4, rot(12, 50.0), DENSE(40)),
        delta(1, 1, 28, 10, 1, moe(20, 1, 1)),
        attention(3, 3, 10, 6, 0.3, None, None, None, moe(12, 3, 3, (1, 1))),
        {"type": "delta", "mixer": {"heads": 2, "dim": 12}, "mlp": None},
        attention(2, 1, 6, 14, 0.6, 6, 9, rot(2, 7.0, (2.0, 1.0, 2.0, 16)), None),
        attention(2, 2, 8, 8, 0.5, 7, 0, None, DENSE(36)),
    ],
}
# Sizes the tensor-core kernels take (head sizes that are multiples of 16, keys and values
# alike, pages of 16): a window without kept tokens, one with them, attention without a mask; a
# delta rule with 128 state rows.
CASE_C = {
    "architecture": "Bolovik", "vocab": 384, "width": 128, "norm": {"eps": 1e-6, "groups": 2},
    "layers": [
        attention(8, 2, 32, 32, 0.2, 45, None, rot(16, 10000.0), DENSE(192)),
        delta(4, 2, 64, 32, 4, moe(64, 8, 2, (4, 2))),
        attention(4, 4, 64, 64, 0.15, 40, 17, rot(64, 250000.0, (3.0, 1.0, 5.0, 128)), None),
        delta(2, 1, 128, 16, 3, DENSE(96)),
        attention(4, 1, 64, 64, 0.15, None, None, rot(32, 10000.0), moe(32, 4, 2)),
    ],
}
# One layer of each mixer alone, without feed-forwards: what the mixers and the depth average do.
CASE_D = {
    "architecture": "Bolovik", "vocab": 97, "width": 64, "norm": {"eps": 1e-5, "groups": 4},
    "layers": [delta(2, 1, 32, 24, 3, None), attention(4, 2, 16, 12, 0.3, 9, 2, rot(8, 1000.0), None)],
}
# Models of one kind of mixer only: delta layers alone use no pages, attention layers alone no
# state slots; attention as the first layer; all experts chosen, without groups.
CASE_E = {
    "architecture": "Bolovik", "vocab": 101, "width": 48, "norm": {"eps": 1e-5, "groups": 2},
    "layers": [delta(2, 2, 16, 16, 2, DENSE(40)), delta(4, 1, 8, 8, 4, moe(16, 4, 2, (2, 2))),
               delta(3, 3, 16, 8, 3, None)],
}
CASE_F = {
    "architecture": "Bolovik", "vocab": 89, "width": 64, "norm": {"eps": 1e-5, "groups": 1},
    "layers": [attention(4, 2, 16, 16, 0.25, 12, 2, rot(16, 1000.0), DENSE(64)),
               attention(2, 2, 32, 32, 0.2, None, None, rot(16, 10000.0, (4.0, 1.0, 4.0, 32)), None),
               attention(4, 1, 16, 16, 0.3, 5, None, None, moe(24, 4, 4))],
}


def random_case(seed: int) -> dict:
    """A configuration drawn at random from sizes a small model might have: widths, part counts,
    layer orders, head counts and sizes (values narrower or wider than keys), taps, windows with
    and without kept tokens, rotation over none, part or all of a head with and without rescaled
    frequencies, experts with and without groups, layers without a feed-forward."""
    import random
    rng = random.Random(seed)
    width = rng.choice([128, 192, 256, 320, 384])
    parts = rng.choice([g for g in (1, 2, 4, 8) if width % g == 0])
    layers = []
    for _ in range(rng.randint(3, 6)):
        r = rng.random()
        if r < 0.2:
            mlp = None
        elif r < 0.55:
            mlp = DENSE(rng.choice([128, 200, 256]))
        else:
            experts = rng.choice([4, 6, 8, 12, 16])
            count = rng.choice([g for g in (1, 2, 3, 4) if experts % g == 0])
            keep = rng.randint(1, count)
            if rng.random() < 0.8:
                mlp = moe(rng.choice([32, 64, 96]), experts, rng.randint(1, min(keep * (experts // count), 6)),
                          (count, keep))
            else:
                mlp = moe(rng.choice([32, 64, 96]), experts, rng.randint(1, min(experts, 6)))
        if rng.random() < 0.5:
            heads = rng.choice([2, 4, 6, 8])
            kv = rng.choice([h for h in (1, 2, 3, 4, 8) if heads % h == 0])
            dim = rng.choice([32, 48, 64, 96, 128])
            layers.append(delta(heads, kv, dim, rng.choice([32, 64, 128, dim]), rng.choice([2, 3, 4, 5]), mlp))
        else:
            heads = rng.choice([2, 4, 8, 16])
            kv = rng.choice([h for h in (1, 2, 4, 8) if heads % h == 0])
            dim = rng.choice([32, 64, 96, 128])
            window = rng.choice([None, 32, 48, 64, 100, 128])
            keep_first = rng.choice([None, 0, 1, 4, 16, 20, 33]) if window else None
            rd = rng.choice([0, dim // 4, dim // 2, dim])
            scaling = rng.choice([None, (4.0, 1.0, 4.0, 512), (8.0, 1.0, 4.0, 256), (2.0, 2.0, 8.0, 64)])
            layers.append(attention(heads, kv, dim, rng.choice([dim, dim, 32, 64]), rng.choice([dim ** -0.5, 0.1, 0.2]),
                                    window, keep_first, rot(rd, rng.choice([100.0, 10000.0, 250000.0]), scaling) if rd else None,
                                    mlp))
    return {"architecture": "Bolovik", "vocab": rng.choice([300, 512, 777, 1000]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6]), "groups": parts}, "layers": layers}


CASES = {"A": CASE_A, "B": CASE_B, "C": CASE_C, "D": CASE_D, "E": CASE_E, "F": CASE_F}
PAGE_SIZES = {"A": 4, "B": 8, "C": 16, "D": 4, "E": 8, "F": 16}


def make_folder(folder: str, config: dict, seed: int, sharpen: float = 0.0, drop: Optional[list] = None,
                gain: float = 1.0) -> str:
    """A random model through the package's writer, reshaped so that faults show: slow
    decays (a state lost or mixed up matters many tokens later), write strengths and decays
    that vary with the token, projections large beside their biases, router logits of order
    one, and a depth average that mostly hands on the newest result.  ``sharpen`` multiplies the attention layers'
    ``scale`` so that the softmax is peaked and one wrong key shows in the logits (queries
    and keys are normed, so scaling a projection would not).  ``gain`` below 1 scales the
    projections up less (1 + gain (factor - 1)): their results' rounding is scaled with them."""
    import json

    from infernum_b200.weights.random_init import write_random_model
    from safetensors.torch import load_file, save_file

    if sharpen:
        config = json.loads(json.dumps(config))
        for layer in config["layers"]:
            if layer["type"] == "attention":
                layer["mixer"]["scale"] = layer["mixer"]["scale"] * sharpen
    write_random_model(folder, config, seed)
    path = os.path.join(folder, "model.safetensors")
    tensors = load_file(path)
    for name in list(tensors):
        t = tensors[name].float()
        if name.endswith(".A_log"):
            t = t - 2.5
        elif name.endswith((".mix.a", ".mix.b")):
            t = t * (1.0 + gain * 19.0)
        elif name.endswith((".mix.q", ".mix.k", ".mix.v", ".mix.g", ".gate", ".up", "embed")):
            t = t * (1.0 + gain * 5.0)
        elif name.endswith(".dwa"):
            t[-1] += 1.0
        elif name.endswith(".router"):
            t = t * (2.0 / t.shape[1] ** 0.5)  # logits of order one: scores that are not saturated
        else:
            continue
        tensors[name] = t.to(torch.bfloat16)
    for name in drop or []:
        del tensors[name]
    save_file(tensors, path, metadata={"format": "pt"})
    return folder
