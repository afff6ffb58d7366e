"""Block arrangements.

``prenorm``: the Llama layer (infernum-llama/src/graph_builder.rs:451-507):
``h += mixer(norm1(h))``; ``h += ffn(norm2(h))``.  The two adds are not done
here: each output is pushed on the residual stream as a pending delta and the
next norm kernel folds it in (the reference's optimizer fuses add + rms_norm
the same way, infernum/src/graph/optimizer.rs:105-174).

Parts of a ``prenorm`` layer: ``norm1``, ``mixer``, and - unless the layer has no
feed-forward - ``norm2``, ``ffn``.

``hyper_prenorm``: the same two sub-layers over several residual streams per
token.  Sub-layer q reads ``u = sum_s in_q[s] x_s``, computes ``y = f(norm_q(u))``
and writes ``x_t <- sum_s mix_q[s, t] x_s + out_q[t] y`` into all streams at
once (``mix`` is indexed [from, to]).  The write is not done here either: it is
pushed on the stream with its coefficients, and the next read-and-norm kernel
does write, read and norm in one pass over the row.

``subnorm``: the norm sits on the sub-layer's result: ``x <- x + norm1(mixer(x))``,
then ``x <- x + norm2(ffn(x))``; the sub-layers read the stream itself.  With
``depth_average`` the layer's result is kept and what goes on is a weighted sum
of the embedding's output and all layers' results so far.
"""

from __future__ import annotations

from ..errors import ConfigError
import torch

from .base import BLOCKS, Block, ResidualStream, WeightSpec


@BLOCKS.register("prenorm")
class PreNormBlock(Block):
    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        missing = [r for r in ("norm1", "mixer") if r not in parts]
        if "ffn" in parts and "norm2" not in parts:
            missing.append("norm2")
        if missing:
            raise ConfigError(f"prenorm block {params.get('name', '')!r} lacks parts {missing}")

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        stream.push(p["mixer"].forward(p["norm1"].forward(stream), ctx, cache))
        if "ffn" in p:
            stream.push(p["ffn"].forward(p["norm2"].forward(stream), ctx))


@BLOCKS.register("hyper_prenorm")
class HyperPreNormBlock(Block):
    """Parameters: ``streams``, ``prefix`` (the layer's), ``names`` (default
    ``hc1`` / ``hc2``: the coefficient tensors are ``<prefix><name>.in`` [S],
    ``.out`` [S], ``.mix`` [S, S]).  Parts as ``prenorm``; the norms must take a
    ``read`` mixture (``layernorm`` does)."""

    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        self.streams = int(params["streams"])
        self.prefix = params.get("prefix", params.get("name", ""))
        names = params.get("names") or ("hc1", "hc2")
        missing = [r for r in ("norm1", "mixer") if r not in parts]
        if "ffn" in parts and "norm2" not in parts:
            missing.append("norm2")
        if missing:
            raise ConfigError(f"hyper_prenorm block {params.get('name', '')!r} lacks parts {missing}")
        self.subs = [(self.prefix + names[0], "norm1", "mixer")]
        if "ffn" in parts:
            self.subs.append((self.prefix + names[1], "norm2", "ffn"))
        self.coef = {}

    def weight_specs(self):
        specs = super().weight_specs()
        S = self.streams
        for name, _, _ in self.subs:
            specs[name + ".in"] = WeightSpec((S,), init="norm")
            specs[name + ".out"] = WeightSpec((S,), init="norm")
            specs[name + ".mix"] = WeightSpec((S, S), init="normal", std=0.3)
        return specs

    def bind(self, weights) -> None:
        super().bind(weights)
        for name, _, _ in self.subs:
            self.coef[name] = tuple(weights[name + k].to(torch.float32).contiguous().view(-1)
                                    for k in (".in", ".mix", ".out"))

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        if stream.residual.dim() != 3 or stream.residual.shape[1] != self.streams:
            raise ConfigError(f"hyper_prenorm block: the stream does not carry {self.streams} copies")
        for name, norm, role in self.subs:
            read, mix, out_coef = self.coef[name]
            h = self.parts[norm].forward(stream, read=read)
            y = self.parts[role].forward(h, ctx, cache) if role == "mixer" else self.parts[role].forward(h, ctx)
            stream.push(y, write=(mix, out_coef))


@BLOCKS.register("postnorm")
class PostNormBlock(Block):
    """Norm after the sum: ``h <- norm1(alpha * h + mixer(h))`` and then
    ``h <- norm2(alpha * h + ffn(h))``.  The sub-layers read the stream itself
    (``stream.act``, its rounding to the activation dtype); the normed sum is the
    new stream, kept in float32.  A layer without a feed-forward has no ``ffn``
    part; its ``norm2``, when the checkpoint holds one, norms ``alpha * h``.

    Parameters: ``alpha`` (default 1).  Parts: ``norm1``, ``mixer``, and
    optionally ``ffn`` and ``norm2``; the norms must offer ``renorm``.
    """

    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        self.alpha = float(params.get("alpha", 1.0))
        missing = [r for r in ("norm1", "mixer") if r not in parts]
        if "ffn" in parts and "norm2" not in parts:
            missing.append("norm2")
        if missing:
            raise ConfigError(f"postnorm block {params.get('name', '')!r} lacks parts {missing}")
        for role in ("norm1", "norm2"):
            if role in parts and not hasattr(parts[role], "renorm"):
                raise ConfigError(f"postnorm block: the {parts[role].kind!r} norm cannot norm a stream in place")

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        if stream.act is None:
            raise ConfigError("postnorm block: the stream carries no activation copy (wrong embedding?)")
        stream.push(p["mixer"].forward(stream.act, ctx, cache))
        p["norm1"].renorm(stream, self.alpha)
        ffn, norm2 = p.get("ffn"), p.get("norm2")
        if ffn is not None:
            stream.push(ffn.forward(stream.act, ctx))
            norm2.renorm(stream, self.alpha)
        elif norm2 is not None and getattr(norm2, "present", True):
            norm2.renorm(stream, self.alpha)


@BLOCKS.register("subnorm")
class SubNormBlock(Block):
    """``x <- x + norm1(mixer(x))`` and then ``x <- x + norm2(ffn(x))``: the sub-layers
    read the stream itself (``stream.act``, its rounding to the activation dtype),
    and their results are normed before they are added, in 32-bit.  The norms must
    offer ``add_normed`` (``part_rmsnorm`` does).

    Parameters: ``depth_average`` (a tensor name or None) and ``depth_index`` i:
    with X_0 the embedding's output and X_(j+1) the result of layer j, the stream
    after this layer is ``sum_{j <= i + 1} w[j] X_j``, ``w`` the named tensor of
    i + 2 values.  The sum is taken by the kernel of the layer's last norm.  The
    embedding must then keep room for the results (``result_slots``).
    Parts: ``norm1``, ``mixer``, and optionally ``ffn`` with ``norm2``.
    """

    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        missing = [r for r in ("norm1", "mixer") if r not in parts]
        if "ffn" in parts and "norm2" not in parts:
            missing.append("norm2")
        if missing:
            raise ConfigError(f"subnorm block {params.get('name', '')!r} lacks parts {missing}")
        for role in ("norm1", "norm2"):
            if role in parts and not hasattr(parts[role], "add_normed"):
                raise ConfigError(f"subnorm block: the {parts[role].kind!r} norm cannot norm a sub-layer's result")
        self.depth_name = params.get("depth_average")
        self.depth_index = int(params.get("depth_index", 0))
        self.depth_coef = None

    def weight_specs(self):
        specs = super().weight_specs()
        if self.depth_name:
            specs[self.depth_name] = WeightSpec((self.depth_index + 2,), init="normal", std=0.3)
        return specs

    def bind(self, weights) -> None:
        super().bind(weights)
        if self.depth_name:
            self.depth_coef = weights[self.depth_name].to(torch.float32).contiguous()

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        if stream.act is None:
            raise ConfigError("subnorm block: the stream carries no activation copy (wrong embedding?)")
        depth = None
        if self.depth_coef is not None:
            if stream.results is None or stream.results.shape[0] < self.depth_index + 2:
                raise ConfigError("subnorm block: the stream keeps no room for the layers' results")
            depth = (self.depth_index + 1, self.depth_coef)
        ffn = p.get("ffn")
        y = p["mixer"].forward(stream.act, ctx, cache)
        p["norm1"].add_normed(stream, y, depth if ffn is None else None)
        if ffn is not None:
            p["norm2"].add_normed(stream, ffn.forward(stream.act, ctx), depth)
