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

``sandwich``: norms on both sides of a sub-layer and a fixed factor on the sum:
``x <- x + mult * norm1b(g1 * mixer(c1(norm1(x))))``, then the same with ``ffn``;
``c`` adds a short causal convolution of the normed rows to them, ``g`` is a
sigmoid gate computed from the normed rows.
"""

from __future__ import annotations

from ..errors import ConfigError
import torch

from ..ops import core
from .base import BLOCKS, Block, ResidualStream, StateSpec, WeightSpec
from .linear import Linear


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


@BLOCKS.register("sandwich")
class SandwichBlock(Block):
    """For sub-layer n in (1: ``mixer``, 2: ``ffn``), with ``h = norm<n>(x)``:

        u = h + conv_n(h)                     (``canon``: a causal convolution per channel over time,
                                               ``taps`` wide, no bias; zeros before the sequence)
        y = f_n(u) * sigmoid(W_gn h + b_gn)   (``gates``; the gate reads h, not u)
        x <- x + mult * norm<n>b(y)

    The sum stays 32-bit.  The last ``taps - 1`` normed rows of either sub-layer
    are the arrangement's state of a request ([2, taps - 1, hidden] floats per
    slot and scheduled run).  The norms after the sub-layers must offer
    ``add_gated`` (``part_rmsnorm`` does).

    Parameters: ``hidden_size``, ``mult`` (default 1), ``canon`` (None or {"taps",
    "names": (n1, n2)}), ``gates`` (None or {"names": (n1, n2)}: tensors ``<name>``
    [hidden, hidden] and ``<name>.b``).  Parts: ``norm1``, ``norm1b``, ``mixer`` and,
    optionally, ``norm2``, ``norm2b``, ``ffn``.
    """

    def __init__(self, params, rt, parts):
        super().__init__(params, rt, parts)
        self.hidden_size = int(params["hidden_size"])
        self.mult = float(params.get("mult", 1.0))
        need = ["norm1", "norm1b", "mixer"] + (["norm2", "norm2b"] if "ffn" in parts else [])
        missing = [r for r in need if r not in parts]
        if missing:
            raise ConfigError(f"sandwich block {params.get('name', '')!r} lacks parts {missing}")
        for role in ("norm1b", "norm2b"):
            if role in parts and not hasattr(parts[role], "add_gated"):
                raise ConfigError(f"sandwich block: the {parts[role].kind!r} norm cannot norm a gated result")
        canon = params.get("canon") or {}
        self.taps = int(canon.get("taps") or 0)
        self.canon_names = tuple(canon.get("names") or ()) if self.taps else ()
        gates = params.get("gates") or {}
        self.gate_names = tuple(gates.get("names") or ())
        self.subs = [(0, "norm1", "mixer", "norm1b")] + ([(1, "norm2", "ffn", "norm2b")] if "ffn" in parts else [])
        self.canon_w = {}
        self.gate = {}

    def state_spec(self):
        if self.taps <= 1:
            return None
        return StateSpec((2 * (self.taps - 1) * self.hidden_size,), torch.float32)

    def weight_specs(self):
        specs = super().weight_specs()
        h = self.hidden_size
        for n, _, _, _ in self.subs:
            if self.taps:
                specs[self.canon_names[n]] = WeightSpec((h, self.taps), init="normal", std=0.3)
            if self.gate_names:
                specs[self.gate_names[n]] = WeightSpec((h, h))
                specs[self.gate_names[n] + ".b"] = WeightSpec((h,), init="normal", std=0.5)
        return specs

    def bind(self, weights) -> None:
        super().bind(weights)
        for n, _, _, _ in self.subs:
            if self.taps:
                self.canon_w[n] = weights[self.canon_names[n]].to(torch.float32).contiguous()
            if self.gate_names:
                self.gate[n] = (Linear(weights[self.gate_names[n]], self.rt),
                                weights[self.gate_names[n] + ".b"].to(torch.float32).contiguous())

    def weight_bytes(self) -> int:
        return super().weight_bytes() + sum(lin.nbytes for lin, _ in self.gate.values())

    def forward(self, stream: ResidualStream, ctx, cache) -> None:
        p = self.parts
        for n, pre, role, post in self.subs:
            h = p[pre].forward(stream)
            gate = self.gate.get(n)
            g = gate[0](h) if gate is not None else None
            u = h
            if self.taps:
                state, off = cache.block_state, n * (self.taps - 1) * self.hidden_size
                u = torch.empty_like(h)
                core.causal_conv(h, self.canon_w[n], state, off, ctx, u, add_input=True)
                core.conv_state_update(h, self.taps, state, off, ctx)
            y = p[role].forward(u, ctx, cache) if role == "mixer" else p[role].forward(u, ctx)
            p[post].add_gated(stream, y, g, gate[1] if gate is not None else None, self.mult)
