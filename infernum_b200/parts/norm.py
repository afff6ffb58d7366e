"""RMSNorm: ``y = x * rsqrt(mean(x^2) + eps) * w`` (the weight multiplies
directly, no ``1 + w``), sum of squares and rsqrt in 32-bit, one rounding at
the store.  Reference: infernum-cuda/kernels/rmsnorm.cu:64-94 and, fused with
the residual add, infernum-cuda/kernels/add_rmsnorm.cu:78-108.

Parameters: ``hidden_size``, ``eps``, ``weight`` (checkpoint tensor name).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..ops import core
from .base import NORMS, Norm, ResidualStream, Runtime, WeightSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.weight_name = params["weight"]
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden_size,), init="norm")}

    def bind(self, weights) -> None:
        self.weight = weights[self.weight_name].contiguous()

    def weight_bytes(self) -> int:
        return self.weight.numel() * self.weight.element_size()

    def forward(self, stream: ResidualStream, row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        residual = stream.residual
        n_out = residual.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((n_out, self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        core.add_rmsnorm(residual, stream.pending, self.weight, self.eps, out, row_idx=row_idx,
                         write_residual=row_idx is None)
        if row_idx is None:
            stream.pending = None
        return out

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        core.add_rmsnorm(x, None, self.weight, self.eps, out)
        return out


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """Layer norm with weight and optional bias, or - ``centred: False`` - an RMS
    norm through the same kernel: ``y = (s - mean(s)) / sqrt(var(s) + eps) * w + b``
    with ``var`` the mean of the squared deviations, all in 32-bit.

    Two uses.  ``forward(stream, row_idx)`` is the pre-norm / final-norm use:
    the stream's pending delta is folded into the residual and the normed rows
    are returned.  ``renorm(stream, alpha)`` is the use of layers that norm
    after the sum: the residual becomes ``norm(alpha * residual + pending)``
    (kept in float32) and ``stream.act`` its rounding to the activation dtype.

    Parameters: ``hidden_size``, ``eps``, ``weight``, ``bias`` (tensor name or
    None), ``centred`` (default True).
    """

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.weight_name = params["weight"]
        self.bias_name = params.get("bias")
        self.centred = bool(params.get("centred", True))
        self.optional = bool(params.get("optional", False))
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        specs = {self.weight_name: WeightSpec((self.hidden_size,), init="norm", optional=self.optional)}
        if self.bias_name:
            specs[self.bias_name] = WeightSpec((self.hidden_size,), init="normal", std=0.05,
                                               optional=self.optional)
        return specs

    def bind(self, weights) -> None:
        w = weights.get(self.weight_name)
        self.weight = w.contiguous() if w is not None else None
        b = weights.get(self.bias_name) if self.bias_name else None
        self.bias = b.contiguous() if b is not None else None

    @property
    def present(self) -> bool:
        """False for an optional norm whose tensors the checkpoint left out."""
        return self.weight is not None

    def weight_bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.weight, self.bias) if t is not None)

    def forward(self, stream: ResidualStream, row_idx: Optional[torch.Tensor] = None,
                read: Optional[torch.Tensor] = None) -> torch.Tensor:
        residual = stream.residual
        n_out = residual.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((n_out, self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        if residual.dim() == 3:
            # Several streams per token: the pending sub-layer result is written into
            # them, and the mixture ``sum_s read[s] x_s`` (``read`` None: their sum)
            # is normed, in one pass.  With a row gather nothing is written back, so
            # what is pending stays pending.
            mix, out_coef = stream.pending_write if stream.pending is not None else (None, None)
            core.hc_norm(residual, stream.pending, mix, out_coef, read, self.weight, self.bias, self.eps, out,
                         centred=self.centred, row_idx=row_idx)
            if row_idx is None:
                stream.pending = None
                stream.pending_write = None
            return out
        if stream.pending is not None:
            stream.flush()
        core.scale_add_norm(residual, None, self.weight, self.bias, self.eps, out, alpha=1.0,
                            centred=self.centred, store=False, row_idx=row_idx)
        return out

    def renorm(self, stream: ResidualStream, alpha: float) -> None:
        residual = stream.residual
        out = None if self.rt.is_fp32 else torch.empty(residual.shape, dtype=self.rt.dtype, device=residual.device)
        core.scale_add_norm(residual, stream.pending, self.weight, self.bias, self.eps, out, alpha=alpha,
                            centred=self.centred, store=True)
        stream.pending = None
        stream.act = residual if out is None else out

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        core.scale_add_norm(x, None, self.weight, self.bias, self.eps, out, centred=self.centred)
        return out


@NORMS.register("part_rmsnorm")
class PartRMSNorm(Norm):
    """RMS norm over ``parts`` equal consecutive parts of the vector: each part is
    divided by its own ``sqrt(mean(part^2) + eps)`` and the whole multiplied by the
    weight; 32-bit throughout.

    Two uses.  ``forward(stream, row_idx)``: the norm of the stream's rows (the
    final norm).  ``add_normed(stream, y, depth)``: for layers that norm a
    sub-layer's result, not its input: the stream becomes ``x + norm(y)`` - or,
    with ``depth = (slot, coef)``, that sum is stored as the stream's result
    ``slot`` and the stream becomes ``sum_{j <= slot} coef[j] results[j]`` - in one
    kernel, which also writes the stream's rounding to the activation dtype.

    ``add_gated(stream, y, gate, bias, mult)``: ``x + mult * norm(y * sigmoid(gate + bias))``.

    Parameters: ``hidden_size``, ``eps``, ``parts`` (default 1), ``weight``.
    """

    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.eps = float(params["eps"])
        self.parts = int(params.get("parts", 1))
        self.weight_name = params["weight"]
        self.weight: Optional[torch.Tensor] = None
        self._stored_bytes = 0

    def weight_specs(self) -> Dict[str, WeightSpec]:
        return {self.weight_name: WeightSpec((self.hidden_size,), init="norm")}

    def bind(self, weights) -> None:
        w = weights[self.weight_name]
        self._stored_bytes = w.numel() * w.element_size()
        self.weight = w.to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self._stored_bytes

    def forward(self, stream: ResidualStream, row_idx: Optional[torch.Tensor] = None) -> torch.Tensor:
        if stream.pending is not None:
            stream.flush()
        residual = stream.residual
        n_out = residual.shape[0] if row_idx is None else row_idx.numel()
        out = torch.empty((n_out, self.hidden_size), dtype=self.rt.dtype, device=residual.device)
        core.part_rmsnorm(residual, self.weight, self.parts, self.eps, out, row_idx=row_idx)
        return out

    def add_normed(self, stream: ResidualStream, y: torch.Tensor, depth=None) -> None:
        x = stream.residual
        results = stream.results if depth is not None else None
        # (the embedding's output is also result 0: it is never written over)
        aliases = stream.results is not None and x.data_ptr() == stream.results.data_ptr()
        out = torch.empty_like(x) if aliases else x
        act = None if self.rt.is_fp32 else torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        slot, coef = depth if depth is not None else (0, None)
        core.sub_norm_add(x, y, self.weight, self.parts, self.eps, out, act, results=results, slot=slot, coef=coef)
        stream.residual = out
        stream.act = out if act is None else act

    def add_gated(self, stream: ResidualStream, y: torch.Tensor, gate: Optional[torch.Tensor],
                  gate_bias: Optional[torch.Tensor], mult: float = 1.0) -> None:
        """The stream becomes ``x + mult * norm(y * sigmoid(gate + gate_bias))`` (``gate``
        None: ``norm(y)``), in place and in 32-bit; no activation copy is made."""
        if stream.pending is not None:
            stream.flush()
        x = stream.residual
        # (the embedding's output, when the stream keeps it, is never written over)
        out = torch.empty_like(x) if stream.origin is not None and stream.origin.data_ptr() == x.data_ptr() else x
        core.gated_norm_add(x, y, gate, gate_bias, self.weight, self.parts, self.eps, mult, out)
        stream.residual = out
        stream.act = None

    def apply(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=self.rt.dtype, device=x.device)
        core.part_rmsnorm(x, self.weight, self.parts, self.eps, out)
        return out

    def apply_f32(self, x: torch.Tensor) -> torch.Tensor:
        """The norm of 32-bit rows, returned in 32-bit."""
        out = torch.empty(x.shape, dtype=torch.float32, device=x.device)
        core.part_rmsnorm(x, self.weight, self.parts, self.eps, out)
        return out
