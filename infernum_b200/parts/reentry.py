"""What happens to the stream where a model begins a pass through a run of
layers that it walks several times with the same weights.

``concat_reentry``: before pass t the stream becomes ``W [x ; x0] + s_t``, with
``x`` the stream as it arrives, ``x0`` the embedding's output (kept by the
embedding in ``stream.origin``), ``W`` [hidden, 2 hidden] and ``s`` [passes,
hidden] a learned vector per pass.  The product reads both streams rounded to
the activation dtype and returns 32-bit, which is the new stream; the vector
is added in 32-bit.

Parameters: ``hidden_size``, ``passes``, ``weight``, ``step`` (tensor names).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from ..errors import ConfigError
from ..ops import core
from .base import ENTRIES, Part, ResidualStream, Runtime, WeightSpec
from .linear import Linear


@ENTRIES.register("concat_reentry")
class ConcatReentry(Part):
    def __init__(self, params, rt: Runtime):
        super().__init__(params, rt)
        self.hidden_size = int(params["hidden_size"])
        self.passes = int(params["passes"])
        self.weight_name = params["weight"]
        self.step_name = params["step"]
        self.proj: Optional[Linear] = None
        self.step: Optional[torch.Tensor] = None

    def weight_specs(self) -> Dict[str, WeightSpec]:
        h = self.hidden_size
        return {self.weight_name: WeightSpec((h, 2 * h), std=0.7 / (2 * h) ** 0.5 * 1.4),
                self.step_name: WeightSpec((self.passes, h), std=0.1)}

    def bind(self, weights) -> None:
        self.proj = Linear(weights[self.weight_name], self.rt)
        self.step = weights[self.step_name].to(torch.float32).contiguous()

    def weight_bytes(self) -> int:
        return self.proj.nbytes

    def forward(self, stream: ResidualStream, number: int) -> None:
        if stream.origin is None:
            raise ConfigError("a pass entry needs the embedding's output (the embedding keeps none)")
        if not 0 <= number < self.passes:
            raise ConfigError(f"pass {number} is outside the {self.passes} the model has")
        stream.flush()
        x = stream.residual
        both = torch.empty((x.shape[0], 2 * self.hidden_size), dtype=self.rt.dtype, device=x.device)
        core.concat_round(x, stream.origin, both)
        out = self.proj(both, out_dtype=torch.float32)
        core.add_row(out, self.step[number])
        stream.residual = out
        stream.act = None
