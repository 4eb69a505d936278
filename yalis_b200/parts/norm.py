"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, all in float32
(yalis/external/model.py:957-989), fused with the residual add before it."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import add_rmsnorm
from .base import Norm, ParamSpec, ResidualStream, register_part


class RMSNorm(Norm):
    """Parameters: ``size`` (width of the stream), ``eps``.  The scale is held in float32."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), init="ones", keep_float32=True)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors["weight"].contiguous()

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        y = add_rmsnorm(stream.x, stream.pending, self.weight, self.eps, stream.dtype, rows=rows)
        if rows is None:
            stream.pending = None   # the kernel has written x + delta back
        return y

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        # the same kernel over a zero stream with y as its pending delta: float32 math, one rounding
        zero = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
        return add_rmsnorm(zero, y.contiguous(), self.weight, self.eps, y.dtype)

    def capture_key(self, host):
        return None


register_part("norm", "rms_norm", RMSNorm)
