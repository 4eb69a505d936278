"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * weight, all in float32
(yalis/external/model.py:957-989), fused with the residual add before it."""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.elementwise import add_rmsnorm
from yalis_b200.ops.linear import DeferredLinear, fused_residual_supported, linear_add_to_stream
from .base import Norm, ParamSpec, ResidualStream, register_part


class RMSNorm(Norm):
    """Parameters: ``size`` (width of the stream), ``eps``.  The scale is held in float32."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.size = int(spec.params["size"])
        self.eps = float(spec.params["eps"])
        self.weight: Optional[torch.Tensor] = None
        self.applied: Optional[torch.Tensor] = None     # the scale the kernel multiplies by: the weight, or ones once folded
        self.folded = False

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((self.size,), init="ones", keep_float32=True)}

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = self.applied = tensors["weight"].contiguous()
        self.folded = False

    def foldable_weight(self) -> Optional[torch.Tensor]:
        return self.weight

    def weight_folded(self) -> None:
        self.folded = True
        self.applied = torch.ones_like(self.weight)

    def forward(self, stream: ResidualStream, rows: Optional[torch.Tensor] = None):
        pending = stream.pending
        if isinstance(pending, DeferredLinear):
            if rows is None and self.folded and fused_residual_supported(pending.x, pending.w):
                # the product, the addition to the stream and this norm's statistics in one kernel; the factor
                # of each row is applied by the product that takes the result
                stream.pending = None
                return linear_add_to_stream(pending.x, pending.w, stream.x, self.eps)
            pending = pending.compute()
        y = add_rmsnorm(stream.x, pending, self.applied, self.eps, stream.dtype, rows=rows)
        if rows is None:
            stream.pending = None   # the kernel has written x + delta back
        else:
            stream.pending = pending    # still to be added: computed now, so not computed twice
        return y

    def normalize(self, y: torch.Tensor) -> torch.Tensor:
        # the same kernel over a zero stream with y as its pending delta: float32 math, one rounding
        zero = torch.zeros(y.shape, dtype=torch.float32, device=y.device)
        return add_rmsnorm(zero, y.contiguous(), self.weight, self.eps, y.dtype)

    def capture_key(self, host):
        return None


register_part("norm", "rms_norm", RMSNorm)
