"""Dense SwiGLU feed-forward: down(silu(gate(x)) * up(x)) (yalis/external/model.py:710-744).

gate and up are stored as one matrix [Wgate; Wup] so that one product feeds the
activation kernel (the reference interleaves their rows instead, model.py:741).
"""

from __future__ import annotations

from typing import Dict, Optional

import torch

from yalis_b200.config.spec import PartSpec
from yalis_b200.ops.linear import linear_partial, linear_silu_mul
from .base import FeedForward, ParamSpec, register_part


class SwiGLU(FeedForward):
    """Parameters: ``hidden_size``, ``intermediate_size``."""

    def __init__(self, spec: PartSpec):
        super().__init__(spec)
        self.hidden = int(spec.params["hidden_size"])
        self.inter = int(spec.params["intermediate_size"])
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {
            "gate_proj": ParamSpec((self.inter, self.hidden)),
            "up_proj": ParamSpec((self.inter, self.hidden)),
            "down_proj": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_gate_up = torch.cat([tensors["gate_proj"], tensors["up_proj"]], dim=0).contiguous()
        self.w_down = tensors["down_proj"].contiguous()

    def forward(self, x: torch.Tensor, ctx) -> torch.Tensor:
        return linear_partial(linear_silu_mul(x, self.w_gate_up), self.w_down)

    def capture_key(self, host):
        return None


register_part("feed_forward", "swiglu", SwiGLU)
