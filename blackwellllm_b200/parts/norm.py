"""RMSNorm: y = x * rsqrt(mean(x^2) + eps) * w, the sum and the scaling in float32.

Formula of the reference: src/kernels/rmsnorm.cu:107-120,133-138 (it sums in
double and rounds twice through bfloat16; here: one float32 computation and one
rounding on store).  ``rows`` normalises only the named rows (final norm on the
positions whose logits are wanted, src/core/engine.cpp:1029-1035).  With the spec's ``offset`` the gain is
``offset + w`` (a weight stored around zero with offset 1), made once at load in float32.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import BuildContext, Norm, ParamSpec, register_norm


class RMSNorm(Norm):
    adds_pending = True

    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.eps = float(spec.eps)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.param = getattr(spec, "param", "weight")
        self.offset = float(getattr(spec, "offset", 0.0))
        self.weight: Optional[torch.Tensor] = None
        self._gain_f32: Optional[torch.Tensor] = None

    def param_specs(self) -> List[ParamSpec]:
        return [ParamSpec(self.param, (self.hidden_size,), role="gain", init="ones" if self.offset == 0.0 else "bias_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.param]
        if self.offset != 0.0:
            w = w.float() + self.offset     # the gain itself, float32
        self.weight = w.contiguous()
        self._gain_f32 = None

    def gain_f32(self) -> torch.Tensor:
        """The gain as a float32 vector (for kernels that norm inside another pass over the row)."""
        if self._gain_f32 is None:
            self._gain_f32 = self.weight.float().contiguous()
        return self._gain_f32

    def add_to(self, x: torch.Tensor, stream: torch.Tensor) -> None:
        """``stream += norm(x)`` (float32 both): the norm of a sublayer's output on its way into the stream."""
        ops.rmsnorm_add(x, self.weight, self.eps, stream)

    def add_to_then(self, x: torch.Tensor, stream: torch.Tensor, then: "Norm") -> torch.Tensor:
        """``stream += norm(x)``, then ``then.forward(stream)``: one kernel when ``then`` is an RMS norm too."""
        if type(then) is RMSNorm and then.weight.dtype == self.weight.dtype:
            return ops.rmsnorm_add_norm(x, self.weight, self.eps, stream, then.weight, then.eps, self.ctx.dtype)
        self.add_to(x, stream)
        return then.forward(stream)

    def forward(self, x: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        return ops.rmsnorm(x, self.weight, self.eps, self.ctx.dtype, rows=rows)


register_norm("rmsnorm", RMSNorm)
