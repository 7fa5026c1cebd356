"""Routed feed-forward (mixture of experts).

    z = W_r x (float32)      s = sigmoid(z) or softmax(z)      the top_k largest s are chosen
    y = sum over chosen e of  s_e * expert_e(x)      or, with scale_input,  expert_e(s_e * x)
    expert(u) = W_down (silu(W_gate u) * (W_up u))

The step's (token, choice) rows are regrouped by expert on the device (``csrc/moe.cu``): each expert's
rows form a stretch padded to whole tiles, two grouped matrix products run over the tiles (the first
with the gate's activation in its epilogue; bfloat16: tcgen05 tensor cores, ``csrc/moe_tc.cu``; float32,
and sizes that kernel does not take: CUDA cores), and one kernel sums each token's rows back in the order of
its choices, so a token's result does not depend on what else is in the batch.  Nothing is read back to
the host, so a decode step can be captured in a CUDA graph.

The experts' weights are three stacked tensors [E, F, H], [E, F, H], [E, H, F] made at load.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FeedForward, ParamSpec, register_ffn
from .linear import Linear


class RoutedFFN(FeedForward):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.E, self.top, self.F = int(spec.num_experts), int(spec.top_k), int(spec.expert_size)
        if not 0 < self.top <= self.E:
            raise ValueError(f"top_k {self.top} must be in 1..{self.E}")
        if spec.score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {spec.score!r}")
        self.softmax = spec.score == "softmax"
        self.renormalize, self.scale_input = bool(spec.renormalize), bool(spec.scale_input)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.router_name = spec.router_name
        self.stem, self.gate_name, self.up_name, self.down_name = spec.expert_names
        self.router: Linear = None
        self.w_gate = self.w_up = self.w_down = self.w_gate_up = None
        self.tc = False
        self._post_gain = None

    def _expert(self, e: int, which: str) -> str:
        return self.stem.format(e=e) + which

    def param_specs(self) -> List[ParamSpec]:
        H, F = self.hidden_size, self.F
        specs = [ParamSpec(self.router_name, (self.E, H))]
        for e in range(self.E):
            specs += [ParamSpec(self._expert(e, self.gate_name), (F, H)), ParamSpec(self._expert(e, self.up_name), (F, H)),
                      ParamSpec(self._expert(e, self.down_name), (H, F))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.router = Linear(tensors[self.router_name])
        stack = lambda which: torch.stack([tensors[self._expert(e, which)] for e in range(self.E)]).contiguous()
        self.w_down = stack(self.down_name)
        self.tc = (self.w_down.dtype == torch.bfloat16 and self.w_down.is_cuda
                   and ops.moe_gemm_tc_supports(self.hidden_size, self.F))
        if self.tc:   # one gate/up tensor whose rows alternate in blocks of 16: the activation runs in the product's epilogue
            self.w_gate_up = torch.stack([ops.interleave_gate_up(tensors[self._expert(e, self.gate_name)],
                                                                 tensors[self._expert(e, self.up_name)])
                                          for e in range(self.E)]).contiguous()
        else:
            self.w_gate, self.w_up = stack(self.gate_name), stack(self.up_name)

    def _experts(self, x):
        """(rows' results float32 [rows, H], place of every (token, choice), weights)"""
        logits = self.router(x, out_dtype=torch.float32)      # float32 sums of exact products
        tile = ops.moe_tc_tile_rows() if self.tc else ops.moe_tile_rows()
        if x.shape[0] * self.top <= ops.MOE_FUSED_FRONT_MAX_ROWS:     # few tokens (a decode step): one kernel
            wt, pos_of, tile_expert, xs = ops.moe_route_plan_scatter(logits, x, self.top, tile, self.softmax,
                                                                     self.renormalize, self.scale_input)
        else:
            sel, wt = ops.moe_route(logits, self.top, self.softmax, self.renormalize)
            pos_of, tile_expert = ops.moe_plan(sel, self.E, tile)
            xs = ops.moe_scatter(x, pos_of, wt, tile_expert.numel() * tile, self.scale_input)
        if self.tc:
            a = ops.moe_gemm_tc(xs, self.w_gate_up, tile_expert, gated=True)
            y = ops.moe_gemm_tc(a, self.w_down, tile_expert, out_dtype=torch.float32)
        else:
            a = ops.moe_gemm(xs, self.w_gate, tile_expert, w2=self.w_up)
            y = ops.moe_gemm(a, self.w_down, tile_expert, out_dtype=torch.float32)
        return y, pos_of, wt

    def forward(self, x, residual, batch, accumulate: bool = True) -> None:
        y, pos_of, wt = self._experts(x)
        ops.moe_combine(y, pos_of, wt, residual, not self.scale_input, "add" if accumulate else "write")

    def forward_post(self, x, residual, batch, post_norm) -> None:
        """``residual += post_norm(ffn(x))``, the norm inside the kernel that sums the experts' rows."""
        if self._post_gain is None or self._post_gain[0] is not post_norm.weight:
            self._post_gain = (post_norm.weight, post_norm.weight.float().contiguous())   # the kernel reads a float32 gain
        y, pos_of, wt = self._experts(x)
        ops.moe_combine(y, pos_of, wt, residual, not self.scale_input, "norm_add", self._post_gain[1], post_norm.eps)


register_ffn("routed_ffn", RoutedFFN)
