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

Options of the spec: a bias per router output that enters the CHOICE only (``choice_bias``); a small constant in
the renormalising sum (``renorm_eps``); router outputs beyond the experts that stand for experts which return
their input (``identity_experts``: such a choice takes no row in the regrouping, the summing kernel adds
weight * x for it); another gated activation for the experts (``activation``, run in the first product's
epilogue like the default); and a shared expert (``shared``: a dense gated feed-forward that every token runs
through and whose result is added).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FeedForward, ParamSpec, build_ffn, register_ffn
from .linear import Linear


class RoutedFFN(FeedForward):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.E, self.top, self.F = int(spec.num_experts), int(spec.top_k), int(spec.expert_size)
        if not 0 < self.top <= self.E + int(getattr(spec, "identity_experts", 0) or 0):
            raise ValueError(f"top_k {self.top} must be in 1..{self.E} (plus the experts that return their input)")
        if spec.score not in ("sigmoid", "softmax"):
            raise ValueError(f"unknown router score {spec.score!r}")
        self.softmax = spec.score == "softmax"
        self.renormalize, self.scale_input = bool(spec.renormalize), bool(spec.scale_input)
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.router_name = spec.router_name
        self.n_identity = int(getattr(spec, "identity_experts", 0) or 0)
        if self.n_identity < 0 or self.top > self.E + self.n_identity:
            raise ValueError("identity_experts must be >= 0 and top_k at most the router's outputs")
        if self.n_identity and self.scale_input:
            raise ValueError("experts that return their input go with weights on the experts' outputs")
        self.bias_name = getattr(spec, "choice_bias", None)
        self.renorm_eps = float(getattr(spec, "renorm_eps", 0.0))
        activation = getattr(spec, "activation", "silu")
        if activation not in ops.GATED_ACTIVATIONS:
            raise ValueError(f"unknown gated activation {activation!r}; known: {sorted(ops.GATED_ACTIVATIONS)}")
        self.act = ops.GATED_ACTIVATIONS[activation]
        self.limit, self.alpha = float(getattr(spec, "act_limit", 0.0)), float(getattr(spec, "act_alpha", 1.0))
        self.shared = None
        self.shared_prefix = getattr(spec, "shared_prefix", "shared.")
        if getattr(spec, "shared", None) is not None:
            self.shared = build_ffn(spec.shared, hidden_size, ctx)
        self.bias = None
        self.stem, self.gate_name, self.up_name, self.down_name = spec.expert_names
        self.router: Linear = None
        self.w_gate = self.w_up = self.w_down = self.w_gate_up = None
        self.tc = False
        self._post_gain = None

    def _expert(self, e: int, which: str) -> str:
        return self.stem.format(e=e) + which

    def param_specs(self) -> List[ParamSpec]:
        H, F = self.hidden_size, self.F
        specs = [ParamSpec(self.router_name, (self.E + self.n_identity, H))]
        if self.bias_name:
            specs.append(ParamSpec(self.bias_name, (self.E + self.n_identity,), role="bias", init="bias_normal"))
        if self.shared is not None:
            specs += [ParamSpec(self.shared_prefix + p.name, p.shape, p.role, p.init, p.optional) for p in self.shared.param_specs()]
        for e in range(self.E):
            specs += [ParamSpec(self._expert(e, self.gate_name), (F, H)), ParamSpec(self._expert(e, self.up_name), (F, H)),
                      ParamSpec(self._expert(e, self.down_name), (H, F))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.router = Linear(tensors[self.router_name])
        if self.bias_name:
            self.bias = tensors[self.bias_name].float().contiguous()
        if self.shared is not None:
            n = len(self.shared_prefix)
            self.shared.bind({k[n:]: v for k, v in tensors.items() if k.startswith(self.shared_prefix)})
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
                                                                     self.renormalize, self.scale_input, experts=self.E,
                                                                     bias=self.bias, renorm_eps=self.renorm_eps)
        else:
            sel, wt = ops.moe_route(logits, self.top, self.softmax, self.renormalize, self.bias, self.renorm_eps)
            pos_of, tile_expert = ops.moe_plan(sel, self.E, tile)
            xs = ops.moe_scatter(x, pos_of, wt, tile_expert.numel() * tile, self.scale_input)
        if self.tc:
            a = ops.moe_gemm_tc(xs, self.w_gate_up, tile_expert, gated=True, act=self.act, limit=self.limit, alpha=self.alpha)
            y = ops.moe_gemm_tc(a, self.w_down, tile_expert, out_dtype=torch.float32)
        else:
            a = ops.moe_gemm(xs, self.w_gate, tile_expert, w2=self.w_up, act=self.act, limit=self.limit, alpha=self.alpha)
            y = ops.moe_gemm(a, self.w_down, tile_expert, out_dtype=torch.float32)
        return y, pos_of, wt

    def forward(self, x, residual, batch, accumulate: bool = True) -> None:
        y, pos_of, wt = self._experts(x)
        ops.moe_combine(y, pos_of, wt, residual, not self.scale_input, "add" if accumulate else "write",
                        x=x if self.n_identity else None)     # (accumulate None: written, like False)
        if self.shared is not None:
            self.shared.forward(x, residual, batch)

    def forward_post(self, x, residual, batch, post_norm) -> None:
        """``residual += post_norm(ffn(x))``, the norm inside the kernel that sums the experts' rows."""
        if self._post_gain is None or self._post_gain[0] is not post_norm.weight:
            self._post_gain = (post_norm.weight, post_norm.weight.float().contiguous())   # the kernel reads a float32 gain
        if self.shared is not None or self.n_identity:
            raise ops.KernelError("a norm inside the experts' sum does not go with a shared expert or experts that return their input")
        y, pos_of, wt = self._experts(x)
        ops.moe_combine(y, pos_of, wt, residual, not self.scale_input, "norm_add", self._post_gain[1], post_norm.eps)


register_ffn("routed_ffn", RoutedFFN)
