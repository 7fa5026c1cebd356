"""Gated linear attention: a recurrent mixer whose memory is a [key_dim, value_dim] matrix per head.

    q = W_q x / sqrt(key_dim)     k = W_k x     v = W_v x
    a = sigmoid(W_2 (W_1 x) + b) ** (1 / tau)          one decay per key channel, in (0, 1)
    S <- diag(a) S + k v^T        o = S^T q            per head, token by token
    y = W_o (concat_heads(o / rms(o) * gain) * silu(W_g x))

The state S is float32, lives in the request's slot of the cache manager's fixed-size state
(``FixedStateRequest``: zeroed when the slot is handed out, given back with the request) and is carried
from step to step; a step's tokens of a request are walked in order, so a single decoded token and a
portion of a prompt are one code path (``csrc/gla.cu``).  The decay, its logarithm, the recurrence and the
head norm are float32; the projections run in the compute dtype with float32 sums and float32 results.

q, k, v, the gate and the decay's first projection are one matrix made at load, so the input is read once;
the decay's second projection (a small inner size), its sigmoid, the division of the logarithm by tau
and the exponential are one float32 kernel.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import BuildContext, FixedStateRequest, Mixer, ParamSpec, register_mixer
from .linear import Linear

_DEFAULT_NAMES = {"q": "q_proj.weight", "k": "k_proj.weight", "v": "v_proj.weight", "g": "g_proj.weight",
                  "o": "o_proj.weight", "norm": "g_norm.weight", "decay_in": "gk_proj.0.weight",
                  "decay_out": "gk_proj.1.weight", "decay_bias": "gk_proj.1.bias"}


class GatedLinearAttention(Mixer):
    def __init__(self, spec, hidden_size: int, ctx: BuildContext):
        self.heads, self.dk, self.dv = int(spec.num_heads), int(spec.key_dim), int(spec.value_dim)
        self.tau, self.eps = float(spec.tau), float(spec.norm_eps)
        if not self.tau > 0:
            raise ValueError(f"tau must be > 0, got {self.tau}")
        if self.dk > ops.GLA_MAX_KEY_DIM:
            raise ops.KernelError(f"gated linear attention: key size {self.dk} exceeds the kernel's {ops.GLA_MAX_KEY_DIM}")
        self.rank = spec.decay_rank
        self.hidden_size = hidden_size
        self.ctx = ctx
        self.names = dict(_DEFAULT_NAMES)
        self.names.update(dict(getattr(spec, "names", ()) or ()))
        self.proj: Linear = None
        self.decay_w = self.decay_b = None
        self.o: Linear = None
        self.gain = None

    def cache_request(self):
        return FixedStateRequest((self.heads, self.dk, self.dv), torch.float32)

    def param_specs(self) -> List[ParamSpec]:
        H, K, V, n = self.hidden_size, self.heads * self.dk, self.heads * self.dv, self.names
        r = -1 if self.rank is None else int(self.rank)
        return [ParamSpec(n["q"], (K, H)), ParamSpec(n["k"], (K, H)), ParamSpec(n["v"], (V, H)),
                ParamSpec(n["g"], (V, H)), ParamSpec(n["o"], (H, V)),
                ParamSpec(n["norm"], (self.dv,), role="gain", init="ones"),
                ParamSpec(n["decay_in"], (r, H)), ParamSpec(n["decay_out"], (K, r)),
                ParamSpec(n["decay_bias"], (K,), role="bias", init="bias_normal")]

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.proj = Linear(torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]],
                                      tensors[n["decay_in"]]], dim=0))
        self.decay_w = tensors[n["decay_out"]].contiguous()
        self.decay_b = tensors[n["decay_bias"]].to(self.decay_w.dtype).contiguous()
        self.o = Linear(tensors[n["o"]])
        self.gain = tensors[n["norm"]].float().contiguous()

    def forward(self, x, residual, batch, cache, owns_cache: bool = True, accumulate: bool = True) -> None:
        if not owns_cache:
            raise ops.KernelError("gated linear attention: a run cannot read another run's state")
        K, V = self.heads * self.dk, self.heads * self.dv
        proj = self.proj(x, out_dtype=torch.float32)                 # [T, q | k | v | g | decay's first projection]
        a = ops.gla_decay(proj, 2 * K + 2 * V, self.decay_w, self.decay_b, self.tau)
        o = ops.gla_scan(proj, 0, K, 2 * K, a, batch, cache.state, self.heads, self.dk, self.dv, self.dk ** -0.5)
        y = ops.gla_gate(o, proj, 2 * K + V, self.gain, self.heads, self.dv, self.eps, self.ctx.dtype)
        if accumulate:
            self.o.add_to(y, residual)
        else:
            self.o(y, out=residual)


register_mixer("gated_linear_attention", GatedLinearAttention)
