"""Arrangements of norms, mixer and feed-forward in a layer.

``prenorm`` (src/core/engine.cpp:946-1024): the norm stands before each sublayer
and reads the residual stream without changing it; each sublayer adds its output
to the residual stream, which stays float32.  A sublayer's last product may leave its sum to the
next reader of the stream (``Linear.add_to``): the next norm, which adds it while it normalises.
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ..kernels import ops
from .base import (Block, BuildContext, ParamSpec, build_ffn, build_mixer, build_norm,
                   register_block)


class PreNormBlock(Block):
    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        self.spec = layer_spec
        self.mixer_norm = build_norm(layer_spec.mixer_norm, hidden_size, ctx)
        self.mixer = build_mixer(layer_spec.mixer, hidden_size, ctx)
        self.ffn = None
        self.ffn_norm = None
        if layer_spec.ffn is not None:
            self.ffn_norm = build_norm(layer_spec.ffn_norm, hidden_size, ctx)
            self.ffn = build_ffn(layer_spec.ffn, hidden_size, ctx)

    def _children(self):
        s = self.spec
        kids = [(s.mixer_norm_prefix, self.mixer_norm), (s.mixer_prefix, self.mixer)]
        if self.ffn is not None:
            kids += [(s.ffn_norm_prefix, self.ffn_norm), (s.ffn_prefix, self.ffn)]
        return kids

    def param_specs(self) -> List[ParamSpec]:
        out = []
        for prefix, part in self._children():
            for p in part.param_specs():
                out.append(ParamSpec(prefix + p.name, p.shape, p.role, p.init, p.optional))
        return out

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        for prefix, part in self._children():
            part.bind({k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)})

    takes_pending = True

    @staticmethod
    def _normed(norm, residual):
        # a sublayer may have left the sum of its last product to the stream's next reader: a norm
        # that adds it while it normalises, or else a kernel of its own here
        if not norm.adds_pending:
            ops.resolve_pending()
        return norm.forward(residual)

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        x = self._normed(self.mixer_norm, residual)
        self.mixer.forward(x, residual, batch, cache, owns_cache)
        if self.ffn is not None:
            x = self._normed(self.ffn_norm, residual)
            self.ffn.forward(x, residual, batch)


class SandwichBlock(PreNormBlock):
    """A norm before AND after each sublayer: ``x += post(mixer(pre(x)))``, ``x += post(ffn(pre(x)))``.  The
    sublayer writes its output to a float32 buffer of its own (``accumulate=False``); the second norm reads
    it and adds the result to the stream in one kernel.  A feed-forward with ``forward_post`` does the
    second norm inside its own last kernel."""
    takes_pending = False

    def __init__(self, layer_spec, hidden_size: int, ctx: BuildContext):
        super().__init__(layer_spec, hidden_size, ctx)
        if layer_spec.mixer_post_norm is None or (layer_spec.ffn is not None and layer_spec.ffn_post_norm is None):
            raise ValueError("the sandwich arrangement needs a norm after each sublayer")
        self.mixer_post = build_norm(layer_spec.mixer_post_norm, hidden_size, ctx)
        self.ffn_post = build_norm(layer_spec.ffn_post_norm, hidden_size, ctx) if self.ffn is not None else None
        for norm in (self.mixer_post, self.ffn_post):
            if norm is not None and not hasattr(norm, "add_to"):
                raise ValueError(f"{type(norm).__name__} cannot follow a sublayer (it has no add_to)")

    def _children(self):
        s = self.spec
        kids = super()._children() + [(s.mixer_post_norm_prefix, self.mixer_post)]
        if self.ffn is not None:
            kids.append((s.ffn_post_norm_prefix, self.ffn_post))
        return kids

    def forward(self, residual, batch, cache, owns_cache: bool = True) -> None:
        x = self._normed(self.mixer_norm, residual)
        branch = torch.empty_like(residual)
        self.mixer.forward(x, branch, batch, cache, owns_cache, accumulate=False)
        if self.ffn is None:
            self.mixer_post.add_to(branch, residual)
        else:
            # the norm after the mixer and the norm before the feed-forward read the same row: one kernel if they can
            if hasattr(self.mixer_post, "add_to_then"):
                x = self.mixer_post.add_to_then(branch, residual, self.ffn_norm)
            else:
                self.mixer_post.add_to(branch, residual)
                x = self.ffn_norm.forward(residual)
            if hasattr(self.ffn, "forward_post"):
                self.ffn.forward_post(x, residual, batch, self.ffn_post)
            else:
                self.ffn.forward(x, branch, batch, accumulate=False)
                self.ffn_post.add_to(branch, residual)


register_block("prenorm", PreNormBlock)
register_block("sandwich", SandwichBlock)
