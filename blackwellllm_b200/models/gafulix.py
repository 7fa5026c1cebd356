"""Gafulix: config.json -> :class:`ModelConfig`.

A decoder whose layers differ: config ``layers`` lists them, each with ``type`` (which mixer), ``mixer``
(its sizes) and ``mlp`` (its feed-forward, or null).  Every layer norms the input AND the output of each
sublayer (the "sandwich" arrangement).  Mixers:

* ``gla``: gated linear attention (``parts/gla.py``): heads, dim, vdim, tau;
* ``attention``: grouped-query softmax attention with q/k/v biases, an RMS norm over the whole query
  and the whole key projection, rotary pairs (2i, 2i + 1) over ``rot.dims`` channels with YaRN
  frequencies (``rot.scaling``: factor, original, fast, slow), the score scale ``scale``, and a mask that
  keeps a query inside its own block of ``mask.size`` positions.

Feed-forward ``moe``: ``router.experts`` gated experts of size ``expert.ff``, ``router.top`` per token,
sigmoid scores that are not renormalised and multiply the expert's input.

``loop`` {start, stop, times}: layers start .. stop-1 run ``times`` times in a row with the same weights,
each pass with a cache or state of its own; before every pass but the first the embedding's output is
added to the stream.  Sizes: ``vocab``, ``width``; ``norm.eps`` for every norm.

Tensors: ``embed``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.router``,
``l<i>.mlp.e<j>.gate|up|down``, ``final.norm``, ``head``.

This module only describes the model.  It builds nothing and owns no tensor.
"""
from __future__ import annotations

from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, GatedLinearAttentionSpec, LayerSpec, ModelConfig, NoPositionSpec,
                            RMSNormSpec, RopeSpec, RoutedFFNSpec, ScheduleEntry, YarnRopeScaling)

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("q_bias", "q.b"), ("k_bias", "k.b"),
                    ("v_bias", "v.b"), ("q_norm", "q.norm"), ("k_norm", "k.norm"))
_GLA_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("norm", "norm"), ("decay_in", "a1"),
              ("decay_out", "a2"), ("decay_bias", "a2.b"))


def _get(d: Mapping[str, Any], key: str, where: str, kind=None):
    if not isinstance(d, Mapping) or key not in d:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    v = d[key]
    if kind is int and (isinstance(v, bool) or not isinstance(v, int) or v <= 0):
        raise ConfigError(f"config.json: {where}.{key} must be a positive integer, got {v!r}")
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: {where}.{key} must be a number, got {v!r}")
        v = float(v)
    return v


def _position(m: Mapping[str, Any], where: str):
    rot = m.get("rot")
    if rot is None:
        return NoPositionSpec()
    dims = _get(rot, "dims", where + ".rot", int)
    base = _get(rot, "base", where + ".rot", float)
    if dims % 2 or dims > m["dim"] or not base > 1.0:
        raise ConfigError(f"config.json: {where}.rot needs an even dims <= dim and a base > 1")
    sc = rot.get("scaling")
    scaling = None
    if sc is not None:
        w = where + ".rot.scaling"
        scaling = YarnRopeScaling(factor=_get(sc, "factor", w, float), original=_get(sc, "original", w, int),
                                  fast=_get(sc, "fast", w, float), slow=_get(sc, "slow", w, float))
        if not (scaling.factor > 0 and scaling.fast > 0 and scaling.slow > 0):
            raise ConfigError(f"config.json: {w} needs factor, fast and slow > 0")
    return RopeSpec(theta=base, rotary_dim=dims, scaling=scaling, interleaved=True)


def _mixer(layer: Mapping[str, Any], where: str, eps: float):
    kind = _get(layer, "type", where)
    m = _get(layer, "mixer", where)
    w = where + ".mixer"
    if kind == "gla":
        rank = m.get("rank")
        return GatedLinearAttentionSpec(num_heads=_get(m, "heads", w, int), key_dim=_get(m, "dim", w, int),
                                        value_dim=_get(m, "vdim", w, int), tau=_get(m, "tau", w, float), norm_eps=eps,
                                        decay_rank=int(rank) if rank is not None else None, names=_GLA_NAMES)
    if kind == "attention":
        heads, kv = _get(m, "heads", w, int), _get(m, "kv_heads", w, int)
        if heads % kv:
            raise ConfigError(f"config.json: {w}: heads ({heads}) is not a multiple of kv_heads ({kv})")
        dim, vdim = _get(m, "dim", w, int), _get(m, "vdim", w, int)
        mask = m.get("mask")
        chunk = _get(mask, "size", w + ".mask", int) if mask is not None else None
        return AttentionSpec(num_heads=heads, num_kv_heads=kv, head_dim=dim, qkv_bias=True, position=_position(m, w),
                             window=None, softmax_scale=_get(m, "scale", w, float), chunk=chunk,
                             v_head_dim=vdim if vdim != dim else None, qk_norm_eps=eps, names=_ATTENTION_NAMES)
    raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ('gla', 'attention')")


def _ffn(layer: Mapping[str, Any], where: str):
    f = layer.get("mlp")
    if f is None:
        return None
    w = where + ".mlp"
    if f.get("kind", "moe") != "moe":
        raise ConfigError(f"config.json: {w}.kind {f.get('kind')!r} is not a feed-forward of this design ('moe')")
    router = _get(f, "router", w)
    experts, top = _get(router, "experts", w + ".router", int), _get(router, "top", w + ".router", int)
    if top > experts:
        raise ConfigError(f"config.json: {w}.router.top ({top}) exceeds experts ({experts})")
    return RoutedFFNSpec(num_experts=experts, top_k=top, expert_size=_get(_get(f, "expert", w), "ff", w + ".expert", int),
                         score="sigmoid", renormalize=False, scale_input=True)


def parse_gafulix(raw: Mapping[str, Any]) -> ModelConfig:
    width, vocab = _get(raw, "width", "the top level", int), _get(raw, "vocab", "the top level", int)
    eps = _get(_get(raw, "norm", "the top level"), "eps", "norm", float)
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be > 0, got {eps!r}")
    raw_layers = _get(raw, "layers", "the top level")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    layers = []
    for i, layer in enumerate(raw_layers):
        where = f"layers[{i}]"
        ffn = _ffn(layer, where)
        layers.append(LayerSpec(
            mixer=_mixer(layer, where, eps), ffn=ffn, block="sandwich",
            mixer_norm=RMSNormSpec(eps=eps, param="norm1"), mixer_post_norm=RMSNormSpec(eps=eps, param="norm1b"),
            ffn_norm=RMSNormSpec(eps=eps, param="norm2") if ffn is not None else None,
            ffn_post_norm=RMSNormSpec(eps=eps, param="norm2b") if ffn is not None else None,
            mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm_prefix="", ffn_norm_prefix="",
            mixer_post_norm_prefix="", ffn_post_norm_prefix=""))
    n = len(layers)
    loop = raw.get("loop")
    start, stop, times = 0, 0, 1
    if loop is not None:
        start, stop, times = (loop.get(k) for k in ("start", "stop", "times"))
        if not all(isinstance(v, int) and not isinstance(v, bool) for v in (start, stop, times)) \
                or not (0 <= start <= stop <= n) or times < 0:
            raise ConfigError(f"config.json: loop needs integers 0 <= start <= stop <= {n} and times >= 0, got {loop!r}")
    schedule = [ScheduleEntry(layer=i) for i in range(start)]
    for rep in range(times):
        schedule += [ScheduleEntry(layer=i, add_embedding=(rep > 0 and i == start)) for i in range(start, stop)]
    schedule += [ScheduleEntry(layer=i) for i in range(stop, n)]
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
    return ModelConfig(
        architecture="Gafulix", hidden_size=width, vocab_size=vocab, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=RMSNormSpec(eps=eps, param="norm"), tie_word_embeddings=False, max_position_embeddings=0,
        weight_prefix="", layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        eos_token_ids=eos_ids, stored_dtype=str(raw.get("torch_dtype", "bfloat16")), raw=dict(raw))


register_architecture("Gafulix", parse_gafulix, model_type="gafulix")
