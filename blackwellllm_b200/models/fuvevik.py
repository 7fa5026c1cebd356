"""Fuvevik: config.json -> :class:`ModelConfig`.

A decoder whose layers are listed one by one (config ``layers``: each with ``type``, the mixer; ``mixer``, its
sizes; ``mlp``, its feed-forward or null).  What sets the design apart:

* the embedding's output is the token's row plus a sine/cosine vector of the position;
* with ``streams`` the stream is kept as that many copies, which every sublayer reads as a weighted sum and
  writes through a mixing matrix (tensors ``l<i>.hc1.*`` for the mixer, ``l<i>.hc2.*`` for the feed-forward);
  without the key the layers are plain pre-norm layers;
* every norm of the stream stores its gain minus one (``norm.eps`` for all norms);
* mixer ``attention``: grouped-query softmax attention without rotation; queries and keys normed per head
  (one gain vector shared by the heads); the queries of position p times
  ``1 + coef * log(1 + n)``, n the number of whole periods of ``q_temp.every`` positions in p + 1 (``coef`` = ``q_temp.coef``); the score scale ``scale``; a learned sink per
  head in the softmax's denominator; the heads' outputs gated by ``sigmoid(W_g x)``; ``kv_from: j`` makes the
  layer read layer j's keys and values (it has no key and value tensors of its own);
* feed-forward ``dense``: ``down(max(up x, 0)^2)``; ``moe``: a softmax router over ``router.experts`` +
  ``router.identity`` outputs, a stored correction added to the scores for the choice only, ``router.top``
  choices renormalised by their sum + 1e-20, the last ``identity`` outputs standing for experts that return
  their input, experts ``down(g sigmoid(1.702 g) (u + 1))`` with g = min(gate x, limit) and
  u = clamp(up x, -limit, limit), and a shared expert of the same form (``mlp.shared``: ff, limit);
* the output head is the embedding table.

Tensors: ``embed``, ``l<i>.norm1|norm2``, ``l<i>.mix.q|k|v|g|o|q.norm|k.norm|sink``, ``l<i>.mlp.up|down``,
``l<i>.mlp.router|correction``, ``l<i>.mlp.e<j>.gate|up|down``, ``l<i>.mlp.shared.gate|up|down``,
``l<i>.hc1|hc2.in|out|mix``, ``final.norm``.

This module only describes the model.  It builds nothing and owns no tensor.
"""
from __future__ import annotations

from typing import Any, Mapping

from ..config.registry import ConfigError, register_architecture
from ..config.specs import (AttentionSpec, DenseMLPSpec, HyperConnectionSpec, LayerSpec, ModelConfig, NoPositionSpec,
                            RMSNormSpec, RoutedFFNSpec, ScheduleEntry, SinusoidalEmbeddingSpec, SwiGLUSpec)

# constants that the design fixes
POSITION_BASE = 10000.0
SWISH_ALPHA = 1.702
RENORM_EPS = 1e-20

_ATTENTION_NAMES = (("q", "q"), ("k", "k"), ("v", "v"), ("o", "o"), ("g", "g"), ("q_norm", "q.norm"), ("k_norm", "k.norm"),
                    ("sink", "sink"))


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


def _mixer(layer: Mapping[str, Any], where: str, eps: float, index: int, raw_layers) -> AttentionSpec:
    kind = _get(layer, "type", where)
    if kind != "attention":
        raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ('attention')")
    m = _get(layer, "mixer", where)
    w = where + ".mixer"
    heads, kv = _get(m, "heads", w, int), _get(m, "kv_heads", w, int)
    if heads % kv:
        raise ConfigError(f"config.json: {w}: heads ({heads}) is not a multiple of kv_heads ({kv})")
    dim, vdim = _get(m, "dim", w, int), _get(m, "vdim", w, int)
    q_temp = None
    if m.get("q_temp") is not None:
        qt = m["q_temp"]
        q_temp = (_get(qt, "coef", w + ".q_temp", float), _get(qt, "every", w + ".q_temp", float))
        if not q_temp[1] > 0:
            raise ConfigError(f"config.json: {w}.q_temp.every must be > 0")
    src = m.get("kv_from")
    if src is not None:
        if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < index:
            raise ConfigError(f"config.json: {w}.kv_from must name an earlier layer, got {src!r}")
        other = raw_layers[src].get("mixer", {})
        if other.get("kv_from") is not None:
            raise ConfigError(f"config.json: {w}.kv_from names layer {src}, which has no keys and values of its own")
        if (other.get("kv_heads"), other.get("dim"), other.get("vdim")) != (kv, dim, vdim):
            raise ConfigError(f"config.json: {w}.kv_from names layer {src}, whose kv_heads, dim or vdim differ")
    return AttentionSpec(num_heads=heads, num_kv_heads=kv, head_dim=dim, qkv_bias=False, position=NoPositionSpec(),
                         window=None, softmax_scale=_get(m, "scale", w, float),
                         v_head_dim=vdim if vdim != dim else None, qk_norm_eps=eps, names=_ATTENTION_NAMES,
                         qk_norm="head", q_temperature=q_temp, sink=True, output_gate=True, shares_kv=src is not None)


def _gated(f: Mapping[str, Any], where: str) -> SwiGLUSpec:
    return SwiGLUSpec(intermediate_size=_get(f, "ff", where, int), activation="clamped_swish",
                      act_limit=_get(f, "limit", where, float), act_alpha=SWISH_ALPHA, names=("gate", "up", "down"))


def _ffn(layer: Mapping[str, Any], where: str):
    f = layer.get("mlp")
    if f is None:
        return None
    w = where + ".mlp"
    kind = _get(f, "kind", w)
    if kind == "dense":
        return DenseMLPSpec(intermediate_size=_get(f, "ff", w, int), activation="relu2", names=("up", "down"))
    if kind != "moe":
        raise ConfigError(f"config.json: {w}.kind {kind!r} is not a feed-forward of this design ('dense', 'moe')")
    router = _get(f, "router", w)
    experts, top = _get(router, "experts", w + ".router", int), _get(router, "top", w + ".router", int)
    identity = router.get("identity", 0) or 0
    if isinstance(identity, bool) or not isinstance(identity, int) or identity < 0:
        raise ConfigError(f"config.json: {w}.router.identity must be a non-negative integer, got {identity!r}")
    if top > experts + identity:
        raise ConfigError(f"config.json: {w}.router.top ({top}) exceeds the router's outputs ({experts + identity})")
    expert = _gated(_get(f, "expert", w), w + ".expert")
    shared = _gated(f["shared"], w + ".shared") if f.get("shared") is not None else None
    return RoutedFFNSpec(num_experts=experts, top_k=top, expert_size=expert.intermediate_size, score="softmax",
                         renormalize=True, scale_input=False, identity_experts=identity, choice_bias="correction",
                         renorm_eps=RENORM_EPS, activation="clamped_swish", act_limit=expert.act_limit,
                         act_alpha=SWISH_ALPHA, shared=shared, shared_prefix="shared.")


def parse_fuvevik(raw: Mapping[str, Any]) -> ModelConfig:
    width, vocab = _get(raw, "width", "the top level", int), _get(raw, "vocab", "the top level", int)
    eps = _get(_get(raw, "norm", "the top level"), "eps", "norm", float)
    if not eps > 0:
        raise ConfigError(f"config.json: norm.eps must be > 0, got {eps!r}")
    raw_layers = _get(raw, "layers", "the top level")
    if not isinstance(raw_layers, list) or not raw_layers:
        raise ConfigError("config.json: 'layers' must be a non-empty list")
    streams = raw.get("streams")
    if streams is not None and (isinstance(streams, bool) or not isinstance(streams, int) or streams <= 0):
        raise ConfigError(f"config.json: streams must be a positive integer, got {streams!r}")
    # (a single copy may come without its three tensors: they then stand for a plain residual sum)
    hyper = HyperConnectionSpec(streams=streams, mixer_prefix="hc1.", ffn_prefix="hc2.", optional_tensors=streams == 1) \
        if streams is not None else None
    norm = lambda name: RMSNormSpec(eps=eps, param=name, offset=1.0)
    layers, schedule, owner = [], [], {}
    for i, layer in enumerate(raw_layers):
        where = f"layers[{i}]"
        mixer = _mixer(layer, where, eps, i, raw_layers)
        ffn = _ffn(layer, where)
        layers.append(LayerSpec(
            mixer=mixer, ffn=ffn, block="hyper" if hyper is not None else "prenorm", hyper=hyper,
            mixer_norm=norm("norm1"), ffn_norm=norm("norm2") if ffn is not None else None,
            mixer_prefix="mix.", ffn_prefix="mlp.", mixer_norm_prefix="", ffn_norm_prefix=""))
        src = layer["mixer"].get("kv_from")
        schedule.append(ScheduleEntry(layer=i, cache_of=None if src is None else owner[src]))
        if src is None:
            owner[i] = len(schedule) - 1
    eos = raw.get("eos_token_id")
    eos_ids = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(int(e) for e in eos))
    return ModelConfig(
        architecture="Fuvevik", hidden_size=width, vocab_size=vocab, layers=tuple(layers), schedule=tuple(schedule),
        final_norm=norm("norm"), tie_word_embeddings=True, max_position_embeddings=0,
        weight_prefix="", layer_prefix="l{i}.", embed_name="embed", final_norm_prefix="final.", head_name="head",
        position_embedding=SinusoidalEmbeddingSpec(base=POSITION_BASE), streams=streams,
        eos_token_ids=eos_ids, stored_dtype=str(raw.get("torch_dtype", "bfloat16")), raw=dict(raw))


register_architecture("Fuvevik", parse_fuvevik, model_type="fuvevik")
