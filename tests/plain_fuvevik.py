"""Plain, slow implementation of the Fuvevik decoder: the tests' oracle for that design.

Whole sequences, no cache, one function per mechanism, torch tensor ops on the CPU in float64 (or any
dtype asked for).  It shares no code with the product package: it reads the configuration's keys itself
and takes weights as a dict of tensors by their checkpoint names.

The design: token embedding plus a sine/cosine vector of the position; ``streams`` copies of the stream
that every sublayer reads as a weighted sum and writes back through a mixing matrix (hyper-connections);
RMS norms whose stored weight is the gain minus one; softmax attention without rotation whose queries and
keys are normed per head, whose queries grow with the logarithm of the position, whose softmax has one
more, keyless term per head (a sink) and whose output is gated by a sigmoid of the mixer's input, and
which may read the keys and values of an earlier layer; feed-forwards that are either dense
(squared relu) or a mixture of experts (softmax router, a bias on the choice only, renormalised
weights, experts that return their input, a clamped gated activation, a shared expert); the embedding
table is the output head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


# --------------------------------------------------------------------------- small pieces

def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def offset_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the stored weight lies around zero, the gain is one plus it."""
    return unit_rms(x, eps) * (1.0 + w)


def plain_gain_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm of queries and keys: the stored weight is the gain."""
    return unit_rms(x, eps) * w


def position_vectors(positions: torch.Tensor, width: int, dtype) -> torch.Tensor:
    """[T, width]: entry 2i is sin(p * 10000^(-2i/width)), entry 2i + 1 the cosine of the same angle."""
    n = (width + 1) // 2
    i = torch.arange(n, dtype=torch.float64)
    ang = positions.to(torch.float64)[:, None] * torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width)[None, :]
    out = torch.zeros(positions.numel(), 2 * n, dtype=torch.float64)
    out[:, 0::2] = torch.sin(ang)
    out[:, 1::2] = torch.cos(ang)
    return out[:, :width].to(dtype)


def query_temperature(positions: torch.Tensor, q_temp: Optional[dict]) -> torch.Tensor:
    """1 + coef * log(1 + n) per position p, n the whole periods of ``every`` positions that p + 1 holds (ones without the option)."""
    p = positions.to(torch.float64)
    if not q_temp:
        return torch.ones_like(p)
    return 1.0 + float(q_temp["coef"]) * torch.log(torch.floor((p + 1.0) / float(q_temp["every"])) + 1.0)


# --------------------------------------------------------------------------- attention

def project_keys_values(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float):
    """Normed keys [T, G, dim] and values [T, G, vdim] of a layer that owns them."""
    T = h.shape[0]
    G, d, dv = m["kv_heads"], m["dim"], m["vdim"]
    k = (h @ w["mix.k"].T).view(T, G, d)
    k = plain_gain_norm(k, w["mix.k.norm"], eps)
    v = (h @ w["mix.v"].T).view(T, G, dv)
    return k, v


def sink_softmax(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, T, T] with -inf where masked, sink [H]: softmax over the keys and one more term exp(sink)
    that has no key: the weights of a row sum to less than one."""
    m = torch.maximum(scores.max(dim=-1, keepdim=True).values, sink[:, None, None])
    e = torch.exp(scores - m)
    return e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink[:, None, None] - m))


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, positions: torch.Tensor,
                    keys_values=None):
    """Returns (output [T, width], (keys, values)); ``keys_values``: those of the layer it reads them from."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w["mix.q"].T).view(T, H, d)
    q = plain_gain_norm(q, w["mix.q.norm"], eps)
    q = q * query_temperature(positions, m.get("q_temp")).to(q.dtype)[:, None, None]
    if keys_values is None:
        keys_values = project_keys_values(h, w, m, eps)
    k, v = keys_values
    rep = H // G
    kk = k.repeat_interleave(rep, dim=1)          # query head h uses key/value head h // rep
    vv = v.repeat_interleave(rep, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, kk) * float(m["scale"])
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    scores = scores.masked_fill(~(j <= i)[None], float("-inf"))
    p = sink_softmax(scores, w["mix.sink"].to(scores.dtype))
    o = torch.einsum("hij,jhd->ihd", p, vv).reshape(T, H * dv)
    o = o * torch.sigmoid(h @ w["mix.g"].T)
    return o @ w["mix.o"].T, keys_values


# --------------------------------------------------------------------------- feed-forwards

def dense_ffn(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    a = torch.relu(h @ w["mlp.up"].T)
    return (a * a) @ w["mlp.down"].T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.T, max=limit)
    u = torch.clamp(h @ up.T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict):
    """(chosen outputs of the router [T, top], their weights [T, top])."""
    top = f["router"]["top"]
    s = torch.softmax(h @ w["mlp.router"].T, dim=-1)
    choice = s + w["mlp.correction"].to(s.dtype) if "mlp.correction" in w else s
    idx = torch.topk(choice, top, dim=-1).indices
    chosen = torch.gather(s, 1, idx)
    return idx, chosen / (chosen.sum(dim=-1, keepdim=True) + 1e-20)


def moe_ffn(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    E = f["router"]["experts"]
    limit = float(f["expert"]["limit"])
    idx, wt = route(h, w, f)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            if e >= E:                     # the router's last outputs stand for experts that return their input
                out[t] += a * h[t]
            else:
                out[t] += a * clamped_expert(h[t:t + 1], w[f"mlp.e{e}.gate"], w[f"mlp.e{e}.up"], w[f"mlp.e{e}.down"], limit)[0]
    if f.get("shared"):
        out = out + clamped_expert(h, w["mlp.shared.gate"], w["mlp.shared.up"], w["mlp.shared.down"], float(f["shared"]["limit"]))
    return out


# --------------------------------------------------------------------------- layers

def layer_tensors(weights: Dict[str, torch.Tensor], i: int, dtype) -> Dict[str, torch.Tensor]:
    stem = f"l{i}."
    return {k[len(stem):]: v.to(dtype) for k, v in weights.items() if k.startswith(stem)}


def hyper_read(xs: torch.Tensor, w_in: torch.Tensor) -> torch.Tensor:
    """xs [s, T, width] -> the sublayer's input sum_s in[s] xs[s]."""
    return torch.einsum("s,std->td", w_in, xs)


def hyper_write(xs: torch.Tensor, y: torch.Tensor, mix: torch.Tensor, w_out: torch.Tensor) -> torch.Tensor:
    """new xs[t] = sum_s mix[s, t] xs[s] + out[t] y, all from the old streams."""
    return torch.einsum("sr,std->rtd", mix, xs) + w_out[:, None, None] * y[None]


def plain_forward(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64,
                  streams_after_layers: Optional[List[torch.Tensor]] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  ``streams_after_layers``: a list that receives the stream
    (the sum of the copies) after every layer."""
    eps = float(raw["norm"]["eps"])
    width = raw["width"]
    ids = torch.as_tensor(list(ids), dtype=torch.long)
    T = ids.numel()
    positions = torch.arange(T)
    embed = weights["embed"].to(dtype)
    x = embed[ids] + position_vectors(positions, width, dtype)
    hyper = "streams" in raw
    xs = x[None].repeat(int(raw["streams"]), 1, 1) if hyper else x[None]
    kept = {}
    for i, layer in enumerate(raw["layers"]):
        w = layer_tensors(weights, i, dtype)
        subs = [("1", "mixer")] + ([("2", "ffn")] if layer.get("mlp") else [])
        for q, what in subs:
            u = hyper_read(xs, w[f"hc{q}.in"]) if hyper else xs[0]
            hn = offset_norm(u, w[f"norm{q}"], eps)
            if what == "mixer":
                if layer["type"] != "attention":
                    raise ValueError(f"unknown mixer {layer['type']!r}")
                m = layer["mixer"]
                src = m.get("kv_from")
                y, kept[i] = attention_mixer(hn, w, m, eps, positions, None if src is None else kept[src])
            else:
                f = layer["mlp"]
                y = dense_ffn(hn, w) if f["kind"] == "dense" else moe_ffn(hn, w, f)
            xs = hyper_write(xs, y, w[f"hc{q}.mix"], w[f"hc{q}.out"]) if hyper else xs + y[None]
        if streams_after_layers is not None:
            streams_after_layers.append(xs.sum(dim=0))
    x = xs.sum(dim=0)
    return offset_norm(x, weights["final.norm"].to(dtype), eps) @ embed.T
