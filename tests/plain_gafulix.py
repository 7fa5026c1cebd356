"""Plain, slow implementation of the Gafulix decoder: the tests' oracle for that design.

Whole sequences, no cache, one function per mechanism, torch tensor ops on the CPU in
float64 (or any dtype asked for).  It shares no code with the product package: it reads the
configuration's keys itself and takes weights as a dict of tensors by their checkpoint names.

The design: an embedding; layers ``x += post1(mixer(pre1(x)))``, ``x += post2(ffn(pre2(x)))`` with RMS
norms before and after each sublayer; two kinds of mixer (a gated linear recurrence with a decay per
key channel, and softmax attention with biases, a norm over the whole query / key projection,
interleaved rotary pairs with YaRN frequencies, and a mask that confines a query to its own block of
positions); a routed feed-forward whose gate scales the expert's INPUT; a stretch of layers that runs
several times with the embedding added again before every repeat; a final norm and the head.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- rotary

def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """Per pair i < dims / 2 the angle step, and the factor on cosine and sine.

    Without scaling: base ** (-2 i / dims) and 1.  With {factor, original, fast, slow}: pairs that turn
    more than ``fast`` times within ``original`` positions keep their step, pairs that turn fewer than
    ``slow`` times have it divided by ``factor``, and a linear ramp over the pair index joins the two."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    f = torch.tensor(float(base), dtype=torch.float64) ** (-2.0 * i / dims)
    if not scaling:
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns):
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float,
                       scaling: Optional[dict]) -> torch.Tensor:
    """x [T, heads, d]: channels (2i, 2i + 1), i < dims / 2, of every head turn by position * step_i;
    channels from ``dims`` on stay."""
    f, mag = yarn_frequencies(dims, base, scaling)
    ang = positions.to(torch.float64)[:, None] * f[None, :]
    c, s = (torch.cos(ang) * mag).to(x.dtype)[:, None, :], (torch.sin(ang) * mag).to(x.dtype)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


# --------------------------------------------------------------------------- mixers

def block_mask(T: int, size: Optional[int]) -> torch.Tensor:
    """[T, T] bool: query i sees key j <= i, and with a block size only if both lie in the same block
    of ``size`` positions counted from position 0."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    m = j <= i
    if size:
        m = m & (i // size == j // size)
    return m


def attention_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """h [T, width] -> [T, width]; ``w`` holds the mixer's tensors by their names below the layer."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w["mix.q"].T + w["mix.q.b"]
    k = h @ w["mix.k"].T + w["mix.k.b"]
    v = h @ w["mix.v"].T + w["mix.v.b"]
    q = rms_norm(q, w["mix.q.norm"], eps).view(T, H, d)      # over the whole projection, heads and all
    k = rms_norm(k, w["mix.k.norm"], eps).view(T, G, d)
    v = v.view(T, G, dv)
    pos = torch.arange(T)
    rot = m.get("rot")
    if rot:
        q = rotate_interleaved(q, pos, rot["dims"], rot["base"], rot.get("scaling"))
        k = rotate_interleaved(k, pos, rot["dims"], rot["base"], rot.get("scaling"))
    mask = block_mask(T, (m.get("mask") or {}).get("size"))
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]
        s = s.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(T, H * dv) @ w["mix.o"].T


def gla_mixer(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
              state: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Gated linear attention, token by token: S <- diag(a_t) S + k_t v_t^T, o_t = S^T q_t per head,
    a_t = sigmoid(z_t) ** (1 / tau) per key channel."""
    T = h.shape[0]
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], float(m["tau"])
    q = (h @ w["mix.q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["mix.k"].T).view(T, H, d)
    v = (h @ w["mix.v"].T).view(T, H, dv)
    z = (h @ w["mix.a1"].T) @ w["mix.a2"].T + w["mix.a2.b"]
    a = torch.sigmoid(z).pow(1.0 / tau).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype) if state is None else state
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms_norm(o, w["mix.norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w["mix.g"].T)) @ w["mix.o"].T


# --------------------------------------------------------------------------- feed-forward

def routed_ffn(h: torch.Tensor, w: Dict[str, torch.Tensor], f: dict) -> torch.Tensor:
    """Sigmoid scores, the ``top`` largest chosen, not renormalised; the score multiplies what the
    expert READS: out = sum_e expert_e(s_e * h), expert(u) = W_down (silu(W_gate u) * (W_up u))."""
    E, top = f["router"]["experts"], f["router"]["top"]
    s = torch.sigmoid(h @ w["mlp.router"].T)
    chosen = torch.topk(s, top, dim=-1).indices
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e in chosen[t].tolist():
            u = s[t, e] * h[t]
            out[t] += (silu(u @ w[f"mlp.e{e}.gate"].T) * (u @ w[f"mlp.e{e}.up"].T)) @ w[f"mlp.e{e}.down"].T
    return out


# --------------------------------------------------------------------------- the model

def layer_order(raw: dict) -> List[tuple]:
    """[(layer index, whether the embedding is added before it)] with the repeated stretch unrolled."""
    n = len(raw["layers"])
    loop = raw.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


def layer_tensors(weights: Dict[str, torch.Tensor], i: int) -> Dict[str, torch.Tensor]:
    stem = f"l{i}."
    return {k[len(stem):]: v for k, v in weights.items() if k.startswith(stem)}


def plain_layer(x: torch.Tensor, w: Dict[str, torch.Tensor], layer: dict, eps: float) -> torch.Tensor:
    mixer = {"attention": attention_mixer, "gla": gla_mixer}[layer["type"]]
    x = x + rms_norm(mixer(rms_norm(x, w["norm1"], eps), w, layer["mixer"], eps), w["norm1b"], eps)
    if layer.get("mlp") is not None:
        x = x + rms_norm(routed_ffn(rms_norm(x, w["norm2"], eps), w, layer["mlp"]), w["norm2b"], eps)
    return x


def plain_forward(raw: dict, weights: Dict[str, torch.Tensor], ids: Sequence[int], dtype=torch.float64,
                  streams: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.  ``streams``: a list that receives the residual stream
    after every layer run."""
    W = {k: v.to(dtype) for k, v in weights.items()}
    eps = float(raw["norm"]["eps"])
    x0 = W["embed"][torch.as_tensor(list(ids), dtype=torch.long)]
    x = x0
    for i, again in layer_order(raw):
        if again:
            x = x + x0
        x = plain_layer(x, layer_tensors(W, i), raw["layers"][i], eps)
        if streams is not None:
            streams.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
