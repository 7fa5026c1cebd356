"""Tiny Fuvevik configurations for the tests, and their random weights.

They differ from one another in every size and option: how many copies of the stream (one, two, four, or
no copies at all: plain pre-norm layers), heads and kv heads (one query head per kv head, several), key
and value sizes that are equal or differ either way, head sizes the tcgen05 prompt kernel takes (64) and
sizes it does not, the temperature's constants (a period that is no power of two, none at all), the score
scale, which layer lends its keys and values to which (the first, a later one, several borrowers, none),
dense and routed feed-forwards in either order, a layer without feed-forward, experts that return their input
(none, one, several), a token using one, some or all experts, with and without a shared expert, limits, eps.
Stored norm weights and corrections are not small, so that one read from the wrong place shows.
"""
import json
import os

import torch

from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
from blackwellllm_b200.weights.safetensors_io import write_file


def _attn(heads, kv, dim, vdim, scale, q_temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m}


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(experts, identity, top, ff, limit, shared=None):
    f = {"kind": "moe", "expert": {"ff": ff, "limit": limit}, "router": {"experts": experts, "identity": identity, "top": top}}
    if shared is not None:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return f


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# two copies; value size below key size; the second and third layers borrow from the first; a period of 5
PAIR = {
    "architecture": "Fuvevik", "vocab": 210, "width": 64, "norm": {"eps": 1e-5}, "streams": 2,
    "layers": [
        _layer(_attn(4, 2, 32, 16, 0.2, (0.7, 5)), _moe(5, 2, 2, 48, 1.2, (32, 0.8))),
        _layer(_attn(4, 2, 32, 16, 0.15, (0.3, 7), kv_from=0), _dense(96)),
        _layer(_attn(4, 2, 32, 16, 0.25, None, kv_from=0), None),
    ],
}
# four copies; head size 64 with equal sizes (the tcgen05 prompt kernel in bfloat16); the borrower reads from the
# SECOND layer; all experts used and none returns its input (no routing decision: the bfloat16 comparison with
# the plain implementation is continuous); no shared expert; dense first
QUAD = {
    "architecture": "Fuvevik", "vocab": 300, "width": 96, "norm": {"eps": 1e-6}, "streams": 4,
    "layers": [
        _layer(_attn(2, 1, 48, 80, 0.18, (0.25, 16)), _dense(80)),
        _layer(_attn(4, 2, 64, 64, 0.125, (0.5, 32)), _moe(3, 0, 3, 64, 2.0)),
        _layer(_attn(4, 2, 64, 64, 0.11, (1.0, 3), kv_from=1), _moe(2, 0, 2, 32, 0.7, (48, 1.5))),
    ],
}
# one copy of the stream (with its three tensors); one kv head for three query heads; one expert of many per
# token, most of the router's outputs standing for experts that return their input
SINGLE = {
    "architecture": "Fuvevik", "vocab": 150, "width": 48, "norm": {"eps": 1e-4}, "streams": 1,
    "layers": [
        _layer(_attn(3, 1, 16, 16, 0.3, (0.4, 10)), _moe(2, 3, 1, 32, 1.0, (16, 1.0))),
        _layer(_attn(3, 1, 16, 16, 0.3, (0.4, 10), kv_from=0), _moe(6, 1, 2, 16, 3.0)),
    ],
}
# no copies at all (plain pre-norm layers), no borrowing, no temperature in one layer; sizes that no kernel's fast
# form takes: a width that is no multiple of 8, an expert size that is no multiple of 16, key 24 / value 40
PLAIN = {
    "architecture": "Fuvevik", "vocab": 77, "width": 50, "norm": {"eps": 3e-5},
    "layers": [
        _layer(_attn(3, 1, 24, 40, 0.21, (0.6, 9)), _moe(3, 1, 2, 20, 1.1, (12, 0.9))),
        _layer(_attn(2, 2, 8, 8, 0.35), _dense(30)),
    ],
}
# three copies like many real configurations, but head size 128, a wide feed-forward and more experts
BROAD = {
    "architecture": "Fuvevik", "vocab": 400, "width": 128, "norm": {"eps": 1e-6}, "streams": 3,
    "layers": [
        _layer(_attn(2, 1, 128, 128, 0.09, (0.5, 48)), _moe(8, 2, 3, 32, 1.5, (64, 1.0))),
        _layer(_attn(2, 1, 128, 128, 0.09, (0.5, 48), kv_from=0), _dense(256)),
    ],
}

# name -> (config, page size)
CONFIGS = {"pair": (PAIR, 8), "quad": (QUAD, 16), "single": (SINGLE, 32), "plain": (PLAIN, 16), "broad": (BROAD, 64)}


def make_tensors(raw, seed, std=0.08, bias_std=0.3, dtype=torch.bfloat16):
    """Random weights by their checkpoint names, rounded to ``dtype``.  Query and key gains 1 + noise; stored norm
    weights, sinks and corrections N(0, 0.3); mixing matrices near the identity; router rows spread out."""
    specs = model_param_specs(raw)
    tensors = random_tensors(specs, seed, std, bias_std, dtype=torch.float32, skip_optional=False)
    g = torch.Generator().manual_seed(seed + 4321)
    for name, spec in specs.items():
        if spec.role == "gain" and spec.init == "ones":
            tensors[name] = 1.0 + 0.4 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mlp.router"):
            tensors[name] = tensors[name] * 4.0       # scores spread out: few near-ties
        if name.endswith(".mlp.correction"):
            tensors[name] = 0.1 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mix") and ".hc" in name:
            tensors[name] = torch.eye(spec.shape[0]) + 0.2 * torch.randn(spec.shape, generator=g)
        if (name.endswith(".in") or name.endswith(".out")) and ".hc" in name:
            tensors[name] = 0.8 + 0.3 * torch.randn(spec.shape, generator=g)
    return {k: v.to(dtype) for k, v in tensors.items()}


def make_folder(name, dtype, root, seed=5):
    raw, _ = CONFIGS[name]
    d = os.path.join(root, f"fuvevik-{name}-{dtype}")
    if not os.path.isdir(d):
        os.makedirs(d)
        tensors = make_tensors(raw, seed, dtype={"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype])
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(raw, f)
        write_file(os.path.join(d, "model.safetensors"), tensors, metadata={"format": "pt"})
    return d


def prompt(n, vocab, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
