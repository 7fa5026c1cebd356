"""Tiny Gafulix configurations for the tests, and their random weights.

They differ from one another in every size and option: heads and kv heads, key and value sizes that
differ, the rotated span of a head, YaRN parameters or none, no rotation at all, the score scale, the
block size of the mask (a multiple of the kernels' tile, not one, smaller than a page, absent), experts
and how many a token uses (one, some, all), a layer without feed-forward, the order of the layers, the
repeated stretch (none, the whole model, a part, a single layer), eps and tau.  Norm gains are not all
ones and biases are not small, so that a gain or bias read from the wrong place shows.
"""
import json
import os

import torch

from blackwellllm_b200.weights.random_init import model_param_specs, random_tensors
from blackwellllm_b200.weights.safetensors_io import write_file


def _attn(heads, kv, dim, vdim, scale, rot=None, mask=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if mask is not None:
        m["mask"] = {"size": mask}
    return {"type": "attention", "mixer": m}


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}}


def _moe(experts, top, ff):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


YARN_A = {"factor": 2.0, "original": 64, "fast": 4.0, "slow": 1.0}
YARN_B = {"factor": 8.0, "original": 256, "fast": 16.0, "slow": 2.0}

# attention first, value size below key size, half a head rotated, block of 24 (no multiple of anything),
# two experts of four; a GLA layer without feed-forward; the first two layers run three times
MIXED = {
    "architecture": "Gafulix", "vocab": 200, "width": 64, "norm": {"eps": 1e-4},
    "layers": [
        _layer(_attn(4, 2, 32, 16, 0.3, {"base": 5000.0, "dims": 16, "scaling": YARN_A}, 24), _moe(4, 2, 48)),
        _layer(_gla(3, 24, 40, 4.0, 8), None),
        _layer(_gla(2, 16, 16, 9.0, 4), _moe(3, 1, 40)),
    ],
    "loop": {"start": 0, "stop": 2, "times": 3},
}
# head size 64 with equal key and value sizes (the tcgen05 prompt kernel in bfloat16), block of 64 = the tile,
# rotary without rescaling over the whole head, value size above key size in the second attention layer with a
# block smaller than a page, a key size above 64 and an odd value size in the GLA layer, no loop,
# all experts used (no routing decision: the bfloat16 comparison with the plain implementation is continuous)
WIDE = {
    "architecture": "Gafulix", "vocab": 320, "width": 96, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_gla(2, 72, 33, 16.0, 16), _moe(3, 3, 64)),
        _layer(_attn(2, 2, 64, 64, 0.125, {"base": 10000.0, "dims": 64}, 64), _moe(3, 3, 64)),
        _layer(_attn(6, 3, 16, 48, 0.25, {"base": 100.0, "dims": 16, "scaling": YARN_B}, 10), _moe(2, 2, 24)),
    ],
}
# no rotation and no mask in one attention layer, a single repeated layer in the middle, one expert of many
LOOPED = {
    "architecture": "Gafulix", "vocab": 150, "width": 48, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_attn(3, 1, 16, 16, 0.25), _moe(6, 1, 32)),
        _layer(_gla(1, 40, 24, 2.0, 4), _moe(6, 2, 32)),
        _layer(_attn(2, 1, 32, 32, 0.2, {"base": 1000.0, "dims": 8, "scaling": YARN_A}, 128), None),
    ],
    "loop": {"start": 1, "stop": 2, "times": 4},
}

# sizes that no kernel's fast form takes: a width that is no multiple of 8 (no TMA row: the CUDA-core products, in
# bfloat16 too), an expert size that is no multiple of 16, three query heads on one kv head, key 24 / value 40
ODD = {
    "architecture": "Gafulix", "vocab": 77, "width": 50, "norm": {"eps": 3e-5},
    "layers": [
        _layer(_attn(3, 1, 24, 40, 0.21, {"base": 777.0, "dims": 24, "scaling": YARN_B}, 7), _moe(3, 2, 20)),
        _layer(_gla(2, 20, 12, 5.0, 3), _moe(5, 5, 12)),
    ],
}
# recurrent layers only: no page pool at all, state slots alone; both layers twice
RECURRENT = {
    "architecture": "Gafulix", "vocab": 90, "width": 72, "norm": {"eps": 1e-5},
    "layers": [_layer(_gla(2, 16, 24, 3.0, 4), _moe(2, 1, 16)), _layer(_gla(4, 8, 8, 8.0, 2), None)],
    "loop": {"start": 0, "stop": 2, "times": 2},
}

# name -> (config, page size)
CONFIGS = {"mixed": (MIXED, 8), "wide": (WIDE, 16), "looped": (LOOPED, 32), "odd": (ODD, 16), "recurrent": (RECURRENT, 16)}


def make_tensors(raw, seed, std=0.08, bias_std=0.3, dtype=torch.bfloat16):
    """Random weights by their checkpoint names, rounded to ``dtype``; gains 1 + noise."""
    specs = model_param_specs(raw)
    tensors = random_tensors(specs, seed, std, bias_std, dtype=torch.float32)
    g = torch.Generator().manual_seed(seed + 12345)
    for name, spec in specs.items():
        if spec.role == "gain":
            tensors[name] = 1.0 + 0.4 * torch.randn(spec.shape, generator=g)
        if name.endswith(".mlp.router"):
            tensors[name] = tensors[name] * 4.0       # scores spread out: few near-ties
    return {k: v.to(dtype) for k, v in tensors.items()}


def make_folder(name, dtype, root, seed=5):
    raw, _ = CONFIGS[name]
    d = os.path.join(root, f"gafulix-{name}-{dtype}")
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
