"""Gafulix without a GPU: config.json -> the model's description, the order of layer runs, the tensors it
asks for, refusals; and the plain implementation against itself where a property must hold exactly."""
import copy

import pytest
import torch

import plain_gafulix as plain
import tiny_gafulix as tg
from blackwellllm_b200.config import ConfigError, parse_config
from blackwellllm_b200.config.specs import (AttentionSpec, GatedLinearAttentionSpec, NoPositionSpec, RoutedFFNSpec,
                                            YarnRopeScaling)
from blackwellllm_b200.weights.loader import WeightError, check_names
from blackwellllm_b200.weights.random_init import model_param_specs


def test_description_follows_the_configuration():
    cfg = parse_config(tg.MIXED)
    assert cfg.architecture == "Gafulix" and cfg.hidden_size == 64 and cfg.vocab_size == 200
    a, g, g2 = (l.mixer for l in cfg.layers)
    assert isinstance(a, AttentionSpec) and (a.num_heads, a.num_kv_heads, a.head_dim, a.v_head_dim) == (4, 2, 32, 16)
    assert a.chunk == 24 and a.softmax_scale == 0.3 and a.qkv_bias and a.qk_norm_eps == 1e-4 and a.window is None
    assert a.position.interleaved and a.position.rotary_dim == 16 and a.position.theta == 5000.0
    assert a.position.scaling == YarnRopeScaling(factor=2.0, original=64, fast=4.0, slow=1.0)
    assert isinstance(g, GatedLinearAttentionSpec) and (g.num_heads, g.key_dim, g.value_dim, g.tau) == (3, 24, 40, 4.0)
    assert cfg.layers[1].ffn is None and cfg.layers[1].ffn_norm is None
    f = cfg.layers[0].ffn
    assert isinstance(f, RoutedFFNSpec) and (f.num_experts, f.top_k, f.expert_size) == (4, 2, 48)
    assert f.score == "sigmoid" and not f.renormalize and f.scale_input
    assert all(l.block == "sandwich" for l in cfg.layers)
    # equal key and value sizes, no rescaling, no rotation, no mask
    wide, looped = parse_config(tg.WIDE), parse_config(tg.LOOPED)
    assert wide.layers[1].mixer.v_head_dim is None and wide.layers[1].mixer.position.scaling is None
    assert isinstance(looped.layers[0].mixer.position, NoPositionSpec) and looped.layers[0].mixer.chunk is None


@pytest.mark.parametrize("raw", [c for c, _ in tg.CONFIGS.values()])
def test_order_of_layer_runs(raw):
    cfg = parse_config(raw)
    assert [(e.layer, e.add_embedding) for e in cfg.schedule] == plain.layer_order(raw)
    assert all(e.cache_of is None for e in cfg.schedule)      # every pass has a cache or state of its own


def test_loop_variants():
    raw = copy.deepcopy(tg.MIXED)
    for loop, want in [(None, [0, 1, 2]), ({"start": 0, "stop": 3, "times": 2}, [0, 1, 2, 0, 1, 2]),
                       ({"start": 2, "stop": 3, "times": 3}, [0, 1, 2, 2, 2]), ({"start": 1, "stop": 1, "times": 5}, [0, 1, 2]),
                       ({"start": 0, "stop": 1, "times": 1}, [0, 1, 2])]:
        if loop is None:
            raw.pop("loop", None)
        else:
            raw["loop"] = loop
        cfg = parse_config(raw)
        assert [e.layer for e in cfg.schedule] == want
        again = [i for i, e in enumerate(cfg.schedule) if e.add_embedding]
        times = (loop or {}).get("times", 1)
        span = (loop["stop"] - loop["start"]) if loop else 0
        assert len(again) == (max(times - 1, 0) if span else 0)


def test_tensor_names_and_shapes():
    specs = model_param_specs(tg.MIXED)
    assert specs["embed"].shape == (200, 64) and specs["head"].shape == (200, 64) and specs["final.norm"].shape == (64,)
    for n, shape in {"l0.norm1": (64,), "l0.norm1b": (64,), "l0.norm2": (64,), "l0.norm2b": (64,), "l0.mix.q": (128, 64),
                     "l0.mix.q.b": (128,), "l0.mix.k": (64, 64), "l0.mix.v": (32, 64), "l0.mix.v.b": (32,),
                     "l0.mix.q.norm": (128,), "l0.mix.k.norm": (64,), "l0.mix.o": (64, 64), "l0.mlp.router": (4, 64),
                     "l0.mlp.e3.gate": (48, 64), "l0.mlp.e3.up": (48, 64), "l0.mlp.e3.down": (64, 48),
                     "l1.mix.q": (72, 64), "l1.mix.k": (72, 64), "l1.mix.v": (120, 64), "l1.mix.g": (120, 64),
                     "l1.mix.o": (64, 120), "l1.mix.norm": (40,), "l1.mix.a1": (8, 64), "l1.mix.a2": (72, 8),
                     "l1.mix.a2.b": (72,)}.items():
        assert specs[n].shape == shape, n
    assert "l1.norm2" not in specs and "l1.mlp.router" not in specs       # a layer without feed-forward
    assert not any(n.startswith("l3.") for n in specs)


def test_a_size_the_configuration_leaves_open_is_taken_from_the_tensor():
    raw = copy.deepcopy(tg.MIXED)
    del raw["layers"][1]["mixer"]["rank"]
    specs = model_param_specs(raw)
    assert specs["l1.mix.a1"].shape == (-1, 64) and specs["l1.mix.a2"].shape == (72, -1)
    found = {n: torch.empty([5 if d == -1 else d for d in s.shape]) for n, s in specs.items()}
    check_names("x", specs, found)
    found["l1.mix.a2"] = torch.empty(71, 5)
    with pytest.raises(WeightError):
        check_names("x", specs, found)
    with pytest.raises(ValueError):
        tg.make_tensors(raw, 0)


@pytest.mark.parametrize("edit,word", [
    (lambda r: r["layers"][0].update(type="conv"), "not a mixer"),
    (lambda r: r["layers"][0]["mixer"].update(kv_heads=3), "multiple"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=9), "exceeds"),
    (lambda r: r["layers"][0]["mixer"]["rot"].update(dims=34), "dims"),
    (lambda r: r.update(loop={"start": 2, "stop": 1, "times": 2}), "loop"),
    (lambda r: r.pop("width"), "width"),
    (lambda r: r["norm"].update(eps=0.0), "eps"),
    (lambda r: r["layers"][1]["mixer"].pop("tau"), "tau"),
])
def test_refusals(edit, word):
    raw = copy.deepcopy(tg.MIXED)
    edit(raw)
    with pytest.raises(ConfigError, match=word):
        parse_config(raw)


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_recurrence_goes_on_from_a_state():
    m = {"heads": 2, "dim": 6, "vdim": 5, "tau": 3.0}
    g = torch.Generator().manual_seed(0)
    w = {"mix." + n: torch.randn(*s, generator=g, dtype=torch.float64) * 0.5 for n, s in
         {"q": (12, 8), "k": (12, 8), "v": (10, 8), "g": (10, 8), "o": (8, 10), "norm": (5,), "a1": (3, 8), "a2": (12, 3),
          "a2.b": (12,)}.items()}
    h = torch.randn(9, 8, generator=g, dtype=torch.float64)
    whole = plain.gla_mixer(h, w, m, 1e-5)
    # the first four tokens leave a state; the rest go on from it
    T = 4
    q = (h @ w["mix.q"].T).view(9, 2, 6)
    k = (h @ w["mix.k"].T).view(9, 2, 6)
    v = (h @ w["mix.v"].T).view(9, 2, 5)
    a = torch.sigmoid((h @ w["mix.a1"].T) @ w["mix.a2"].T + w["mix.a2.b"]).pow(1 / 3.0).view(9, 2, 6)
    S = torch.zeros(2, 6, 5, dtype=torch.float64)
    for t in range(T):
        S = a[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
    rest = plain.gla_mixer(h[T:], w, m, 1e-5, state=S)
    assert float((rest - whole[T:]).abs().max()) < 1e-12
    assert float(a.min()) > 0 and float(a.max()) < 1


def test_plain_block_mask_edges():
    m = plain.block_mask(10, 4)
    assert m[3, 0] and m[3, 3] and not m[4, 3] and m[4, 4] and not m[7, 3] and m[7, 4] and not m[3, 4]
    assert torch.equal(plain.block_mask(6, None), torch.tril(torch.ones(6, 6, dtype=torch.bool)))


def test_plain_router_scales_the_input():
    g = torch.Generator().manual_seed(1)
    w = {"mlp.router": torch.tensor([[5.0, 0.0], [-5.0, 0.0]], dtype=torch.float64)}
    for e in range(2):
        for n, s in (("gate", (3, 2)), ("up", (3, 2)), ("down", (2, 3))):
            w[f"mlp.e{e}.{n}"] = torch.randn(*s, generator=g, dtype=torch.float64)
    h = torch.tensor([[1.0, 0.3]], dtype=torch.float64)
    out = plain.routed_ffn(h, w, {"router": {"experts": 2, "top": 1}})
    s = torch.sigmoid(torch.tensor(5.0, dtype=torch.float64))
    u = s * h[0]
    want = (plain.silu(u @ w["mlp.e0.gate"].T) * (u @ w["mlp.e0.up"].T)) @ w["mlp.e0.down"].T
    assert float((out[0] - want).abs().max()) < 1e-12
    assert float((out[0] - s * want / s).abs().max()) < 1e-12 and not torch.allclose(out[0], s * (
        (plain.silu(h[0] @ w["mlp.e0.gate"].T) * (h[0] @ w["mlp.e0.up"].T)) @ w["mlp.e0.down"].T))
