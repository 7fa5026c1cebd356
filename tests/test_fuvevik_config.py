"""The Fuvevik design without a GPU: what a configuration turns into (layer descriptions, which run reads whose
cache, names and shapes of the tensors), refusals, and properties of the plain implementation itself."""
import copy

import pytest
import torch

import plain_fuvevik as plain
import tiny_fuvevik as tf
from blackwellllm_b200.config.registry import ConfigError, parse_config
from blackwellllm_b200.weights.random_init import model_param_specs


def test_registered_under_its_name_and_model_type():
    cfg = parse_config(tf.PAIR)
    assert cfg.architecture == "Fuvevik" and cfg.tie_word_embeddings and cfg.streams == 2
    raw = {k: v for k, v in tf.PAIR.items() if k != "architecture"}
    raw["model_type"] = "fuvevik"
    assert parse_config(raw).architecture == "Fuvevik"


@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_layers_and_schedule(name):
    raw, _ = tf.CONFIGS[name]
    cfg = parse_config(raw)
    assert len(cfg.layers) == len(cfg.schedule) == len(raw["layers"])
    assert cfg.position_embedding is not None and cfg.position_embedding.base == 10000.0
    assert cfg.streams == raw.get("streams")
    for i, (layer, spec, entry) in enumerate(zip(raw["layers"], cfg.layers, cfg.schedule)):
        m = layer["mixer"]
        a = spec.mixer
        assert (a.num_heads, a.num_kv_heads, a.head_dim) == (m["heads"], m["kv_heads"], m["dim"])
        assert (a.v_head_dim or a.head_dim) == m["vdim"] and a.softmax_scale == m["scale"]
        assert a.qk_norm == "head" and a.sink and a.output_gate and not a.qkv_bias and a.window is None and a.chunk is None
        assert a.q_temperature == ((m["q_temp"]["coef"], m["q_temp"]["every"]) if "q_temp" in m else None)
        assert entry.layer == i and entry.cache_of == m.get("kv_from") and a.shares_kv == ("kv_from" in m)
        assert spec.block == ("hyper" if "streams" in raw else "prenorm")
        assert spec.mixer_norm.offset == 1.0 and spec.mixer_norm.eps == raw["norm"]["eps"]
        f = layer["mlp"]
        if f is None:
            assert spec.ffn is None
        elif f["kind"] == "dense":
            assert spec.ffn.kind == "dense_mlp" and spec.ffn.intermediate_size == f["ff"] and spec.ffn.activation == "relu2"
        else:
            r = spec.ffn
            assert (r.num_experts, r.identity_experts, r.top_k) == (f["router"]["experts"], f["router"]["identity"], f["router"]["top"])
            assert r.score == "softmax" and r.renormalize and not r.scale_input and r.choice_bias == "correction"
            assert r.activation == "clamped_swish" and r.act_limit == f["expert"]["limit"] and r.act_alpha == 1.702
            assert r.renorm_eps == 1e-20
            assert (r.shared is None) == ("shared" not in f)
            if r.shared is not None:
                assert (r.shared.intermediate_size, r.shared.act_limit) == (f["shared"]["ff"], f["shared"]["limit"])


def test_names_and_shapes():
    specs = model_param_specs(tf.PAIR)
    shapes = {k: tuple(v.shape) for k, v in specs.items() if not v.optional}
    assert "head" in specs and specs["head"].optional          # the embedding table is the head
    assert shapes["embed"] == (210, 64) and shapes["final.norm"] == (64,)
    assert shapes["l0.mix.q"] == (128, 64) and shapes["l0.mix.k"] == (64, 64) and shapes["l0.mix.v"] == (32, 64)
    assert shapes["l0.mix.g"] == (64, 64) and shapes["l0.mix.o"] == (64, 64)
    assert shapes["l0.mix.q.norm"] == (32,) and shapes["l0.mix.k.norm"] == (32,) and shapes["l0.mix.sink"] == (4,)
    assert shapes["l0.mlp.router"] == (7, 64) and shapes["l0.mlp.correction"] == (7,)
    assert shapes["l0.mlp.e4.gate"] == (48, 64) and shapes["l0.mlp.e4.down"] == (64, 48) and "l0.mlp.e5.gate" not in shapes
    assert shapes["l0.mlp.shared.up"] == (32, 64)
    assert shapes["l0.hc1.in"] == (2,) and shapes["l0.hc2.mix"] == (2, 2)
    # a layer that borrows keys and values has none of their tensors; a layer without feed-forward has no second sublayer
    for absent in ("l1.mix.k", "l1.mix.v", "l1.mix.k.norm", "l2.norm2", "l2.hc2.in", "l2.mlp.up"):
        assert absent not in specs
    assert shapes["l1.mlp.up"] == (96, 64) and shapes["l1.mlp.down"] == (64, 96) and "l1.mix.q.norm" in shapes
    assert not any(".hc" in k for k in model_param_specs(tf.PLAIN))   # no copies: no such tensors


def test_one_copy_may_come_without_its_tensors():
    specs = model_param_specs(tf.SINGLE)
    assert specs["l0.hc1.mix"].optional and specs["l0.hc1.mix"].shape == (1, 1)
    assert not model_param_specs(tf.PAIR)["l0.hc1.mix"].optional


@pytest.mark.parametrize("change, needle", [
    (lambda r: r["layers"][1]["mixer"].update(kv_from=1), "earlier layer"),
    (lambda r: r["layers"][2]["mixer"].update(kv_from=1), "no keys and values of its own"),
    (lambda r: r["layers"][1]["mixer"].update(dim=16), "differ"),
    (lambda r: r["layers"][0]["mixer"].update(heads=3), "multiple"),
    (lambda r: r["layers"][0].update(type="gla"), "not a mixer"),
    (lambda r: r["layers"][1]["mlp"].update(kind="swiglu"), "not a feed-forward"),
    (lambda r: r["layers"][0]["mlp"]["router"].update(top=8), "exceeds"),
    (lambda r: r.update(streams=0), "streams"),
    (lambda r: r["norm"].update(eps=0), "eps"),
    (lambda r: r["layers"][0]["mixer"]["q_temp"].update(every=0), "every"),
    (lambda r: r["layers"][0]["mixer"].pop("scale"), "scale"),
])
def test_refusals(change, needle):
    raw = copy.deepcopy(tf.PAIR)
    change(raw)
    with pytest.raises(ConfigError, match=needle):
        parse_config(raw)


# ------------------------------------------------------------------ the plain implementation itself

def test_plain_sink_takes_weight_from_every_row():
    scores = torch.randn(2, 5, 5, dtype=torch.float64)
    scores = scores.masked_fill(torch.triu(torch.ones(5, 5, dtype=torch.bool), 1)[None], float("-inf"))
    sink = torch.tensor([0.3, -20.0], dtype=torch.float64)
    p = plain.sink_softmax(scores, sink)
    assert torch.all(p.sum(-1) < 1.0)
    assert torch.allclose(p[1], torch.softmax(scores[1], -1), atol=1e-8)       # a sink far below the scores vanishes
    assert torch.allclose(p[0, 0, 0], 1.0 / (1.0 + torch.exp(sink[0] - scores[0, 0, 0])))


def test_plain_temperature_steps_with_the_period():
    p = torch.arange(0, 30)
    t = plain.query_temperature(p, {"coef": 0.5, "every": 7})
    assert float(t[5]) == 1.0 and float(t[6]) == pytest.approx(1.0 + 0.5 * torch.log(torch.tensor(2.0)).item())
    assert float(t[12]) == float(t[6]) and float(t[13]) > float(t[12])
    assert torch.all(plain.query_temperature(p, None) == 1.0)


def test_plain_position_vectors():
    v = plain.position_vectors(torch.tensor([0, 3]), 6, torch.float64)
    assert torch.allclose(v[0], torch.tensor([0.0, 1.0, 0.0, 1.0, 0.0, 1.0], dtype=torch.float64))
    f = 10000.0 ** (-2.0 / 6)
    assert v[1, 2].item() == pytest.approx(torch.sin(torch.tensor(3.0 * f, dtype=torch.float64)).item())
    assert v[1, 1].item() == pytest.approx(torch.cos(torch.tensor(3.0, dtype=torch.float64)).item())


def test_plain_experts_that_return_their_input_and_the_choice_bias():
    g = torch.Generator().manual_seed(0)
    H, F = 8, 4
    f = {"router": {"experts": 2, "identity": 2, "top": 1}, "expert": {"ff": F, "limit": 1.0}}
    w = {"mlp.router": torch.zeros(4, H, dtype=torch.float64), "mlp.correction": torch.tensor([0.0, 0.0, 0.0, 1.0], dtype=torch.float64)}
    for e in range(2):
        w[f"mlp.e{e}.gate"], w[f"mlp.e{e}.up"] = torch.randn(F, H, generator=g).double(), torch.randn(F, H, generator=g).double()
        w[f"mlp.e{e}.down"] = torch.randn(H, F, generator=g).double()
    h = torch.randn(3, H, generator=g).double()
    # equal scores: the correction alone decides; the weight is the score renormalised (one choice: 1), the output the input
    assert torch.allclose(plain.moe_ffn(h, w, f), h)
    w["mlp.correction"] = torch.tensor([1.0, 0.0, 0.0, 0.0], dtype=torch.float64)
    want = plain.clamped_expert(h, w["mlp.e0.gate"], w["mlp.e0.up"], w["mlp.e0.down"], 1.0)
    assert torch.allclose(plain.moe_ffn(h, w, f), want)


def test_plain_borrowed_keys_are_the_lenders():
    raw, _ = tf.CONFIGS["pair"]
    W = tf.make_tensors(raw, 3, dtype=torch.float32)
    ids = tf.prompt(12, raw["vocab"], 1)
    a = plain.plain_forward(raw, W, ids)
    W2 = dict(W)
    W2["l0.mix.k"] = W["l0.mix.k"] * 1.5            # the lender's keys change: so do the borrowers' scores
    b = plain.plain_forward(raw, W2, ids)
    assert not torch.allclose(a, b)
    streams_a, streams_b = [], []
    plain.plain_forward(raw, W, ids, streams_after_layers=streams_a)
    raw2 = copy.deepcopy(raw)
    raw2["layers"] = raw2["layers"][:1]
    W1 = {k: v for k, v in W.items() if not k.startswith(("l1.", "l2."))}
    plain.plain_forward(raw2, W1, ids, streams_after_layers=streams_b)
    assert torch.allclose(streams_a[0], streams_b[0])


# ------------------------------------------------------------------ the new options beside the older ones

def test_attention_options_combine_with_the_older_ones():
    """The gate and the sink go with biases, a whole-projection norm and a rotation too: the gate's rows ride in the
    q/k/v product where the per-head kernel follows it (with zero biases for them), else they are a product of their own."""
    from blackwellllm_b200.config.specs import AttentionSpec, NoPositionSpec, RopeSpec
    from blackwellllm_b200.parts import BuildContext, build_mixer
    ctx = BuildContext(torch.device("cpu"), torch.float32)
    H, nh, nkv, hd = 32, 4, 2, 8

    def tensors(mixer):
        return {p.name: torch.randn(p.shape) for p in mixer.param_specs()}

    a = build_mixer(AttentionSpec(nh, nkv, hd, qkv_bias=True, position=NoPositionSpec(), qk_norm_eps=1e-5, qk_norm="head",
                                  sink=True, output_gate=True), H, ctx)
    names = {p.name: p.shape for p in a.param_specs()}
    assert names["q_norm.weight"] == (hd,) and names["sinks"] == (nh,) and names["g_proj.weight"] == (nh * hd, H)
    a.bind(tensors(a))
    assert a.gate is None and a.qkv.weight.shape == ((nh + 2 * nkv) * hd + nh * hd, H) and a.g_off == (nh + 2 * nkv) * hd
    assert a.qkv.bias.numel() == a.qkv.weight.shape[0] and float(a.qkv.bias[a.g_off:].abs().max()) == 0.0
    b = build_mixer(AttentionSpec(nh, nkv, hd, qkv_bias=False, position=RopeSpec(10000.0, hd), qk_norm_eps=1e-5,
                                  output_gate=True), H, ctx)
    assert {p.name: p.shape for p in b.param_specs()}["q_norm.weight"] == (nh * hd,)
    b.bind(tensors(b))
    assert b.gate is not None and b.qkv.weight.shape == ((nh + 2 * nkv) * hd, H)     # the whole-projection kernel has fixed rows
    c = build_mixer(AttentionSpec(nh, nkv, hd, qkv_bias=False, position=NoPositionSpec(), qk_norm_eps=1e-5, qk_norm="head",
                                  shares_kv=True), H, ctx)
    assert sorted(p.name for p in c.param_specs()) == ["o_proj.weight", "q_norm.weight", "q_proj.weight"]
    with pytest.raises(ValueError):
        build_mixer(AttentionSpec(nh, nkv, hd, qkv_bias=True, position=NoPositionSpec(), shares_kv=True), H, ctx)
    with pytest.raises(ValueError):
        build_mixer(AttentionSpec(nh, nkv, hd, qkv_bias=False, position=NoPositionSpec(), qk_norm="row"), H, ctx)


def test_routed_feed_forward_options_are_checked():
    from blackwellllm_b200.config.specs import RoutedFFNSpec
    from blackwellllm_b200.parts import BuildContext, build_ffn
    ctx = BuildContext(torch.device("cpu"), torch.float32)
    r = build_ffn(RoutedFFNSpec(4, 5, 16, score="softmax", identity_experts=2, choice_bias="correction"), 32, ctx)
    shapes = {p.name: p.shape for p in r.param_specs()}
    assert shapes["router"] == (6, 32) and shapes["correction"] == (6,) and "e3.gate" in shapes and "e4.gate" not in shapes
    with pytest.raises(ValueError):
        build_ffn(RoutedFFNSpec(4, 7, 16, identity_experts=2), 32, ctx)               # more choices than outputs
    with pytest.raises(ValueError):
        build_ffn(RoutedFFNSpec(4, 2, 16, identity_experts=2, scale_input=True), 32, ctx)
    with pytest.raises(ValueError):
        build_ffn(RoutedFFNSpec(4, 2, 16, activation="gelu"), 32, ctx)
