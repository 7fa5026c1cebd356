"""The Fuvevik design on the GPU against its plain implementation (tests/plain_fuvevik.py): each mechanism's
kernels alone, then whole models through Engine.step in every way of cutting and batching, through the
scheduler's generate(), the command line and bin/trace_run."""
import math

import pytest
import torch

import plain_fuvevik as plain
import replay
import tiny_fuvevik as tf

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
# of the largest logit of the compared request.  The sharp comparison is the float32 one; every bfloat16 kernel
# has its own tight test below, and whole bfloat16 models of 48 to 128 channels average little rounding away.
TOL = {"float32": 1e-4, "bfloat16": 5e-2}


@pytest.fixture(scope="module")
def ops():
    from blackwellllm_b200.kernels import ops as o
    return o


def rnd(*shape, seed=0, scale=1.0):
    return torch.randn(*shape, generator=torch.Generator().manual_seed(seed)) * scale


# =============================================================================== mechanisms alone

@pytest.mark.parametrize("H,copies", [(64, 1), (50, 3), (7, 2), (320, 4)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embedding_with_position_vector(ops, H, copies, dtype):
    from blackwellllm_b200.models.decoder import sinusoid_frequencies
    V = 37
    table = rnd(V, H, seed=H).to(dtype)
    ids = torch.randint(0, V, (9,), generator=torch.Generator().manual_seed(1))
    pos = torch.tensor([0, 1, 2, 63, 64, 500, 1023, 4000, 12345])
    out = ops.embed_positions(table.to(DEV), ids.int().to(DEV), pos.int().to(DEV), sinusoid_frequencies(H, 10000.0).to(DEV),
                              copies=copies).cpu().view(9, copies, H)
    want = table[ids].double() + plain.position_vectors(pos, H, torch.float64)
    # the angle is a float32 product of the position and a float32 frequency: its rounding grows with the position
    bound = 2e-6 + pos.double() * 2.0 ** -22
    for c in range(copies):
        assert torch.all((out[:, c].double() - want).abs().max(dim=1).values <= bound)
    plain_rows = ops.embed_positions(table.to(DEV), ids.int().to(DEV), pos.int().to(DEV), None, copies=1).cpu()
    assert torch.equal(plain_rows, table[ids].float())


@pytest.mark.parametrize("S", [1, 2, 3, 4, 8])
@pytest.mark.parametrize("H", [48, 50, 320])
def test_copies_of_the_stream_write_then_read(ops, S, H):
    T = 11
    xs = rnd(T, S, H, seed=S * H)
    y = rnd(T, H, seed=1)
    mix, w_out, w_in = torch.eye(S) + rnd(S, S, seed=2, scale=0.3), rnd(S, seed=3), rnd(S, seed=4)
    gain = 1.0 + rnd(H, seed=5, scale=0.3)
    eps = 1e-5
    new = plain.hyper_write(xs.double().transpose(0, 1), y.double(), mix.double(), w_out.double())      # [S, T, H]
    u = plain.hyper_read(new, w_in.double())
    want = plain.unit_rms(u, eps) * gain.double()
    d = lambda t: t.to(DEV).contiguous()
    # write + read + norm in one kernel
    streams = d(xs.reshape(T, S * H))
    got = ops.hc_step(streams, S, d(y), d(mix), d(w_out), in_w=d(w_in), gain=d(gain), eps=eps, out_dtype=torch.float32)
    assert float((got.cpu().double() - want).abs().max()) <= 1e-5 * float(want.abs().max())
    assert float((streams.cpu().view(T, S, H).transpose(0, 1).double() - new).abs().max()) <= 1e-5 * float(new.abs().max())
    # read alone (the first read of a model), without a norm (the plain sum of the copies)
    streams = d(xs.reshape(T, S * H))
    got = ops.hc_step(streams, S, in_w=d(torch.ones(S)))
    assert float((got.cpu().double() - xs.double().sum(1)).abs().max()) <= 1e-5
    assert torch.equal(streams.cpu(), xs.reshape(T, S * H))
    # write alone
    ops.hc_step(streams, S, d(y), d(mix), d(w_out))
    assert float((streams.cpu().view(T, S, H).transpose(0, 1).double() - new).abs().max()) <= 1e-5 * float(new.abs().max())
    # chosen rows only, bfloat16 out: the copies stay as they are
    streams = d(xs.reshape(T, S * H))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32)
    got = ops.hc_step(streams, S, d(y), d(mix), d(w_out), in_w=d(w_in), gain=d(gain), eps=eps, rows=d(rows),
                      out_dtype=torch.bfloat16)
    assert torch.equal(streams.cpu(), xs.reshape(T, S * H))
    assert float((got.cpu().double() - want[rows.long()]).abs().max()) <= 1e-2 * float(want.abs().max())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,dq,dv,has_kv,extra", [(4, 2, 32, 16, True, 64), (3, 1, 24, 40, True, 0), (6, 3, 96, 96, False, 576),
                                                       (2, 2, 64, 64, True, 128), (5, 5, 8, 8, False, 0)])
def test_per_head_norm_temperature_and_append(ops, out_dtype, nh, nkv, dq, dv, has_kv, extra):
    from test_kernels_gpu import FakeBatch
    page, eps = 8, 1e-5
    step = 16 if out_dtype == torch.bfloat16 else 1
    dpad = -(-max(dq, dv) // step) * step
    q_lens, kv_lens = [5, 1, 2], [5, 64, 130]
    batch = FakeBatch(q_lens, kv_lens)
    T = sum(q_lens)
    width = nh * dq + (nkv * (dq + dv) if has_kv else 0) + extra
    qkv = rnd(T, width, seed=dq + dv)
    qg, kg = 1.0 + rnd(dq, seed=1, scale=0.3), 1.0 + rnd(dq, seed=2, scale=0.3)
    blocks = [-(-k // page) for k in kv_lens]
    num_pages = sum(blocks) + 2
    table = torch.full((3, max(blocks)), -1, dtype=torch.int32)
    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(3)).tolist()
    for r, b in enumerate(blocks):
        table[r, :b] = torch.tensor([perm.pop() for _ in range(b)], dtype=torch.int32)
    kp = torch.full((num_pages, nkv, page, dpad), 7.0, dtype=out_dtype, device=DEV)
    vp = torch.full((num_pages, nkv, page, dpad), 7.0, dtype=out_dtype, device=DEV)
    coef, every = 0.6, 5
    q = ops.head_norm_rope_append(qkv.to(DEV), batch, table.to(DEV), None, 0, False, qg.to(DEV), kg.to(DEV) if has_kv else None,
                                  eps, kp, vp, nh, nkv, dq, dv, has_kv=has_kv, q_temp=(coef, every)).cpu().double()
    pos = batch.positions.cpu()
    temp = plain.query_temperature(pos, {"coef": coef, "every": every})
    want_q = plain.plain_gain_norm(qkv[:, :nh * dq].double().view(T, nh, dq), qg.double(), eps) * temp[:, None, None]
    tol = 1e-5 if out_dtype == torch.float32 else 1e-2
    q = q.view(T, nh, dpad)
    assert float((q[..., :dq] - want_q).abs().max()) <= tol * float(want_q.abs().max())
    assert float(q[..., dq:].abs().max()) == 0.0 if dpad > dq else True
    if not has_kv:
        assert float((kp.float() - 7.0).abs().max()) == 0.0 and float((vp.float() - 7.0).abs().max()) == 0.0
        return
    want_k = plain.plain_gain_norm(qkv[:, nh * dq:nh * dq + nkv * dq].double().view(T, nkv, dq), kg.double(), eps)
    want_v = qkv[:, (nh + nkv) * dq:(nh + nkv) * dq + nkv * dv].double().view(T, nkv, dv)
    req = batch.req_of_token.cpu()
    for t in range(T):
        p = int(pos[t])
        pg = int(table[int(req[t]), p // page])
        k_row, v_row = kp[pg, :, p % page].cpu().double(), vp[pg, :, p % page].cpu().double()
        assert float((k_row[:, :dq] - want_k[t]).abs().max()) <= tol * float(want_k.abs().max())
        assert float((v_row[:, :dv] - want_v[t]).abs().max()) <= tol * float(want_v.abs().max())
        assert float(k_row[:, dq:].abs().sum()) == 0.0 and float(v_row[:, dv:].abs().sum()) == 0.0


def _sink_attention(q, k, v, sink, scale):
    """q [L, nh, hd], k/v [L, nkv, hd] float64 -> [L, nh, hd]: causal, with a sink per query head."""
    L, nh, hd = q.shape
    g = nh // k.shape[1]
    kk, vv = k.repeat_interleave(g, dim=1), v.repeat_interleave(g, dim=1)
    s = torch.einsum("ihd,jhd->hij", q, kk) * scale
    s = s.masked_fill(torch.triu(torch.ones(L, L, dtype=torch.bool), 1)[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", plain.sink_softmax(s, sink), vv)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,page", [(4, 2, 48, 8), (2, 2, 64, 16), (8, 2, 128, 16), (6, 3, 96, 16), (3, 1, 16, 32)])
def test_attention_with_a_sink(ops, dtype, nh, nkv, hd, page):
    """Prompt portions from position 0 and continued, decode tokens with one and with many key slices, a
    two-token portion; sinks from far below the scores to far above them."""
    from test_kernels_gpu import ATT_TOL, FakeBatch, paged_case
    q_lens = [150, 1, 1, 2, 77, 1]
    kv_lens = [150, 900, 17, 130, 400, 1]
    q, kp, vp, table, refs = paged_case(q_lens, kv_lens, nh, nkv, hd, page, dtype, seed=hd + nh)
    sink = torch.linspace(-6.0, 5.0, nh)
    out = ops.paged_attention(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, None, 0.2, sink=sink.to(DEV))
    ref = torch.cat([_sink_attention(qq.double(), kk.double(), vv.double(), sink.double(), 0.2)[start:].reshape(-1, nh * hd)
                     for qq, kk, vv, start in refs])
    assert not torch.isnan(out).any()
    assert float((out.double().cpu() - ref).abs().max()) <= ATT_TOL[dtype] * float(ref.abs().max())
    none = ops.paged_attention(q, kp, vp, FakeBatch(q_lens, kv_lens), table, nh, None, 0.2)
    assert float((none.double().cpu() - ref).abs().max()) > 10 * ATT_TOL[dtype] * float(ref.abs().max())   # the sink shows


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [48, 64])
@pytest.mark.parametrize("q_len", [1, 2, 50])
def test_a_loud_sink_and_a_loud_far_key(ops, dtype, hd, q_len):
    """All scores of the last query are 0 but one far key's, hundreds of positions back: the row returns that
    key's value, whether it is the first token of the sequence, the last of a page or the first of one.  A
    sink that dwarfs every score silences a head; one of exactly the keys' weight halves it."""
    from test_kernels_gpu import FakeBatch, paged_case
    nh, nkv, page = 4, 2, 16
    for loud, L in [(0, 700), (15, 700), (16, 701), (333, 1000), (L0 := 640, L0 + q_len)]:
        def spike(r, q, k, v):
            k[loud] = 0
            k[loud, :, 0] = 8.0
            q[-1] = 0
            q[-1, :, 0] = 5.0          # score 40 against 0 everywhere else
            v[loud] = 5.0
        q, kp, vp, table, _ = paged_case([q_len], [L], nh, nkv, hd, page, dtype, seed=2, spike=spike)
        sink = torch.tensor([-30.0, 0.0, 40.0, 90.0])
        out = ops.paged_attention(q, kp, vp, FakeBatch([q_len], [L]), table, nh, None, 1.0, sink=sink.to(DEV))
        last = out[-1].float().cpu().view(nh, hd)
        assert float((last[0] - 5.0).abs().max()) < 0.05 and float((last[1] - 5.0).abs().max()) < 0.05, (loud, L)
        assert float((last[2] - 2.5).abs().max()) < 0.05, (loud, L)        # exp(40) beside the key's exp(40)
        assert float(last[3].abs().max()) < 1e-6, (loud, L)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_output_gate_and_activations(ops, dtype):
    T, nh, dv, dpad = 9, 3, 24, 32
    o = rnd(T, nh * dpad, seed=1).to(dtype)
    g = rnd(T, nh * dv + 40, seed=2)
    got = ops.sigmoid_gate(o.clone().to(DEV), g.to(DEV)[:, 40:], nh, dv).cpu().double().view(T, nh, dpad)
    want = o.double().view(T, nh, dpad)[..., :dv] * torch.sigmoid(g[:, 40:].double()).view(T, nh, dv)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert float((got[..., :dv] - want).abs().max()) <= tol * float(want.abs().max()) and float(got[..., dv:].abs().max()) == 0.0
    gu = rnd(T, 2 * 40, seed=3, scale=2.0)
    limit = 1.3
    a = ops.glu(gu.to(DEV), ops.ACT_CLAMPED_SWISH, limit, 1.702, out_dtype=dtype).cpu().double()
    gg, uu = gu[:, :40].double().clamp(max=limit), gu[:, 40:].double().clamp(-limit, limit)
    want = gg * torch.sigmoid(1.702 * gg) * (uu + 1.0)
    assert float((a - want).abs().max()) <= tol * float(want.abs().max())
    assert float(a.max()) <= limit * (limit + 1.0) + 1e-2                     # the limits hold
    s = ops.glu(gu.to(DEV), ops.ACT_SILU, out_dtype=dtype).cpu().double()
    assert float((s - gu[:, :40].double() * torch.sigmoid(gu[:, :40].double()) * gu[:, 40:].double()).abs().max()) <= tol * 8
    r = ops.unary_act(gu.to(DEV), ops.ACT_RELU2, out_dtype=dtype).cpu().double()
    assert float((r - torch.relu(gu.double()) ** 2).abs().max()) <= tol * float(gu.abs().max()) ** 2


def _routed_part(ops, dtype, E, identity, top, F, H, limit, shared=None, seed=0):
    from blackwellllm_b200.config.specs import RoutedFFNSpec, SwiGLUSpec
    from blackwellllm_b200.parts import BuildContext, build_ffn
    sh = SwiGLUSpec(shared[0], activation="clamped_swish", act_limit=shared[1], act_alpha=1.702, names=("gate", "up", "down")) \
        if shared else None
    spec = RoutedFFNSpec(E, top, F, score="softmax", renormalize=True, scale_input=False, identity_experts=identity,
                         choice_bias="correction", renorm_eps=1e-20, activation="clamped_swish", act_limit=limit,
                         act_alpha=1.702, shared=sh)
    part = build_ffn(spec, H, BuildContext(DEV, dtype))
    w = {}
    for p in part.param_specs():
        t = rnd(*p.shape, seed=seed + len(w), scale=0.3 if p.name != "router" else 1.0)
        if p.name == "correction":
            t = t * 0.3
        w[p.name] = t.to(dtype)
    part.bind({k: v.to(DEV) for k, v in w.items()})
    f = {"router": {"experts": E, "identity": identity, "top": top}, "expert": {"ff": F, "limit": limit}}
    if shared:
        f["shared"] = {"ff": shared[0], "limit": shared[1]}
    return part, {"mlp." + k: v.double() for k, v in w.items()}, f


@pytest.mark.parametrize("E,identity,top,F,H,shared", [(5, 2, 2, 48, 64, (32, 0.8)), (3, 0, 3, 64, 96, None), (2, 3, 1, 20, 50, (12, 1.0)),
                                                       (16, 4, 4, 64, 320, (96, 1.0)), (6, 1, 7, 16, 48, None)])
@pytest.mark.parametrize("T", [1, 5, 300])
def test_routed_ffn_float32(ops, E, identity, top, F, H, shared, T):
    """Softmax scores over experts and the outputs that return the input, a correction on the choice only, weights
    renormalised, the clamped activation, a shared expert: written and added, few tokens (one fused kernel in
    front) and many (three); a token's result does not depend on its batch, bit for bit."""
    part, w, f = _routed_part(ops, torch.float32, E, identity, top, F, H, 1.2, shared, seed=E)
    x = rnd(T, H, seed=T)
    want = plain.moe_ffn(x.double(), w, f)
    out = torch.full((T, H), 3.0, device=DEV)
    part.forward(x.to(DEV), out, None, accumulate=False)
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    assert float((out.cpu().double() - want).abs().max()) <= 2e-5 * float(want.abs().max())
    acc = torch.full((T, H), 3.0, device=DEV)
    part.forward(x.to(DEV), acc, None)
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    assert float((acc.cpu().double() - 3.0 - want).abs().max()) <= 2e-5 * float(want.abs().max())
    one = torch.zeros((1, H), device=DEV)
    part.forward(x[T // 2:T // 2 + 1].to(DEV), one, None, accumulate=False)
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    assert torch.equal(one[0], out[T // 2])
    # the correction decides the choice, not the weight: with a large one on the last output every token takes it first
    if identity:
        part.bias = part.bias.clone()
        part.bias[-1] = 10.0
        w2 = dict(w)
        w2["mlp.correction"] = w["mlp.correction"].clone()
        w2["mlp.correction"][-1] = 10.0
        part.forward(x.to(DEV), out, None, accumulate=False)
        ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
        want2 = plain.moe_ffn(x.double(), w2, f)
        assert float((out.cpu().double() - want2).abs().max()) <= 2e-5 * float(want2.abs().max())


@pytest.mark.parametrize("T", [3, 200])
def test_routed_ffn_bfloat16_all_experts(ops, T):
    """bfloat16 on the tensor cores with every expert used (no choice that rounding could turn): the clamped
    activation in the grouped product's epilogue, identity outputs in the sum."""
    E, identity, F, H = 3, 2, 64, 96
    part, w, f = _routed_part(ops, torch.bfloat16, E, identity, E + identity, F, H, 1.0, (32, 0.9), seed=9)
    assert part.tc
    x = rnd(T, H, seed=T).to(torch.bfloat16)
    want = plain.moe_ffn(x.double(), w, f)
    out = torch.zeros((T, H), device=DEV)
    part.forward(x.to(DEV), out, None, accumulate=False)
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    assert float((out.cpu().double() - want).abs().max()) <= 2e-2 * float(want.abs().max())
    assert ops.moe_tc_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,F", [(64, 96), (50, 30)])
def test_dense_feed_forwards(ops, dtype, H, F):
    from blackwellllm_b200.config.specs import DenseMLPSpec, SwiGLUSpec
    from blackwellllm_b200.parts import BuildContext, build_ffn
    ctx = BuildContext(DEV, dtype)
    x = rnd(7, H, seed=1).to(dtype)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    up, down, gate = rnd(F, H, seed=2, scale=0.3).to(dtype), rnd(H, F, seed=3, scale=0.3).to(dtype), rnd(F, H, seed=4, scale=0.3).to(dtype)
    part = build_ffn(DenseMLPSpec(F), H, ctx)
    part.bind({"up": up.to(DEV), "down": down.to(DEV)})
    out = torch.zeros((7, H), device=DEV)
    part.forward(x.to(DEV), out, None, accumulate=False)
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    want = plain.dense_ffn(x.double(), {"mlp.up": up.double(), "mlp.down": down.double()})
    assert float((out.cpu().double() - want).abs().max()) <= tol * float(want.abs().max())
    part = build_ffn(SwiGLUSpec(F, activation="clamped_swish", act_limit=0.7, act_alpha=1.702, names=("gate", "up", "down")), H, ctx)
    part.bind({"gate": gate.to(DEV), "up": up.to(DEV), "down": down.to(DEV)})
    part.forward(x.to(DEV), out, None)                     # added to what is there
    ops.resolve_pending()      # a last product of few tokens leaves its sum to the next reader
    want = want + plain.clamped_expert(x.double(), gate.double(), up.double(), down.double(), 0.7)
    assert float((out.cpu().double() - want).abs().max()) <= tol * float(want.abs().max())


# =============================================================================== whole models through the engine

_models = {}
_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def model(name, dtype):
    key = (name, dtype)
    if key not in _models:
        raw, page = tf.CONFIGS[name]
        tensors = tf.make_tensors(raw, seed=7, dtype=_DT[dtype])
        reqs = {f"r{i}": tf.prompt(n, raw["vocab"], 50 + i) for i, n in enumerate([70, 33, 131, 2, 90])}
        ref = {rid: plain.plain_forward(raw, tensors, ids) for rid, ids in reqs.items()}
        _models[key] = (raw, page, tensors, reqs, ref)
    return _models[key]


def engine_for(name, dtype, **kw):
    from blackwellllm_b200.engine.engine import Engine
    raw, page, tensors, _, _ = model(name, dtype)
    opts = dict(dtype=dtype, page_size=page, num_pages=64, max_requests=4, max_batch_tokens=1 << 16)
    opts.update(kw)
    return Engine.from_tensors(raw, tensors, **opts)


def routed(name):
    """Whether a configuration's feed-forwards choose among experts."""
    return any(l["mlp"] and l["mlp"]["kind"] == "moe"
               and l["mlp"]["router"]["top"] < l["mlp"]["router"]["experts"] + l["mlp"]["router"]["identity"]
               for l in tf.CONFIGS[name][0]["layers"])


def check_rows(rows, ref, dtype, what, is_routed=True):
    """rows {(rid, pos): logits}.  float32: every row within the bound.  bfloat16 without a choice among experts:
    the same with its bound.  bfloat16 with a choice: a score that is a near-tie in the plain implementation goes
    the other way now and then, which changes that row altogether; there the rows are judged together: all
    finite, the median within 0.6 of the bound, 4 of 5 within 1.2 of it.  (A wrong key, page or edge moves
    every row it touches by far more; the float32 runs of the same schedules have no such exception.)"""
    errs = []
    for (rid, p), row in rows.items():
        want = ref[rid][p]
        err = float((row.double().cpu() - want).abs().max()) / float(ref[rid].abs().max())
        assert err == err and err != float("inf"), (what, rid, p)
        errs.append((err, rid, p))
    errs.sort()
    if dtype == "float32" or not is_routed:
        assert errs[-1][0] <= TOL[dtype], (what, errs[-1])
    else:
        assert errs[len(errs) // 2][0] <= 0.6 * TOL[dtype], (what, "median", errs[len(errs) // 2])
        assert errs[(4 * len(errs)) // 5][0] <= 1.2 * TOL[dtype], (what, "4 of 5", errs[(4 * len(errs)) // 5])


def run_steps(eng, steps):
    """steps: [[(rid, tokens, start)]]: every position's logits by (rid, position)."""
    from blackwellllm_b200.engine.engine import StepEntry
    rows = {}
    for step in steps:
        out = eng.step([StepEntry(rid, toks, list(range(len(toks)))) for rid, toks, _ in step]).cpu()
        at = 0
        for rid, toks, start in step:
            for i in range(len(toks)):
                rows[(rid, start + i)] = out[at + i].clone()
            at += len(toks)
    return rows


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_whole_prompts_and_the_stream_after_every_layer(name, dtype):
    raw, _, tensors, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    streams, want_streams = [], []
    plain.plain_forward(raw, tensors, reqs["r0"], streams_after_layers=want_streams)
    eng.model.stream_hook = lambda pos, h: streams.append(h.double().cpu().clone())
    rows = run_steps(eng, [[("r0", reqs["r0"], 0)]])
    eng.model.stream_hook = None
    assert len(streams) == len(want_streams) == len(raw["layers"])
    if dtype == "float32":
        for i, (got, want) in enumerate(zip(streams, want_streams)):
            assert float((got - want).abs().max()) <= 2e-5 * float(want.abs().max()), f"layer {i}"
    eng.end_request("r0")
    for rid in ("r1", "r2", "r3", "r4"):
        rows.update(run_steps(eng, [[(rid, reqs[rid], 0)]]))
        eng.end_request(rid)
    check_rows(rows, ref, dtype, "whole", routed(name))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_token_by_token_from_the_first_token(name, dtype):
    """Decoding from position 0 (the first tokens of a sequence, every step of the temperature, every page border),
    long enough that the decode steps are replayed from a CUDA graph."""
    _, _, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    ids = reqs["r2"]
    rows = run_steps(eng, [[("r2", [t], i)] for i, t in enumerate(ids)])
    check_rows(rows, ref, dtype, "token by token", routed(name))
    assert eng.graph_kernel_count(1) > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tf.CONFIGS))
@pytest.mark.parametrize("sizes", [(2,), (7, 2, 13, 3, 5, 2, 16, 17, 4, 31, 2), (64, 1, 1, 1, 40, 1)])
def test_portions(name, dtype, sizes):
    _, _, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype)
    rows = {}
    for rid in ("r0", "r2", "r4"):
        ids, at, k, steps = reqs[rid], 0, 0, []
        while at < len(ids):
            n = min(sizes[k % len(sizes)], len(ids) - at)
            steps.append([(rid, ids[at:at + n], at)])
            at, k = at + n, k + 1
        rows.update(run_steps(eng, steps))
        eng.end_request(rid)
    check_rows(rows, ref, dtype, f"portions {sizes}", routed(name))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_unequal_requests_together_and_pages_used_again(name, dtype):
    """A pool that holds two requests: five pass through, portions of one beside single tokens of another; every
    later request gets a slot and pages that an earlier one gave back."""
    raw, page, _, reqs, ref = model(name, dtype)
    eng = engine_for(name, dtype, num_pages=-(-(131 + 90) // page) + 2, max_requests=2)
    waiting = list(reqs.items())
    live, rows = {}, {}
    g = torch.Generator().manual_seed(3)
    while waiting or live:
        while waiting and len(live) < 2:
            rid, ids = waiting.pop(0)
            live[rid] = 0
        step = []
        for rid in list(live):
            ids, at = reqs[rid], live[rid]
            if at >= len(ids) - 6:
                n = 1
            else:
                n = min(int(torch.randint(2, 30, (1,), generator=g)), len(ids) - 6 - at)
            step.append((rid, ids[at:at + n], at))
            live[rid] = at + n
        rows.update(run_steps(eng, [step]))
        for rid in list(live):
            if live[rid] == len(reqs[rid]):
                eng.end_request(rid)
                del live[rid]
    check_rows(rows, ref, dtype, "mixed", routed(name))
    eng.cache.check_invariants()
    assert eng.cache.slots.num_free == 2


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["quad", "pair"])
def test_a_long_request_in_portions_then_decoded(name, dtype):
    """700 tokens: dozens of pages, a temperature that has stepped many times, keys hundreds of positions back;
    prompt portions that start and end inside pages, then 40 tokens one by one (several key slices a token)."""
    raw, page, tensors, _, _ = model(name, dtype)
    ids = tf.prompt(700, raw["vocab"], 999)
    ref = {"long": plain.plain_forward(raw, tensors, ids)}
    eng = engine_for(name, dtype, num_pages=-(-700 // page) + 1, max_requests=1)
    steps, at = [], 0
    for n in (333, 2, 190, 135):
        steps.append([("long", ids[at:at + n], at)])
        at += n
    steps += [[("long", [ids[i]], i)] for i in range(at, 700)]
    check_rows(run_steps(eng, steps), ref, dtype, "long", routed(name))


@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_a_batch_changes_no_bit_of_a_request(name):
    """float32: a request's logits beside other requests equal its logits alone, bit for bit."""
    _, _, _, reqs, _ = model(name, "float32")
    alone = engine_for(name, "float32")
    a = run_steps(alone, [[("r1", reqs["r1"][:20], 0)], [("r1", reqs["r1"][20:21], 20)]])
    both = engine_for(name, "float32")
    b = run_steps(both, [[("r4", reqs["r4"][:9], 0), ("r1", reqs["r1"][:20], 0), ("r0", reqs["r0"][:3], 0)],
                         [("r0", reqs["r0"][3:4], 3), ("r1", reqs["r1"][20:21], 20), ("r4", reqs["r4"][9:40], 9)]])
    for key, row in a.items():
        assert torch.equal(row, b[key]), key


def test_the_borrower_reads_what_the_lender_wrote_in_the_same_step():
    """A layer that borrows keys and values sees the lender's rows of THIS step's tokens, portion by portion: changing
    the lender's key weights changes the borrower's output, and the borrower appends nothing of its own (the pool of
    the lender's geometry is the only one)."""
    raw, page, tensors, reqs, ref = model("pair", "float32")
    eng = engine_for("pair", "float32")
    assert len(eng.cache.groups) == 1 and eng.model.cache_requests()[1] is None and eng.model.cache_requests()[2] is None
    rows = run_steps(eng, [[("r0", reqs["r0"][:30], 0)], [("r0", reqs["r0"][30:], 30)]])
    check_rows(rows, ref, "float32", "borrowed", False)


@pytest.mark.parametrize("name", list(tf.CONFIGS))
def test_greedy_generation_through_the_entry_point(name, tmp_path):
    """generate() (scheduler, sampling, continuous batching) gives the plain implementation's greedy tokens."""
    import os
    from safetensors.torch import load_file
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, SamplingParams
    raw, page = tf.CONFIGS[name]
    folder = tf.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompts = [tf.prompt(n, raw["vocab"], 80 + n) for n in (5, 40, 1)]
    steps = 12
    llm = BlackwellEngine(folder, InferenceConfig(max_context_length=128, max_batch_size=3), dtype="float32")
    got = llm.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=steps))
    for p, g in zip(prompts, got):
        ids = list(p)
        for _ in range(steps):
            ids.append(int(torch.argmax(plain.plain_forward(raw, W, ids)[-1])))
        assert list(g.token_ids) == ids[len(p):]


def test_command_line_and_position_addressed_calls(tmp_path, capsys):
    import os
    from safetensors.torch import load_file
    from blackwellllm_b200 import BlackwellEngine, InferenceConfig, cli
    name = "single"
    raw, _ = tf.CONFIGS[name]
    folder = tf.make_folder(name, "float32", str(tmp_path))
    W = load_file(os.path.join(folder, "model.safetensors"))
    prompt = tf.prompt(9, raw["vocab"], 4)
    ids = list(prompt)
    for _ in range(6):
        ids.append(int(torch.argmax(plain.plain_forward(raw, W, ids)[-1])))
    want = ids[len(prompt):]
    rc = cli.main(["-m", folder, "--dtype", "float32", "--ctx", "128", "--temperature", "0", "--max-new-tokens", "6",
                   "--prompt-ids", ",".join(map(str, prompt))])
    out = capsys.readouterr().out
    assert rc == 0 and [int(t) for t in out.strip().splitlines()[0].split()] == want
    llm = BlackwellEngine(folder, InferenceConfig(max_context_length=128, max_batch_size=2), dtype="float32")
    nxt = llm.prefill(prompt, start_pos=0, temperature=0.0, seq_id=0)
    got = [nxt]
    for i in range(5):
        nxt = llm.forward(nxt, pos=len(prompt) + i, temperature=0.0, seq_id=0)
        got.append(nxt)
    assert got == want


def test_one_copy_without_its_tensors_is_a_plain_residual_sum():
    raw, page, tensors, reqs, _ = model("single", "float32")
    from blackwellllm_b200.engine.engine import Engine
    bare = {k: v for k, v in tensors.items() if ".hc" not in k}
    eng = Engine.from_tensors(raw, bare, dtype="float32", page_size=page, num_pages=16, max_requests=2)
    raw2 = {k: v for k, v in raw.items() if k != "streams"}
    want = {"r1": plain.plain_forward(raw2, bare, reqs["r1"])}
    check_rows(run_steps(eng, [[("r1", reqs["r1"], 0)]]), want, "float32", "one copy", False)


# =============================================================================== bin/trace_run

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("family", ["tail", "portions", "mixed"])
def test_replay(tmp_path_factory, dtype, family):
    import os
    from safetensors.torch import load_file
    name = "pair"
    raw, page = tf.CONFIGS[name]
    folder = tf.make_folder(name, dtype, str(tmp_path_factory.mktemp("fuvevik")))
    W = load_file(os.path.join(folder, "model.safetensors"))
    reqs = {f"q{i}": tf.prompt(n, raw["vocab"], 200 + i) for i, n in enumerate([40, 97, 50, 70, 130, 65])}
    ref = {rid: plain.plain_forward(raw, W, ids) for rid, ids in reqs.items()}
    if family == "tail":
        steps, max_tokens = replay.trace_tail(reqs)
    elif family == "portions":
        steps, max_tokens = replay.trace_portions(reqs)
    else:
        max_tokens = 384
        steps = replay.trace_mixed(reqs, max_tokens, seed=3)
    rows = replay.run_trace(folder, dtype, steps, max_tokens, raw["vocab"], page_size=page)
    check_rows(rows, ref, dtype, f"replay {family}", routed(name))


# =============================================================================== random configurations

def _random_configuration(rng):
    """A configuration drawn at random: copies of the stream or none, two to five layers, head counts and sizes (equal
    and unequal key and value sizes), borrowers of any earlier lender (with the same or another number of query
    heads), temperature constants or none, every kind of feed-forward or none."""
    import math
    layers = []
    for i in range(rng.randint(2, 5)):
        lenders = [j for j in range(i) if "kv_from" not in layers[j]["mixer"]]
        src = rng.choice(lenders) if lenders and rng.random() < 0.45 else None
        if src is not None:
            m0 = layers[src]["mixer"]
            kv, dim, vdim = m0["kv_heads"], m0["dim"], m0["vdim"]
            heads = kv * rng.choice([1, 2, 4]) if rng.random() < 0.3 else m0["heads"]
        else:
            kv = rng.choice([1, 2, 3])
            heads = kv * rng.choice([1, 2, 4])
            dim = rng.choice([8, 16, 24, 32, 64, 80])
            vdim = dim if rng.random() < 0.6 else rng.choice([8, 16, 40, 64])
        m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": rng.uniform(0.6, 1.6) / math.sqrt(dim)}
        if rng.random() < 0.8:
            m["q_temp"] = {"coef": rng.choice([0.1, 0.5, 1.0]), "every": rng.choice([3, 16, 50])}
        if src is not None:
            m["kv_from"] = src
        r = rng.random()
        if r < 0.15:
            mlp = None
        elif r < 0.5:
            mlp = {"kind": "dense", "ff": rng.choice([24, 64, 100])}
        else:
            E, idn = rng.choice([2, 5, 8]), rng.choice([0, 1, 3])
            mlp = {"kind": "moe", "expert": {"ff": rng.choice([12, 16, 48]), "limit": rng.choice([0.5, 1.5, 7.0])},
                   "router": {"experts": E, "identity": idn, "top": rng.randint(1, min(4, E + idn))}}
            if rng.random() < 0.6:
                mlp["shared"] = {"ff": rng.choice([16, 40]), "limit": rng.choice([0.5, 2.0])}
        layers.append({"type": "attention", "mixer": m, "mlp": mlp})
    raw = {"architecture": "Fuvevik", "vocab": rng.choice([100, 256]), "width": rng.choice([40, 48, 64, 96]),
           "norm": {"eps": rng.choice([1e-6, 1e-5])}, "layers": layers}
    streams = rng.choice([None, 1, 2, 3, 5])
    if streams is not None:
        raw["streams"] = streams
    return raw


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_float32(seed):
    """Whole, and in portions with the last tokens one by one, against the plain implementation."""
    import random
    from blackwellllm_b200.engine.engine import Engine
    rng = random.Random(seed)
    raw = _random_configuration(rng)
    W = tf.make_tensors(raw, seed=100 + seed, dtype=torch.float32)
    L = rng.choice([70, 150])
    ids = tf.prompt(L, raw["vocab"], seed)
    ref = {"a": plain.plain_forward(raw, W, ids)}
    ref["b"] = ref["a"]
    page = rng.choice([8, 16, 32])
    eng = Engine.from_tensors(raw, W, dtype="float32", page_size=page, num_pages=2 * (L // page + 2), max_requests=2)
    steps, at = [[("a", ids, 0)]], 0
    while at < L - 12:
        n = min(rng.choice([2, 3, 17, 40]), L - 12 - at)
        steps.append([("b", ids[at:at + n], at)])
        at += n
    steps += [[("b", [ids[i]], i)] for i in range(at, L)]
    check_rows(run_steps(eng, steps), ref, "float32", f"random configuration {seed}: {raw}", False)
