"""The Nipurax design on the GPU against the plain implementation: each mechanism's part alone,
then whole models through the trace replayer in every way of cutting requests into steps, then
greedy generation through the engine and its scheduler."""

import math

import numpy as np
import pytest
import torch

import plain_nipurax as plain
from gefilix_helpers import check, prompts, write_folder
from helpers import mixed_trace
from test_engine_gpu import step_context
from test_tigesun_gpu import ROUNDINGS, Pages, doubles, i32, judge, paged, rounded, row_errors
from tiny_nipurax import NIPURAX, diff_attention, moe, sink_attention

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
EPS = 1e-5
F64 = torch.float64


def on_device(w, dtype):
    """Matrices in the compute dtype, everything with one axis float32 (the pass vectors too)."""
    return {k: v.cuda().to(dtype if v.dim() == 2 and not k.endswith("step") else torch.float32) for k, v in w.items()}


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
def test_pair_embedding_carries_the_last_token_between_steps(dtype):
    """Two requests in portions, single tokens and a slot that is used again: every row equals the
    plain embedding of the whole sequence, whose first token takes the table's last row."""
    from atomserve_b200 import ops
    from atomserve_b200.ops.status import status_for

    g = torch.Generator().manual_seed(3)
    vocab, d, buckets, mp, mc = 50, 40, 13, 1000003, 7
    cfg = dict(embedding=dict(bigram=dict(buckets=buckets, mul_prev=mp, mul_cur=mc)))
    embed, pairs = rounded(torch.randn(vocab, d, generator=g)), rounded(torch.randn(buckets + 1, d, generator=g))
    seqs = {n: torch.randint(0, vocab, (k,), generator=g).tolist() for n, k in (("a", 23), ("b", 9), ("c", 5))}
    refs = {n: plain.embedding(s, embed, pairs, cfg).float() for n, s in seqs.items()}
    last = torch.zeros(4, 1, dtype=torch.int32, device="cuda")
    status = status_for(torch.device("cuda")).embedding
    at = dict(a=0, b=0, c=0)
    slot = dict(a=2, b=0, c=0)  # c takes b's slot once b has ended
    for step in [[("a", 5), ("b", 1)], [("b", 2), ("a", 1)], [("a", 2)], [("b", 6), ("a", 14)], [("c", 1), ("a", 1)], [("c", 4)]]:
        if step[0][0] == "c" and at["c"] == 0:
            last[0].zero_()  # what the state slots do when a slot is handed out
        lens, starts = [n for _, n in step], [at[r] for r, _ in step]
        ctx = step_context(lens, starts, [slot[r] for r, _ in step])
        ctx.token_ids = i32([t for r, n in step for t in seqs[r][at[r] : at[r] + n]])
        out = ops.pair_embedding(ctx.token_ids, ctx.positions, ctx.req_q_start, ctx.state_slots, last, embed.cuda().to(dtype),
                                 pairs.cuda().to(dtype), mp, mc, status).cpu()  # fmt: skip
        row = 0
        for r, n in step:
            assert torch.equal(out[row : row + n], refs[r][at[r] : at[r] + n]), (r, at[r], n)
            row, at[r] = row + n, at[r] + n
    assert at == {n: len(s) for n, s in seqs.items()}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 100, 256, 1030])
def test_sum_of_two_sublayers_and_both_norms_of_it(dtype, d):
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(d)
    x, y1, y2 = (3 * torch.randn(11, d, generator=g) for _ in range(3))
    g1, g2, bias = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g), torch.randn(d, generator=g)
    s = x.double() + 0.3 * (y1.double() + y2.double())
    out, h1, h2 = ops.residual_dual_norm(x.cuda(), y1.cuda(), y2.cuda(), 0.3, g1.cuda(), g2.cuda(), EPS, dtype)
    check(out, s.float(), torch.float32, "the sum")
    check(h1, plain.rms_norm(s, g1.double(), EPS).float(), dtype, "first norm", 0.01)
    check(h2, plain.rms_norm(s, g2.double(), EPS).float(), dtype, "second norm", 0.01)
    # the mixer alone, no second norm; then a product plus a vector with nothing before it
    out, h1, h2 = ops.residual_dual_norm(x.cuda(), y1.cuda(), None, 2.0, g1.cuda(), None, EPS, dtype)
    assert h2 is None
    check(out, (x.double() + 2.0 * y1.double()).float(), torch.float32, "the sum of one")
    out, h1, _ = ops.residual_dual_norm(None, y1.cuda(), None, 1.0, g2.cuda(), None, EPS, dtype, bias=bias.cuda())
    check(out, (y1 + bias), torch.float32, "a product and a vector")
    check(h1, plain.rms_norm((y1 + bias).double(), g2.double(), EPS).float(), dtype, "its norm", 0.01)


@pytest.mark.parametrize("dtype", DTYPES)
def test_opening_of_a_pass(dtype):
    from atomserve_b200.parts import PartSpec, build_part

    d, T = 72, 13
    g = torch.Generator().manual_seed(1)
    w = {"loop.in": rounded(torch.randn(d, 2 * d, generator=g) * (2 * d) ** -0.5), "loop.step": torch.randn(3, d, generator=g)}
    part = build_part("stream_step", PartSpec("mix_with_input", dict(uses=3, tensor="loop.in", step_tensor="loop.step")), d)
    part.load(on_device(w, dtype))
    part.bind_dtype(dtype)
    x, x0 = rounded(torch.randn(T, d, generator=g)), rounded(torch.randn(T, d, generator=g))
    for t in range(3):
        ref = torch.cat([x, x0], -1).double() @ w["loop.in"].double().T + w["loop.step"][t].double()
        check(part.forward(x.cuda(), x0.cuda(), t, None), ref.float(), torch.float32, f"pass {t}")
    with pytest.raises(ValueError):
        part.forward(x.cuda(), x0.cuda(), 3, None)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("maps,dim,vdim,dims,temp", [(2, 12, 40, 8, None), (2, 20, 24, 20, None), (1, 24, 16, 0, (0.7, 7)), (2, 64, 128, 32, None),
                                                     (1, 64, 64, 0, (0.4, 100)), (2, 48, 64, 24, (1.0, 3)), (1, 16, 16, 16, None)])  # fmt: skip
def test_rotation_query_factor_and_padded_heads(dtype, maps, dim, vdim, dims, temp):
    """Positions near and far (float32 angles), every map turned on its first entries only, the query
    factor at the steps of its logarithm, and zeros wherever a head is wider than what it holds;
    pages are filled with ones beforehand: a slot used again keeps nothing of its former owner."""
    from atomserve_b200 import ops

    H, G, bs = 3, 2, 4
    hd = max(maps * dim, vdim)
    g = torch.Generator().manual_seed(dim + dims)
    positions = [0, 1, 2, 5, 6, 7, 98, 99, 100, 1000, 30000]
    T = len(positions)
    q, k, v = (rounded(torch.randn(T, n, generator=g)) for n in (H * maps * dim, G * maps * dim, G * vdim))
    rot = dict(base=100.0, dims=dims, scaling=dict(factor=4.0, low=1.0, high=4.0, original=64))
    f = plain.rotary_frequencies(rot) if dims else None
    pos = torch.tensor(positions)
    rq = plain.rotate(q.double().view(T, H, maps, dim), pos, f, dims) * plain.query_factor(pos, dict(coef=temp[0], every=temp[1]) if temp else None)[:, None, None, None]
    rk = plain.rotate(k.double().view(T, G, maps, dim), pos, f, dims)
    pages_k = torch.ones(8, G, bs, hd, device="cuda", dtype=dtype)
    pages_v = torch.ones_like(pages_k)
    slots = [21, 0, 31, 13, 14, 3, 8, 9, 18, 24, 15]
    out = ops.qk_prepare_store(torch.cat([q, k, v], 1).cuda().to(dtype), H, G, maps, dim, vdim, hd, i32(positions),
                               inv_freq=f.float().cuda() if dims else None, rotary_dim=dims, temperature=temp, slots=i32(slots),
                               k_cache=pages_k, v_cache=pages_v).float().cpu().view(T, H, maps, hd)  # fmt: skip
    tol = 0.02 if dtype == torch.bfloat16 else 2e-5
    # angles are float32 by the design: position x frequency is off by up to 2^-24 of itself
    slack = (tol * 3 + pos.double() * 2.0**-23 * 5)[:, None, None]

    def close(got, ref):
        return bool(((got.double() - ref).abs() <= slack + tol * ref.abs()).all())

    for j in range(maps):
        assert close(out[:, :, j, j * dim : (j + 1) * dim], rq[:, :, j])
        rest = torch.cat([out[:, :, j, : j * dim], out[:, :, j, (j + 1) * dim :]], -1)
        assert not rest.any()
    got_k = pages_k.float().cpu().permute(0, 2, 1, 3).reshape(-1, G, hd)[slots]
    got_v = pages_v.float().cpu().permute(0, 2, 1, 3).reshape(-1, G, hd)[slots]
    assert close(got_k[:, :, : maps * dim], rk.reshape(T, G, maps * dim))
    assert not got_k[:, :, maps * dim :].any() and not got_v[:, :, vdim:].any()
    assert torch.equal(got_v[:, :, :vdim], v.view(T, G, vdim))
    untouched = sorted(set(range(8 * bs)) - set(slots))
    assert (pages_k.float().cpu().permute(0, 2, 1, 3).reshape(-1, G, hd)[untouched] == 1).all()


def attend(q_parts, pages, requests, lens, starts, scale, **more):
    from atomserve_b200 import ops

    ctx = step_context(lens, starts)
    q = torch.cat(q_parts).cuda().to(pages.dtype).contiguous()
    return ops.paged_attention(q, pages.pools[0], pages.pools[1], pages.table(requests), ctx.req_q_start, ctx.req_pos_start,
                               num_requests=len(lens), max_context=ctx.max_context, window=None, scale=scale,
                               host_q_lens=lens, **more).float().cpu()  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk,bs,hd,G", [(10, 16, 24, 1), (64, 16, 96, 2), (16, 16, 64, 2), (100, 16, 128, 4), (1, 4, 16, 1), (33, 8, 128, 1), (300, 16, 64, 1)])
def test_one_key_stands_out_at_the_chunks_edges(dtype, chunk, bs, hd, G):
    """All keys are zero but one with a large score, whose value is e_1: a query sees it exactly when
    it lies in the query's own chunk and not ahead, so the result is known in closed form: the chunk's
    first and last position, the positions around its borders, chunks that end inside a page and on a
    page border, from single tokens and from portions that start before the chunk does."""
    H, scale, T = 2 * G, 0.5, 700
    q = torch.zeros(1, H, hd)
    q[:, :, 0] = 8.0
    marks = sorted({0, chunk - 1, chunk, 2 * chunk - 1, 5 * chunk, 5 * chunk + chunk // 2, (T // chunk) * chunk - 1, T - 1} & set(range(T)))
    for mark in marks:
        k, v = torch.zeros(T, G, hd), torch.zeros(T, G, hd)
        k[mark, :, 0], v[mark, :, 1] = 2.5, 1.0
        pages = Pages([(G, hd), (G, hd)], bs, dtype, blocks=T // bs + 5, seed=mark)
        pages.put("r", k, v)
        first, end = mark - mark % chunk, min(mark - mark % chunk + chunk, T)
        for p in sorted({first - 1, first, mark - 1, mark, mark + 1, end - 1, end, end + 1, T - 1} & set(range(T))):
            seen = first <= mark <= p < end
            want = math.exp(10.0) / (math.exp(10.0) + p - (p - p % chunk)) if seen else 0.0
            one = attend([q], pages, ["r"], [1], [p], scale, chunk=chunk)[0, :, 1].tolist()
            lo = max(0, p - 40)
            many = attend([q.expand(p + 1 - lo, H, hd)], pages, ["r"], [p + 1 - lo], [lo], scale, chunk=chunk)[-1, :, 1].tolist()
            for got in (one, many):
                assert np.allclose(got, want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6), (mark, p, got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,bs,G", [(24, 16, 1), (64, 16, 2), (128, 16, 4), (40, 8, 3)])
def test_capped_scores_far_keys_and_the_sink(dtype, hd, bs, G):
    """One key among hundreds of zero keys has raw score 40; capped at 10 it weighs exp(10 tanh 4)
    against the other keys' exp(0) and the sink's exp(s_h), whatever its distance. With a sink so
    large that it takes nearly everything the output shrinks accordingly; a head's own sink counts."""
    H, scale, T, cap = 2 * G, 0.5, 600, 10.0
    q = torch.zeros(1, H, hd)
    q[:, :, 0] = 16.0  # 16 * 5 * 0.5 = 40
    sink = torch.linspace(-2.0, 12.0, H)
    for mark in [0, 1, bs, 300, T - 1]:
        k, v = torch.zeros(T, G, hd), torch.zeros(T, G, hd)
        k[mark, :, 0], v[mark, :, 1] = 5.0, 1.0
        pages = Pages([(G, hd), (G, hd)], bs, dtype, blocks=T // bs + 5, seed=mark)
        pages.put("r", k, v)
        top = math.exp(cap * math.tanh(40.0 / cap))
        for p in sorted({mark, min(mark + 1, T - 1), T - 1}):
            want = [top / (top + p + math.exp(float(s))) for s in sink]
            one = attend([q], pages, ["r"], [1], [p], scale, softcap=cap, sink=sink.cuda())[0, :, 1].tolist()
            lo = max(0, p - 20)
            many = attend([q.expand(p + 1 - lo, H, hd)], pages, ["r"], [p + 1 - lo], [lo], scale, softcap=cap, sink=sink.cuda())[-1, :, 1].tolist()
            for got in (one, many):
                assert np.allclose(got, want, rtol=3e-2 if dtype == torch.bfloat16 else 2e-5), (mark, p, got, want)


def mixer_weights(g, d, layer):
    m = layer["mixer"]
    maps = 2 if layer["type"] == "attention" else 1
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"x." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in (("q", (H * maps * D, d)), ("k", (G * maps * D, d)), ("v", (G * V, d)), ("o", (d, H * V)))}
    if maps == 2:
        w.update({"x." + n: 0.5 * torch.randn(D, generator=g) * D**-0.25 for n in ("lq1", "lk1", "lq2", "lk2")})
    else:
        w["x.sink"] = torch.randn(H, generator=g)
    return w


def mixer_part(d, layer, eps):
    """The mixer as the model's description names it."""
    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.parts import build_part

    cfg = dict(architecture="Nipurax", vocab=8, width=d, norm=dict(eps=eps), residual_mult=1.0,
               embedding=dict(bigram=dict(buckets=2, mul_prev=1, mul_cur=1)), layers=[dict(layer, mlp=None)])  # fmt: skip
    arch, config = config_from_dict(cfg)
    spec = arch.build_spec(config).layers[0].mixer
    return build_part("mixer", type(spec)(spec.kind, spec.params, "x."), d)


MIXERS = [
    diff_attention(4, 2, 12, 40, 0.6, 0.3, 10, rot=(100.0, 8, (4.0, 1.0, 4.0, 64))),
    diff_attention(3, 3, 20, 24, 0.35, 0.6, 33, rot=(30.0, 20, None)),
    diff_attention(2, 1, 8, 8, 0.9, 0.1, 1),
    diff_attention(4, 2, 64, 128, 0.2, 0.4, 16, rot=(10000.0, 32, (6.0, 1.0, 3.0, 128))),
    diff_attention(4, 1, 32, 64, 0.3, 0.8, None, rot=(500.0, 32, (2.0, 0.001, 0.01, 4096))),
    sink_attention(6, 3, 24, 16, 0.5, temp=(0.7, 7), softcap=5.0),
    sink_attention(4, 4, 12, 20, 0.6),
    sink_attention(8, 2, 128, 128, 0.15, temp=(0.5, 9), softcap=20.0),
    sink_attention(4, 1, 64, 64, 0.25, softcap=2.0),
    # more query heads (or maps) a kv head than one block of the tensor-core kernels takes
    diff_attention(16, 1, 32, 64, 0.3, 0.5, 20, rot=(100.0, 16, None)),
    diff_attention(10, 1, 64, 128, 0.2, 0.3, 12),
    sink_attention(20, 1, 128, 128, 0.15, temp=(0.3, 5), softcap=10.0),
    sink_attention(34, 2, 64, 64, 0.2, softcap=6.0),
]  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("layer", MIXERS, ids=lambda m: f"{m['type']}-{m['mixer']['heads']}x{m['mixer']['dim']}")
def test_mixer_alone(dtype, layer):
    """A sequence in two portions and then token by token through scattered pages equals the plain
    mixer on the whole sequence; then two requests in one step, one of them starting mid-sequence."""
    from atomserve_b200.parts import CacheView

    d, T, bs = 72, 45, 4
    m = layer["mixer"]
    maps = 2 if layer["type"] == "attention" else 1
    g = torch.Generator().manual_seed(m["heads"] * 7 + m["dim"])
    w = mixer_weights(g, d, layer)
    part = mixer_part(d, layer, EPS)
    part.load(on_device(w, dtype))
    h, h2 = rounded(3 * torch.randn(T, d, generator=g)), rounded(3 * torch.randn(9, d, generator=g))
    run = (lambda x: plain.differential_attention(x.double(), doubles(w, "x."), m, EPS)) if maps == 2 else (lambda x: plain.sink_attention(x.double(), doubles(w, "x."), m))
    ref, ref2 = run(h).float(), run(h2).float()
    hd = max(maps * m["dim"], m["vdim"])
    assert part.cache_spec().tensors[0].width == hd and part.cache_spec().tensors[0].heads == m["kv_heads"]
    view = CacheView(k=torch.ones(24, m["kv_heads"], bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.ones_like(view.k)
    table = torch.randperm(24, generator=g).tolist()
    mine, other = table[:12], table[12:]
    view.block_tables = i32([mine])
    outs = []
    for start, n in [(0, 14), (14, 2), (16, 9)] + [(p, 1) for p in range(25, T - 6)]:
        view.slots = paged(mine, bs, range(start, start + n))
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), None, step_context([n], [start]), view))
    done = T - 6
    view.block_tables = i32([other, mine])
    view.slots = torch.cat([paged(other, bs, range(9)), paged(mine, bs, range(done, T))])
    both = part.forward(torch.cat([h2, h[done:]]).cuda().to(dtype), None, step_context([9, 6], [0, done]), view)
    assert both.dtype == torch.float32  # what a block that sums in float32 takes
    # (the two maps' outputs are each rounded to 16 bits; where a query sees few keys they are nearly equal, and
    # with lambda near 1 their difference is small before it is brought to unit size: more slack)
    check(torch.cat(outs + [both[9:]]), ref, dtype, "portions and single tokens", 0.12 if maps == 2 else 0.05)
    check(both[:9], ref2, dtype, "the second request beside it", 0.12 if maps == 2 else 0.05)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,T,E,identity,top,ff,shared", [(72, 40, 5, 1, 2, 40, (56, 1.0)), (64, 9, 2, 3, 4, 16, None), (100, 33, 1, 1, 1, 12, None),
                                                         (256, 300, 8, 2, 3, 128, (192, 1.5)), (96, 70, 7, 4, 4, 8, (20, 1.0)), (64, 5, 4, 0, 2, 24, None)])  # fmt: skip
def test_routed_experts_alone(dtype, d, T, E, identity, top, ff, shared):
    """Softmax scores over experts and identity experts, offsets that change the choice but not the
    weights, unnormalised weights times a scale, the clamped experts, the shared expert with its own
    limit. The inputs are what the plain router separates by more than rounding."""
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(d + E)
    mlp = moe(E, identity, top, ff, 1.5, 2.0, shared)
    cfg = dict(width=d, vocab=4, embedding=dict(bigram=dict(buckets=1, mul_prev=1, mul_cur=1)), layers=[dict(type="attention_2", mixer=dict(heads=1, kv_heads=1, dim=8, vdim=8), mlp=mlp)])
    w = {k[len("l0.mlp."):]: v for k, v in plain.random_checkpoint(cfg, seed=E).items() if k.startswith("l0.mlp.")}
    w["correction"] = 0.3 * torch.randn(E + identity, generator=g)
    h = rounded(2 * torch.randn(T, d, generator=g))
    s = torch.softmax(h.double() @ w["router"].double().T, -1) + w["correction"].double()
    ranked = s.sort(-1, descending=True).values
    clear = ((ranked[:, top - 1] - ranked[:, top]) > 2e-3) if top < E + identity else torch.ones(T, dtype=torch.bool)
    assert clear.sum() >= T // 2
    from atomserve_b200.models.nipurax import _feed_forward

    spec = _feed_forward(mlp, "x.")
    part = build_part("feed_forward", PartSpec(spec.kind, spec.params, "x."), d)
    part.load(on_device({"x." + k: v for k, v in w.items()}, dtype))
    got = part.forward(h.cuda().to(dtype), None, None)
    assert got.dtype == torch.float32
    ref = plain.routed_experts(h.double(), w, mlp).float()
    check(got[clear.cuda()], ref[clear], dtype, "experts", 0.03)
    if identity:
        chosen, _ = plain.route(h.double(), w["router"], w["correction"], top, 2.0)
        assert (chosen >= E).any(), "no token chose an identity expert: the case tests nothing"


# ---- whole models through the step function -------------------------------------------------

LENGTHS = {"a": [5, 49, 130, 1, 64], "b": [33, 2, 97, 40], "c": [300, 9, 70], "d": [70, 3, 130, 20]}


def oracle(cfg, w, prompt):
    return plain.forward(prompt, w, cfg).float()


def sure_positions(cfg, w, prompt, margin):
    """[n] bool: positions at which every router's choice leads by `margin` at least. Elsewhere
    rounding may choose another expert, which is a jump and no rounding error: such positions are
    left out of a comparison (5e-3 for bfloat16, 1e-4 for float32)."""
    margins = []
    plain.forward(prompt, w, cfg, margins=margins)
    return torch.stack(margins).min(0).values > margin if margins else torch.ones(len(prompt), dtype=torch.bool)


def judged(got, ref, dtype, what, lossy, sure):
    keep = sure[dtype if isinstance(dtype, str) else ("float32" if dtype == torch.float32 else "bfloat16")]
    if keep.any():
        judge(got.float().cpu()[keep], ref[keep], dtype, what, lossy[keep] if lossy is not None else None)


def allowance(cfg, w, prompt, ref):
    """What rounding alone does, per position: the largest error of the plain implementation itself
    over several ways of rounding to 16 bits everything an engine may keep in them."""
    return torch.stack([row_errors(plain.forward(prompt, w, cfg, stored=f), ref) for f in ROUNDINGS]).max(0).values


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    out = {}
    for name, (cfg, bs) in NIPURAX.items():
        w = plain.random_checkpoint(cfg, seed=29)
        folder = write_folder(cfg, w, tmp_path_factory.mktemp(f"nipurax_{name}"))
        ps = prompts(cfg, LENGTHS[name], seed=8)
        refs = [oracle(cfg, w, p) for p in ps]
        sure = [dict(float32=sure_positions(cfg, w, p, 1e-4), bfloat16=sure_positions(cfg, w, p, 5e-3)) for p in ps]
        assert all(s["bfloat16"].float().mean() > 0.25 for s in sure if len(s["bfloat16"]) > 8), "too few positions are left to compare"
        out[name] = (cfg, bs, folder, w, ps, refs, [allowance(cfg, w, p, r) for p, r in zip(ps, refs)], sure)
    return out


def replayer(folder, dtype, bs, max_tokens, **more):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, bs, **more)


CASES = [(n, d) for n in NIPURAX for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_then_token_by_token_then_portions(models, name, dtype):
    cfg, bs, folder, _, ps, refs, tols, sures = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    sizes = [2, 7, 3, 16, 2, 17, 5, 31, 2, 9, 1, 33]
    for i, (p, ref, tol, sure) in enumerate(zip(ps, refs, tols, sures)):
        n = len(p)

        def held(logits, places, what):
            judged(logits, ref[places], dtype, f"{name} request {i} {what}", tol[places], {k: v[places] for k, v in sure.items()})

        held(rp.step([dict(id=i, tokens=p, want=list(range(n)))], end=[i]), list(range(n)), "whole")
        head = max(n - 40, 0)
        if head:
            held(rp.step([dict(id=i, tokens=p[:head], want=[0, head - 1])], end=[]), [0, head - 1], "head")
        for j in range(head, n):
            held(rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == n - 1 else []), [j], f"position {j} alone")
        at, k = 0, i
        while at < n:
            m = min(sizes[k % len(sizes)], n - at)
            k += 1
            logits = rp.step([dict(id=i, tokens=p[at : at + m], want=list(range(m)))], end=[i] if at + m == n else [])
            held(logits, list(range(at, at + m)), f"portion {at}:{at + m}")
            at += m


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_requests_reusing_pages_and_slots(models, name, dtype):
    """Up to four live requests in four state slots, portions beside single tokens, in a pool so
    small that pages and slots freed by finished requests are taken again; every request appears
    four times, each equal to itself alone."""
    cfg, bs, folder, _, ps, refs, tols, sures = models[name]
    ps3, refs3, tols3, sures3 = ps * 4, refs * 4, tols * 4, sures * 4
    biggest = sorted((-(-len(p) // 64) * 64 for p in ps3), reverse=True)
    rp = replayer(folder, dtype, bs, sum(biggest[:4]), max_live=4)
    rng = np.random.default_rng(13)
    for entries, end in mixed_trace(ps3, rng, largest=40):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            places = list(range(e["at"], e["at"] + n))
            judged(logits[row : row + n], refs3[e["id"]][places], dtype, f"{name} request {e['id']} at {e['at']}",
                   tols3[e["id"]][places], {k: v[places] for k, v in sures3[e["id"]].items()})
            row += n
    assert sum(len(p) for p in ps3) > rp.cache.num_blocks * bs, "the pool was large enough to never reuse a page"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """400 tokens one by one after a short prompt, from CUDA graphs: chunks begin and end among decoded
    tokens, the query factor steps up, the last token travels from step to step."""
    for name in ("a", "c"):
        cfg, bs, folder, w = models[name][:4]
        p = prompts(cfg, [420], seed=12)[0]
        ref = oracle(cfg, w, p)
        tol = allowance(cfg, w, p, ref)
        sure = dict(float32=sure_positions(cfg, w, p, 1e-4), bfloat16=sure_positions(cfg, w, p, 5e-3))
        rp = replayer(folder, dtype, bs, 448)
        assert rp.runner.use_graphs
        rp.step([dict(id="x", tokens=p[:20], want=[])], end=[])
        for j in range(20, len(p)):
            logits = rp.step([dict(id="x", tokens=[p[j]], want=[0])], end=[])
            if j % 9 == 0 or j > 410:
                judged(logits, ref[j : j + 1], dtype, f"{name} decode position {j}", tol[j : j + 1], {k: v[j : j + 1] for k, v in sure.items()})
        held = rp.live["x"][0]
        chunked = [(g.spec.chunk, table) for g, table in zip(rp.cache.groups, held.block_tables) if g.spec.chunk]
        assert chunked, "no chunked layer kept pages of its own"
        for chunk, table in chunked:  # pages before the current chunk have gone back to the pool
            assert sum(b >= 0 for b in table) <= -(-chunk // bs) + 1 and len(table) == -(-len(p) // bs)


def test_the_stream_after_every_layer(models):
    """The float32 residual stream after each entry of the run order (a layer of the loop counts every
    time it runs) against the plain implementation's, in float32."""
    for name in ("a", "d"):
        cfg, bs, folder, w, ps = models[name][:5]
        p = ps[1]
        layers = []
        plain.forward(p, w, cfg, streams=layers)
        rp = replayer(folder, "float32", bs, 64)
        seen = []
        for block in rp.model.blocks:
            inner = block.forward_chain

            def wrapped(*a, _inner=inner, **k):
                out = _inner(*a, **k)
                seen.append(out[0].double().cpu())
                return out

            block.forward_chain = wrapped
        rp.step([dict(id=0, tokens=p, want=[0])], end=[0])
        assert len(seen) == len(plain.run_order(cfg)) == len(layers)
        for i, (got, ref) in enumerate(zip(seen, layers)):
            assert float((got - ref).abs().max() / ref.abs().max()) < 2e-5, f"{name}: stream after layer run {i}"


# ---- generation through the engine -----------------------------------------------------------

GREEDY = dict(temperature=0.0, ignore_eos=True)


def engine_for(folder, dtype, bs, **kw):
    from atomserve_b200.config import EngineConfig
    from atomserve_b200.engine.engine import create_engine
    from atomserve_b200.weights import load_model

    _, _, model = load_model(folder, dtype, "cuda")
    config = EngineConfig(**{"block_size": bs, "num_blocks": 64, "max_model_len": 64 * bs, "max_num_seqs": 8,
                             "max_num_batched_tokens": 256, **kw})  # fmt: skip
    return create_engine(model, config, sampler_seed=0)


@pytest.mark.parametrize("name", ["a", "b", "d"])
def test_greedy_generation_through_the_engine(models, name):
    """The engine's own entry point and scheduler: batched, in portions under a small budget, and
    with so few pages that requests are preempted and recomputed (state slots given back and
    zeroed again); float32 tokens equal the plain implementation's."""
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, w = models[name][:4]
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(p, w, cfg, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(folder, "float32", bs).generate(ps, params) == expect
    chunked = engine_for(folder, "float32", bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    assert chunked.num_steps > 8 + 3
    short = engine_for(folder, "float32", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    assert short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(p, w, cfg, n) for p in ps2]
    assert short.stats()["kv_blocks_used"] == 0


def test_greedy_generation_in_bfloat16_picks_near_best_tokens(models):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, w = models["c"][:4]
    ps = prompts(cfg, [40, 7, 90], seed=3)
    outs = engine_for(folder, "bfloat16", bs, max_num_batched_tokens=48).generate(ps, SamplingParams(max_tokens=12, **GREEDY))
    for p, out in zip(ps, outs):
        assert len(out) == 12
        ref = oracle(cfg, w, list(p) + list(out))
        spread = float((ref - ref.mean(-1, keepdim=True)).pow(2).mean().sqrt())
        for i, token in enumerate(out):
            row = ref[len(p) + i - 1]
            assert float(row.max() - row[token]) <= 0.15 * spread, f"token {i} lies far below the best"


def test_command_line_and_random_weights(tmp_path):
    """`python -m atomserve_b200` on a Nipurax folder written by the package's own random-weights
    writer from a configuration that round-trips through config.json."""
    import json
    import subprocess
    import sys

    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.weights.random_init import write_model_folder

    arch, config = config_from_dict(NIPURAX["b"][0])
    folder = write_model_folder(config, 3, tmp_path / "m", "bfloat16")
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Nipurax"
    done = subprocess.run([sys.executable, "-m", "atomserve_b200", str(folder), "--prompt-ids", "5,6,7", "--max-tokens", "6",
                           "--temperature", "0"], capture_output=True, text=True, timeout=600)  # fmt: skip
    assert done.returncode == 0, done.stderr[-2000:]
