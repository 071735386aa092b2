"""The Tigesun design on the GPU against the plain implementation: each mechanism's part alone,
then whole models through the trace replayer in every way of cutting requests into steps, then
greedy generation through the engine and its scheduler."""

import math

import numpy as np
import pytest
import torch

import plain_tigesun as plain
from gefilix_helpers import check, prompts, write_folder
from helpers import mixed_trace
from test_engine_gpu import step_context
from tiny_tigesun import TIGESUN

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
EPS = 1e-5
F64 = torch.float64


def rounded(t):
    return t.bfloat16().float()


def on_device(w, dtype):
    """Matrices in the compute dtype, everything with one axis (and convolution taps) float32."""
    return {k: v.cuda().to(dtype if v.dim() == 2 and not k.endswith("conv") else torch.float32) for k, v in w.items()}


def doubles(w, prefix=""):
    return {k[len(prefix):]: v.double() for k, v in w.items() if k.startswith(prefix)}


def i32(v):
    return torch.tensor(v, dtype=torch.int32, device="cuda")


# ---- each mechanism alone -------------------------------------------------------------------


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d", [72, 100, 328, 1030])
def test_norms_around_a_sublayer(dtype, d):
    """N_in of the stream in the compute dtype; the new stream x + N_out(y + bias) gain in float32 with
    the next norm's N_in of it from the same kernel; the last sublayer of a model (nothing follows);
    the norm alone on chosen rows."""
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(d)
    T = 11
    gi, go, gn = (1 + 0.1 * torch.randn(d, generator=g) for _ in range(3))
    x, y, b = torch.randn(T, d, generator=g), 3 + 2 * torch.randn(T, d, generator=g), 0.5 * torch.randn(d, generator=g)
    norm = build_part("norm", PartSpec("sandwich_norm", dict(eps=EPS, tensor="n", out_tensor="nb")), d)
    nxt = build_part("norm", PartSpec("sandwich_norm", dict(eps=3 * EPS, tensor="m", out_tensor="mb")), d)
    norm.load({"n": gi.cuda(), "nb": go.cuda()})
    nxt.load({"m": gn.cuda(), "mb": go.cuda()})
    norm.bind_dtype(dtype)
    nxt.bind_dtype(dtype)
    h = norm.forward(x.cuda())
    assert h.dtype == dtype
    check(h, plain.rms(x.double(), gi.double(), EPS).float(), dtype, "the sublayer's input", 0.01)
    rows = i32([7, 0, 3])
    check(norm.forward(x.cuda(), rows), plain.rms(x.double(), gi.double(), EPS).float()[[7, 0, 3]], dtype, "chosen rows", 0.01)
    for bias in (None, b):
        ref = x.double() + plain.rms(y.double() + (bias.double() if bias is not None else 0), go.double(), EPS)
        stream, copy = norm.add_forward(x.cuda(), y.cuda(), nxt, bias.cuda() if bias is not None else None)
        assert stream.dtype == torch.float32 and copy.dtype == dtype
        check(stream, ref.float(), torch.float32, "stream after the sublayer's output norm")
        check(copy, plain.rms(ref, gn.double(), 3 * EPS).float(), dtype, "the next sublayer's input", 0.01)
        stream, copy = norm.add_forward(x.cuda(), y.cuda(), None, bias.cuda() if bias is not None else None)
        assert copy is None
        check(stream, ref.float(), torch.float32, "stream, nothing follows")
    # a sublayer's output in the compute dtype
    stream, _ = norm.add_forward(x.cuda(), y.cuda().to(dtype), nxt)
    check(stream, (x.double() + plain.rms(y.to(dtype).double(), go.double(), EPS)).float(), torch.float32, "output in the compute dtype")


def test_output_norm_reading_a_products_partial_sums():
    """With few tokens the last product of a sublayer stays as the GEMM's partial sums and the norm's
    kernel adds them up (and the product's bias): the finished product followed by the norm, up to
    the order in which a row's sums are formed."""
    from atomserve_b200 import ops
    from atomserve_b200.ops.linear import PartialSums

    g = torch.Generator().manual_seed(4)
    met = 0
    for T, d, K in ((1, 256, 512), (5, 336, 1024), (8, 2048, 2048), (33, 256, 392)):
        inner = torch.randn(T, K, generator=g).bfloat16().cuda()
        w = (torch.randn(d, K, generator=g) * K**-0.5).bfloat16().cuda()
        x = torch.randn(T, d, generator=g).cuda()
        go, gn, b = ((1 + 0.1 * torch.randn(d, generator=g)).cuda() for _ in range(3))
        for bias, nxt in ((None, gn), (b, gn), (b, None)):
            whole = ops.add_normed(x, ops.linear(inner, w, out_dtype=torch.float32), go, EPS, nxt, 2 * EPS, torch.bfloat16, bias)
            y = ops.linear_for_stream(inner, w)
            met += isinstance(y, PartialSums)
            fused = ops.add_normed(x, y, go, EPS, nxt, 2 * EPS, torch.bfloat16, bias)
            what = f"{T} tokens, width {d}, K {K}"
            assert float((whole[0] - fused[0]).abs().max() / whole[0].abs().max()) < 2e-6, what
            if nxt is not None:
                assert bool(((whole[1].float() - fused[1].float()).abs() <= 2.0**-7 * whole[1].float().abs() + 1e-30).all()), what
    assert met, "no shape ran with partial sums"


@pytest.mark.parametrize("dtype", DTYPES)
def test_normed_embedding_and_capped_head(dtype):
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(1)
    V, d, T = 70, 72, 9
    table, gain = rounded(torch.randn(V, d, generator=g)), 1 + 0.1 * torch.randn(d, generator=g)
    emb = build_part("embedding", PartSpec("normed_embedding", dict(vocab_size=V, eps=EPS, tensor="e", norm_tensor="e.n")), d)
    emb.load({"e": table.cuda().to(dtype), "e.n": gain.cuda()})
    ids = torch.randint(0, V, (T,), generator=g)
    x = emb.forward(ids.to(torch.int32).cuda())
    assert x.dtype == torch.float32
    check(x, plain.rms(table[ids].double(), gain.double(), EPS).float(), torch.float32, "normed embedding")
    head = build_part("head", PartSpec("lm_head", dict(vocab_size=V, tied=True, softcap=4.0)), d)
    head.tie(emb)
    hidden = rounded(2 * torch.randn(T, d, generator=g))
    logits = head.forward(hidden.cuda().to(dtype))
    raw = hidden.double() @ table.double().T
    assert float(raw.abs().max()) > 8, "no logit lies in the cap's flat part"
    assert logits.dtype == torch.float32 and float(logits.abs().max()) <= 4.0
    check(logits, (4.0 * torch.tanh(raw / 4.0)).float(), dtype, "capped logits", 0.02)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,ff,T", [(72, 100, 9), (256, 384, 5), (100, 60, 40), (256, 512, 300)])
def test_gated_feed_forward_alone(dtype, d, ff, T):
    """down(gelu_tanh(gate h + b) * (up h + b)) + b, as the part's own forward and as what it hands a
    block that norms its output (the product, or its partial sums, and the bias apart)."""
    from atomserve_b200 import ops
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(ff)
    w = {"f." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in (("gate", (ff, d)), ("up", (ff, d)), ("down", (d, ff)))}
    w.update({"f.gate.b": torch.randn(ff, generator=g), "f.up.b": torch.randn(ff, generator=g), "f.down.b": torch.randn(d, generator=g)})
    part = build_part("feed_forward", PartSpec("gated_mlp", dict(intermediate_size=ff, activation="gelu_tanh", biases=True), "f."), d)
    part.load(on_device(w, dtype))
    h = rounded(2 * torch.randn(T, d, generator=g))
    ref = plain.gated_mlp(h.double(), doubles(w, "f.")).float()
    ctx = step_context([T], [0])
    check(part.forward(h.cuda().to(dtype), None, ctx), ref, dtype, "feed-forward")
    gain = torch.ones(d, device="cuda")
    y = part.forward_for_stream(h.cuda().to(dtype), ctx)
    stream, _ = ops.add_normed(torch.zeros(T, d, device="cuda"), y, gain, EPS, None, 0.0, dtype, part.output_bias)
    check(stream, plain.rms(ref.double(), None, EPS).float(), dtype, "normed output with the bias joined in the norm's kernel")


@pytest.mark.parametrize("activation", ["gelu_tanh", "silu", "gelu"])
@pytest.mark.parametrize("T,d,ff,biased", [(3, 64, 40, True), (70, 2048, 96, True), (8, 4096, 1024, False), (130, 256, 200, True),
                                           (700, 512, 1100, True), (1100, 192, 72, False)])  # fmt: skip
def test_gated_unit_inside_the_product(activation, T, d, ff, biased):
    """act(h gate^T + b) * (h up^T + b) from the product's own epilogue (few tokens with the weights'
    rows on the lanes, many tokens on one SM and on pairs of them, K cut into partial sums that a
    second kernel adds up) against float64 of the same rounded operands."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(T + ff)
    gate, up = (rounded(torch.randn(ff, d, generator=g) * d**-0.5) for _ in range(2))
    b_gate, b_up = (torch.randn(ff, generator=g) if biased else None for _ in range(2))
    h = rounded(2 * torch.randn(T, d, generator=g))
    zg, zu = h.double() @ gate.double().T, h.double() @ up.double().T
    if biased:
        zg, zu = zg + b_gate.double(), zu + b_up.double()
    act = {"gelu_tanh": plain.gelu_tanh, "silu": plain.silu, "gelu": lambda z: 0.5 * z * (1 + torch.erf(z / math.sqrt(2.0)))}[activation]
    w = ops.interleave_gate_up(gate.cuda().bfloat16(), up.cuda().bfloat16())
    bias = torch.stack([b_gate, b_up], dim=1).reshape(-1).cuda().contiguous() if biased else None
    got = ops.linear_glu(h.cuda().bfloat16(), w, bias, activation)
    assert got.shape == (T, ff) and got.dtype == torch.bfloat16
    check(got, (act(zg) * zu).float(), torch.bfloat16, f"{activation} unit in the epilogue")


def paged(table, bs, positions):
    return i32([table[p // bs] * bs + p % bs for p in positions])


def attention_part(d, m, eps):
    from atomserve_b200.parts import PartSpec, build_part

    rot = m["rot"]
    s = rot.get("scaling")
    if s:
        position = PartSpec("scaled_rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"], factor=s["factor"],
                                                  original=s["original"], fast=s["fast"], slow=s["slow"]))  # fmt: skip
    else:
        position = PartSpec("rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"]))
    names = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm")
    return build_part("mixer", PartSpec("gqa_attention", dict(num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                                              value_dim=m["vdim"], qk_norm_eps=eps, position=position,
                                                              scale=m["scale"], names=names), "x."), d)  # fmt: skip


def attention_weights(g, d, m):
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {"x." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in (("q", (H * D, d)), ("k", (G * D, d)), ("v", (G * V, d)), ("o", (d, H * V)))}
    w.update({"x.q.norm": 1 + 0.3 * torch.randn(D, generator=g), "x.k.norm": 1 + 0.3 * torch.randn(D, generator=g)})
    return w


SCALINGS = {"inside": dict(factor=4.0, original=64, fast=8.0, slow=1.0), "none": None,
            "one step": dict(factor=16.0, original=32, fast=64.0, slow=32.0), "factor one": dict(factor=1.0, original=10, fast=3.0, slow=1.0)}  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,G,D,V,dims,bs,scaling", [(6, 2, 24, 40, 16, 4, "inside"), (4, 4, 16, 16, 16, 8, "none"), (2, 1, 40, 24, 12, 4, "one step"),
                                                    (8, 2, 128, 128, 64, 16, "inside"), (4, 1, 64, 64, 64, 16, "factor one"),
                                                    (3, 3, 96, 32, 96, 8, "inside"), (4, 2, 64, 128, 32, 16, "one step")])  # fmt: skip
def test_attention_part_alone(dtype, H, G, D, V, dims, bs, scaling):
    """The mixer by itself: q/k norms with one gain for all heads, the stretched rotation with its
    magnitude on a part of each head, values wider and narrower than keys. A sequence in two portions
    and then token by token through scattered pages equals the plain mixer on the whole sequence;
    then two requests in one step, one of them starting mid-sequence."""
    from atomserve_b200.parts import CacheView

    d, T = 72, 45
    g = torch.Generator().manual_seed(H * 7 + D)
    rot = dict(base=100.0, dims=dims)
    if SCALINGS[scaling]:
        rot["scaling"] = SCALINGS[scaling]
    m = dict(heads=H, kv_heads=G, dim=D, vdim=V, scale=2.0 * D**-0.5, rot=rot)
    w = attention_weights(g, d, m)
    part = attention_part(d, m, EPS)
    part.load(on_device(w, dtype))
    h, h2 = rounded(3 * torch.randn(T, d, generator=g)), rounded(3 * torch.randn(9, d, generator=g))
    ref = plain.attention_mixer(h.double(), doubles(w, "x."), m, EPS).float()
    ref2 = plain.attention_mixer(h2.double(), doubles(w, "x."), m, EPS).float()
    hd = max(D, V)
    view = CacheView(k=torch.zeros(24, G, bs, hd, device="cuda", dtype=dtype), block_size=bs)
    view.v = torch.zeros_like(view.k)
    table = torch.randperm(24, generator=g).tolist()
    mine, other = table[:12], table[12:]
    view.block_tables = i32([mine])
    outs = []
    for start, n in [(0, 14), (14, 2), (16, 9)] + [(p, 1) for p in range(25, T - 6)]:
        view.slots = paged(mine, bs, range(start, start + n))
        outs.append(part.forward(h[start : start + n].cuda().to(dtype), None, step_context([n], [start]), view))
    done = T - 6
    # the last six tokens beside a second request's whole prompt
    view.block_tables = i32([other, mine])
    view.slots = torch.cat([paged(other, bs, range(9)), paged(mine, bs, range(done, T))])
    both = part.forward(torch.cat([h2, h[done:]]).cuda().to(dtype), None, step_context([9, 6], [0, done]), view)
    check(torch.cat(outs + [both[9:]]), ref, dtype, "portions and single tokens", 0.03)
    check(both[:9], ref2, dtype, "the second request beside it", 0.03)



@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,dims,scaling", [(24, 16, "inside"), (64, 64, "inside"), (128, 64, "one step"), (96, 96, "inside"), (40, 12, "none")])
def test_rotation_at_near_and_far_positions(dtype, hd, dims, scaling):
    """The fused q/k norm and rotation at positions 0, 1 and tens of thousands, with the stretched
    frequencies and the magnitude (carried by the norms' gains, as the attention part does), against
    float64 angles."""
    from atomserve_b200 import ops
    from atomserve_b200.parts import PartSpec, build_part

    g = torch.Generator().manual_seed(hd)
    H, G, bs = 3, 1, 4
    positions = [0, 1, 2, 63, 64, 1000, 4097, 30011, 65535]
    T = len(positions)
    rot = dict(base=20000.0, dims=dims)
    if SCALINGS[scaling]:
        rot["scaling"] = dict(SCALINGS[scaling], original=2048)
        part = build_part("position", PartSpec("scaled_rotary", dict(head_dim=hd, theta=rot["base"], rotary_dim=dims, **rot["scaling"])), 32)
    else:
        part = build_part("position", PartSpec("rotary", dict(head_dim=hd, theta=rot["base"], rotary_dim=dims)), 32)
    part.prepare(torch.device("cuda"))
    fused = part.fused_rotary()
    qkv = rounded(torch.randn(T, (H + 2 * G) * hd, generator=g))
    gq, gk = 1 + 0.3 * torch.randn(hd, generator=g), 1 + 0.3 * torch.randn(hd, generator=g)
    mag = torch.ones(hd)
    mag[:dims] = fused.magnitude
    k_cache = torch.zeros(3, G, bs, hd, device="cuda", dtype=dtype)
    v_cache = torch.zeros_like(k_cache)
    q = ops.qk_norm_rope_store(qkv.cuda().to(dtype), H, G, hd, i32(positions), q_gain=(gq * mag).cuda(), k_gain=(gk * mag).cuda(), eps=EPS,
                               inv_freq=fused.inv_freq, rotary_dim=dims, slots=i32(list(range(T))), k_cache=k_cache, v_cache=v_cache)  # fmt: skip
    cos, sin = plain.scaled_rotary_tables(torch.tensor(positions), rot)
    heads = qkv.double().view(T, H + 2 * G, hd)
    q_ref = plain.rotate_half(plain.rms(heads[:, :H], gq.double(), EPS), cos, sin, dims)
    k_ref = plain.rotate_half(plain.rms(heads[:, H : H + G], gk.double(), EPS), cos, sin, dims)
    # float32: the angle position x frequency is itself a float32 product, good to half a unit in its last
    # place: up to 2^-24 x position radians (0.004 at 65,535); a wrong frequency is of the order of 1 there
    at = torch.tensor(positions, dtype=F64)[:, None, None]
    tol = (2e-6 + 2.0**-24 * at if dtype == torch.float32 else 2.0**-7 + 0 * at) * q_ref.abs().max()
    assert bool(((q.double().cpu() - q_ref).abs() <= tol).all()), float(((q.double().cpu() - q_ref).abs() / tol).max())
    k_got = k_cache.permute(0, 2, 1, 3).reshape(-1, G, hd)[:T].double().cpu()
    assert bool(((k_got - k_ref).abs() <= tol).all()), float(((k_got - k_ref).abs() / tol).max())
    v_got = v_cache.permute(0, 2, 1, 3).reshape(-1, G, hd)[:T].double().cpu()
    assert torch.equal(v_got, heads[:, H + G :].to(dtype).double())


class Pages:
    """Keys and values (or latents) of a few requests laid into pages through scrambled block tables."""

    def __init__(self, shapes, bs, dtype, blocks=128, seed=0):
        self.bs, self.dtype = bs, dtype
        self.pools = [torch.zeros(blocks, heads, bs, width, device="cuda", dtype=dtype) for heads, width in shapes]
        self.free = torch.randperm(blocks, generator=torch.Generator().manual_seed(seed)).tolist()
        self.tables = {}

    def put(self, request, *tensors):
        """Each [T, heads, width] of positions 0 .. T - 1."""
        n = tensors[0].shape[0]
        table = self.tables[request] = [self.free.pop() for _ in range(-(-n // self.bs))]
        at = torch.arange(n)
        block = torch.tensor(table)[at // self.bs].cuda()
        for pool, t in zip(self.pools, tensors):
            pool[block, :, (at % self.bs).cuda()] = t.to(self.dtype).cuda()

    def table(self, requests):
        width = max(len(self.tables[r]) for r in requests)
        return i32([self.tables[r] + [0] * (width - len(self.tables[r])) for r in requests])


def attend(q_parts, pages, requests, lens, starts, scale, window=None):
    from atomserve_b200 import ops

    ctx = step_context(lens, starts)
    q = torch.cat(q_parts).cuda().to(pages.dtype).contiguous()
    return ops.paged_attention(q, pages.pools[0], pages.pools[1], pages.table(requests), ctx.req_q_start, ctx.req_pos_start,
                               num_requests=len(lens), max_context=ctx.max_context, window=window, scale=scale,
                               host_q_lens=lens).float().cpu()  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("hd,bs,G", [(24, 16, 1), (96, 8, 3), (64, 16, 2), (128, 16, 4)])
def test_attention_finds_one_key_among_hundreds(dtype, hd, bs, G):
    """All keys are zero but one whose score is large; its value is e_1. Without a window a query sees
    it wherever it lies (the first position, both sides of page borders, hundreds of tokens back, the
    query's own position) and never when it lies ahead: the result is known in closed form. Single
    tokens and portions, head sizes of the general kernel and of the tensor-core kernels."""
    H, scale, T = 2 * G, 0.5, 700
    q = torch.zeros(1, H, hd)
    q[:, :, 0] = 8.0  # score of the marked key: 8 * 2.5 * 0.5 = 10
    for mark in [0, 1, bs - 1, bs, 2 * bs, 333, T - 2, T - 1]:
        k = torch.zeros(T, G, hd)
        k[mark, :, 0] = 2.5
        v = torch.zeros(T, G, hd)
        v[mark, :, 1] = 1.0
        pages = Pages([(G, hd), (G, hd)], bs, dtype, blocks=T // bs + 5, seed=mark)
        pages.put("r", k, v)
        for p in sorted({T - 1, mark, max(mark - 1, 0), min(mark + 1, T - 1), 400}):
            want = np.exp(10.0) / (np.exp(10.0) + p) if p >= mark else 0.0
            one = attend([q], pages, ["r"], [1], [p], scale)[0, :, 1].tolist()
            lo = max(0, p - 40)
            many = attend([q.expand(p + 1 - lo, H, hd)], pages, ["r"], [p + 1 - lo], [lo], scale)[-1, :, 1].tolist()
            for got in (one, many):
                assert np.allclose(got, want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6), (mark, p, got, want)


def attend_latent(q_parts, pages, requests, lens, starts, scale, window, rank, partitions=None):
    from atomserve_b200 import ops

    ctx = step_context(lens, starts)
    q = torch.cat(q_parts).cuda().float().contiguous()
    return ops.latent_attention(q, pages.pools[0], pages.table(requests), ctx.req_q_start, ctx.req_pos_start, rank=rank,
                                num_requests=len(lens), max_context=ctx.max_context, scale=scale, window=window,
                                partitions=partitions).cpu()  # fmt: skip


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window,bs,R", [(90, 16, 40), (7, 8, 24), (33, 16, 128), (16, 16, 64), (1, 4, 16), (250, 16, 64), (290, 16, 128), (1000, 16, 40)])
def test_one_latent_stands_out_at_the_windows_edges(dtype, window, bs, R):
    """All cached latents are zero but one whose score is large. For a query at position p the latent
    at p - window + 1 is the last one seen and the one at p - window the first one not seen; also the
    first position, the position itself, and latents on both sides of a page border. With zero
    latents elsewhere the result is known in closed form. Single tokens and portions, one and several
    key partitions."""
    H, scale, T = 3, 0.5, 300
    q = torch.zeros(1, H, R)
    q[:, :, 0] = 8.0  # score of the marked latent: 8 * 2.5 * 0.5 = 10
    marks = [0, 1, bs - 1, bs, 2 * bs, T - window - 1, T - window, T - window + 1, T - 2, T - 1]
    for mark in sorted({m for m in marks if 0 <= m < T}):
        c = torch.zeros(T, 1, R)
        c[mark, 0, 0], c[mark, 0, 1] = 2.5, 1.0
        pages = Pages([(1, R)], bs, dtype, blocks=T // bs + 5, seed=mark)
        pages.put("r", c)
        for p in sorted({T - 1, mark, min(mark + window - 1, T - 1), min(mark + window, T - 1)}):
            seen = 0 <= p - mark < window
            want = np.exp(10.0) / (np.exp(10.0) + min(p + 1, window) - 1) if seen else 0.0
            one = attend_latent([q], pages, ["r"], [1], [p], scale, window, R)[0, :, 1].tolist()
            cut = attend_latent([q], pages, ["r"], [1], [p], scale, window, R, partitions=(64, -(-T // 64)))[0, :, 1].tolist()
            lo = max(0, p - 40)
            many = attend_latent([q.expand(p + 1 - lo, H, R)], pages, ["r"], [p + 1 - lo], [lo], scale, window, R)[-1, :, 1].tolist()
            for got in (one, cut, many):
                assert np.allclose(got, want, rtol=2e-2 if dtype == torch.bfloat16 else 1e-5, atol=1e-6), (mark, p, got, want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,D,V,R,bs,window", [(5, 24, 16, 40, 4, 9), (1, 32, 32, 64, 16, 20), (8, 16, 8, 24, 8, 1), (6, 64, 80, 128, 16, 33),
                                               (3, 64, 48, 136, 16, 500), (4, 128, 64, 64, 16, 17), (2, 12, 20, 10, 2, 5)])  # fmt: skip
def test_latent_attention_part_alone(dtype, H, D, V, R, bs, window):
    """Keys and values up-projected from one normed latent per token, no positions, no gate, a
    window: one sequence in portions cut inside pages and windows, then token by token, pages
    scattered in no order; a second request beside the last tokens."""
    from atomserve_b200.parts import CacheView, PartSpec, build_part

    d, T = 56, 75
    g = torch.Generator().manual_seed(H + R)
    m = dict(heads=H, dim=D, vdim=V, kv_rank=R, scale=2.5 / math.sqrt(D), mask=dict(size=window))
    shapes = {"q": (H * D, d), "dkv": (R, d), "uk": (H * D, R), "uv": (H * V, R), "o": (d, H * V)}
    w = {"m." + n: rounded(torch.randn(s, generator=g) * s[1] ** -0.5) for n, s in shapes.items()}
    w["m.dkv.norm"] = 1 + 0.1 * torch.randn(R, generator=g)
    part = build_part("mixer", PartSpec("latent_attention", dict(heads=H, dim=D, rot_dim=0, vdim=V, kv_rank=R, scale=m["scale"], eps=EPS,
                                                                 position=None, gated=False, window=window), "m."), d)  # fmt: skip
    assert sorted(s.name for s in part.tensor_specs()) == sorted(w)
    assert part.cache_spec().window == window
    part.load(on_device(w, dtype))
    h, h2 = rounded(torch.randn(T, d, generator=g)), rounded(torch.randn(11, d, generator=g))
    ref = plain.latent_attention_mixer(h.double(), doubles(w, "m."), m, EPS).float()
    ref2 = plain.latent_attention_mixer(h2.double(), doubles(w, "m."), m, EPS).float()
    blocks = -(-T // bs) + -(-11 // bs) + 3
    table = torch.randperm(blocks, generator=g).tolist()
    mine, other = table[: -(-T // bs)], table[-(-T // bs) :]
    view = CacheView(pages={"latent": torch.zeros(blocks, 1, bs, R, device="cuda", dtype=dtype)}, block_size=bs)
    view.block_tables = i32([mine])
    got, at = [], 0
    for n in [3, 1, 2, 29, 2, 17] + [1] * 15:
        view.slots = paged(mine, bs, range(at, at + n))
        got.append(part.forward(h[at : at + n].cuda().to(dtype), None, step_context([n], [at]), view, True).float().cpu())
        at += n
    view.block_tables = i32([other + [0] * (len(mine) - len(other)), mine])
    view.slots = torch.cat([paged(other, bs, range(11)), paged(mine, bs, range(at, T))])
    both = part.forward(torch.cat([h2, h[at:]]).cuda().to(dtype), None, step_context([11, T - at], [0, at]), view, True).float().cpu()
    check(torch.cat(got + [both[11:]]), ref, dtype, "portions and single tokens", 0.05)
    check(both[:11], ref2, dtype, "the second request beside it", 0.05)


@pytest.mark.parametrize("dtype", DTYPES)
# (rows of even and of odd width: the kernel takes two channels a thread where it can; eight taps fill the
# window it keeps in registers, nine and eleven take its plain loop)
@pytest.mark.parametrize("C,K,H", [(160, 4, 4), (21, 1, 5), (130, 2, 3), (56, 5, 2), (448, 3, 8), (96, 4, 3), (40, 8, 3), (64, 9, 2), (34, 11, 3)])
def test_convolution_steps_and_its_state(dtype, C, K, H):
    """The causal convolution per channel with bias and SiLU, reading what came before a portion from
    the request's state; the step sizes softplus(dt + bias) with decays exp(-exp(A) dt), for
    pre-activations far out on both sides; the state after portions longer and shorter than the taps.
    Three requests in steps of unequal portions, slots in another order."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(C + K)
    lens, slots = [70, 3, 41], [3, 0, 4]
    off, dt_off, width = 8, 8 + C + 5, 8 + C + 5 + H
    proj = [rounded(2 * torch.randn(n, width, generator=g)) for n in lens]
    for p in proj:
        p[:, dt_off:] = rounded(p[:, dt_off:] * 12)  # softplus from exp(-30) to 30
    taps, bias = torch.randn(C, K, generator=g) * K**-0.5, 0.3 * torch.randn(C, generator=g)
    dt_bias, a_log = torch.randn(H, generator=g), torch.linspace(-2, 2, H)
    state = torch.zeros(5, K - 1, C, device="cuda")
    got = {i: [] for i in range(3)}
    # (request, start, count): three in a step; then portions of one and two tokens (shorter than the taps); then the rest
    for cut in ([(0, 0, 33), (1, 0, 1), (2, 0, 2)], [(1, 1, 2), (0, 33, 1), (2, 2, 1)], [(2, 3, 38), (0, 34, 2)], [(0, 36, 34)]):
        rows = torch.cat([proj[i][a : a + n] for i, a, n in cut]).cuda().to(dtype)
        ctx = step_context([n for _, _, n in cut], [a for _, a, _ in cut], [slots[i] for i, _, _ in cut])
        out = ops.conv_steps(rows, off, dt_off, taps.cuda(), bias.cuda(), state, dt_bias.cuda(), a_log.cuda(), ctx.state_slots, ctx.req_q_start, len(cut))
        ops.conv_state_update(state, rows, off, ctx.state_slots, ctx.req_q_start, len(cut))
        at = 0
        for i, _, n in cut:
            got[i].append([o[at : at + n].float().cpu() for o in out])
            at += n
    for i, n in enumerate(lens):
        x = proj[i][:, off : off + C].double()
        conv = plain.silu(plain.causal_conv(x, taps.double(), bias.double()))
        dt = plain.softplus(proj[i][:, dt_off:].double() + dt_bias.double())
        decay = torch.exp(-torch.exp(a_log.double()) * dt)
        mine = [torch.cat([piece[j] for piece in got[i]]) for j in range(3)]
        check(mine[0], conv.float(), dtype, f"request {i}: convolution", 0.01)
        assert torch.allclose(mine[1].double(), decay, rtol=3e-5, atol=1e-30), f"request {i}: decays"
        assert torch.allclose(mine[2].double(), dt, rtol=3e-6, atol=1e-30), f"request {i}: step sizes"
        if K > 1:
            held = torch.cat([torch.zeros(K - 1, C, dtype=F64), x])[-(K - 1) :]
            assert torch.equal(state[slots[i]].cpu().double(), held), f"request {i}: what the convolution keeps"
    assert not state[[1, 2]].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,P,parts", [(4, 16, 4), (5, 3, 1), (8, 64, 2), (6, 12, 6), (3, 20, 3), (16, 64, 1)])
def test_gate_before_the_norm_in_parts(dtype, H, P, parts):
    """(y + D_h x) silu(z), each part of the row divided by its own root mean square, times a gain;
    x and z as column ranges of a wider tensor."""
    from atomserve_b200 import ops

    g = torch.Generator().manual_seed(H + P)
    T, width = 13, H * P
    y = torch.randn(T, width, generator=g) * torch.linspace(0.01, 30, width)  # parts of very unequal size
    wide = rounded(2 * torch.randn(T, 2 * width + 8, generator=g)).cuda().to(dtype)
    z, x = wide[:, :width], wide[:, width + 8 :]
    skip, gain = torch.randn(H, generator=g), 1 + 0.1 * torch.randn(width, generator=g)
    got = ops.gate_group_norm(y.cuda(), x, z, skip.cuda(), gain.cuda(), parts, P, EPS)
    v = (y.double() + skip.double().repeat_interleave(P) * x.double().cpu()) * plain.silu(z.double().cpu())
    ref = plain.rms(v.view(T, parts, width // parts), None, EPS).reshape(T, width) * gain.double()
    assert got.dtype == dtype
    check(got, ref.float(), dtype, "gated norm in parts", 0.01)


def state_space_part(d, m, eps):
    from atomserve_b200.parts import PartSpec, build_part

    return build_part("mixer", PartSpec("selective_state_space", dict(heads=m["heads"], vdim=m["vdim"], state=m["state"], groups=m["groups"],
                                                                      conv=m["conv"], norm_groups=m["norm_groups"], eps=eps), "m."), d)  # fmt: skip


def state_space_weights(g, d, m):
    H, P, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
    inner, channels = H * P, H * P + 2 * G * N
    w = {"m.in": rounded(torch.randn(2 * inner + 2 * G * N + H, d, generator=g) * d**-0.5), "m.o": rounded(torch.randn(d, inner, generator=g) * inner**-0.5),
         "m.conv": torch.randn(channels, K, generator=g) * K**-0.5, "m.conv.b": 0.3 * torch.randn(channels, generator=g),
         "m.dt_bias": torch.linspace(-3, 1, H), "m.A_log": torch.linspace(-1.5, 1.5, H).flip(0), "m.D": torch.randn(H, generator=g),
         "m.norm": 1 + 0.1 * torch.randn(inner, generator=g)}  # fmt: skip
    w["m.in"][-H:] *= 4  # step sizes that move
    w["m.in"] = rounded(w["m.in"])
    return w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("H,P,N,G,K,parts", [(4, 16, 24, 2, 4, 4), (5, 3, 8, 5, 1, 1), (2, 24, 16, 1, 2, 2), (8, 64, 128, 1, 4, 1),
                                             (8, 32, 48, 2, 3, 2), (6, 12, 10, 3, 3, 6), (2, 20, 40, 2, 5, 1), (3, 8, 130, 1, 2, 3)])  # fmt: skip
def test_state_space_layer_alone(dtype, H, P, N, G, K, parts):
    """Whole, in portions down to one token (shorter than the taps), three requests of unequal length
    in one step with slots in another order, and a portion long enough to run in segments after a
    first one that leaves a state: each against the recurrence written out token by token. Heads
    that forget within a few tokens beside heads that keep hundreds."""
    from atomserve_b200.parts import CacheView

    d, T = 48, 37
    g = torch.Generator().manual_seed(H * 100 + N)
    m = dict(heads=H, vdim=P, state=N, groups=G, conv=K, norm_groups=parts)
    w = state_space_weights(g, d, m)
    part = state_space_part(d, m, EPS)
    assert {s.name: tuple(s.shape) for s in part.tensor_specs()} == {k: tuple(v.shape) for k, v in w.items()}
    part.load(on_device(w, dtype))
    hs = [rounded(torch.randn(n, d, generator=g)) for n in (T, 5, 1, 420)]
    refs = [plain.mamba2_mixer(h.double(), doubles(w, "m."), m, EPS).float() for h in hs]
    view = CacheView(state={"s": torch.zeros(7, H, N, P, device="cuda"), "conv": torch.zeros(7, K - 1, H * P + 2 * G * N, device="cuda")})
    assert [tuple(s.shape) for s in part.state_specs()] == [tuple(v.shape[1:]) for v in view.state.values()]

    def run(pieces, lens, slots):
        h = torch.cat(pieces).cuda().to(dtype)
        return part.forward(h, None, step_context(lens, [0] * len(lens), slots), view).float().cpu()

    # bfloat16: twice what rounding the projection, the convolution's output and the gated heads does to
    # the plain implementation itself (a part of the row with a small root mean square magnifies it), at least 0.05
    tol = 0.05
    if dtype == torch.bfloat16:
        for h, ref in zip(hs, refs):
            lossy = plain.mamba2_mixer(h.double(), doubles(w, "m."), m, EPS, stored=lambda t: t.bfloat16().double()).float()
            d_ = (lossy - ref).double()
            d_ = d_ - d_.mean(-1, keepdim=True)
            spread = (ref.double() - ref.double().mean(-1, keepdim=True)).pow(2).mean().sqrt()
            tol = max(tol, 2 * float(d_.pow(2).mean(-1).sqrt().max() / spread))
    check(run([hs[0]], [T], [2]), refs[0], dtype, "whole", tol)
    got, at = [], 0
    for n in (1, 2, 16, 1, 17):  # across the kernel's token tile of 16
        got.append(run([hs[0][at : at + n]], [n], [4]))
        at += n
    check(torch.cat(got), refs[0], dtype, "in portions", tol)
    for buf in view.state.values():
        assert not buf[[0, 1, 3, 5, 6]].any(), "a slot other than the request's was written"
        buf.zero_()
    out = run(hs[:3], [T, 5, 1], [5, 0, 3])
    check(out, torch.cat(refs[:3]), dtype, "three requests in one step", tol)
    assert out.dtype == torch.float32
    got = torch.cat([run([hs[3][:30]], [30], [6]), run([hs[3][30:], hs[1]], [390, 5], [6, 1])])
    check(got, torch.cat([refs[3], refs[1]]), dtype, "a long portion in segments after a short one", tol)
    # token by token for a long time: the state is carried through every step
    for buf in view.state.values():
        buf.zero_()
    got = torch.cat([run([hs[3][t : t + 1]], [1], [1]) for t in range(150)])
    check(got, refs[3][:150], dtype, "150 tokens one by one", tol)


# ---- whole models through the step function ---------------------------------------------------

LENGTHS = {"a": [5, 49, 130, 1, 64], "b": [33, 2, 97, 40], "c": [300, 9, 70], "d": [20, 3, 70], "e": [45, 2, 90], "f": [150, 37, 4, 90]}


def oracle(cfg, w, prompt):
    return plain.forward(cfg, w, prompt).float()


def row_errors(got, ref):
    """Per position: rms of the difference (mean taken off) over the spread of the reference's logits."""
    d = got.double() - ref.double()
    d = d - d.mean(-1, keepdim=True)
    spread = (ref.double() - ref.double().mean(-1, keepdim=True)).pow(2).mean().sqrt()
    return d.pow(2).mean(-1).sqrt() / spread


def _toward_zero(t):
    return (t.float().view(torch.int32) & -65536).view(torch.float32).double()


ROUNDINGS = (lambda t: t.bfloat16().double(), _toward_zero,
             lambda t: (t * (1 + 2.0**-9)).bfloat16().double(), lambda t: (t * (1 - 2.0**-9)).bfloat16().double())  # fmt: skip


def allowance(cfg, w, prompt, ref):
    """What rounding alone does, per position: the error of the plain implementation itself when
    everything an engine may keep in 16 bits is rounded to bfloat16. The design norms every
    sublayer's output, so single positions magnify rounding, and which ones depends on where the
    roundings fall: an engine that rounds other intermediate values than the plain implementation
    (sums inside a product's epilogue, say) lands on other positions. So several ways of rounding
    (to nearest, toward zero, to nearest after a shift of half a step up and down) each give an
    error per position; the largest of them stands for the position."""
    return torch.stack([row_errors(plain.forward(cfg, w, prompt, stored=f), ref) for f in ROUNDINGS]).max(0).values


def judge(got, ref, dtype, what, lossy):
    """float32: 5e-5 of the largest logit (where a sublayer's output is small before its norm, the
    norm magnifies float32 rounding too). bfloat16: no position further off than four times what
    rounding alone does there (at least 0.1 of the spread: a wrong key, window edge or state is of
    the order of 1), and over eight positions or more, a mean error of at most that of rounding
    alone (at least 0.02)."""
    got = got.float().cpu()
    assert got.shape == ref.shape and torch.isfinite(got).all(), what
    if dtype in ("float32", torch.float32):
        err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
        assert err < 5e-5, f"{what}: relative error {err:.3g}"
        return
    errors = row_errors(got, ref)
    over = errors > torch.clamp(4 * lossy, min=0.1)
    assert not over.any(), f"{what}: position {int(over.nonzero()[0])} is {float(errors[over][0]):.3g} of the spread off, rounding alone {float(lossy[over][0]):.3g}"
    if len(errors) >= 8:
        assert float(errors.mean()) <= max(0.02, float(lossy.mean())), f"{what}: mean error {float(errors.mean()):.3g}, rounding alone {float(lossy.mean()):.3g}"


@pytest.fixture(scope="module")
def models(tmp_path_factory):
    """name -> (config, block size, folder, weights, prompts, float64 logits per prompt, what
    rounding alone does per prompt and position)."""
    out = {}
    for name, (cfg, bs) in TIGESUN.items():
        w = plain.random_checkpoint(cfg, seed=23)
        folder = write_folder(cfg, w, tmp_path_factory.mktemp(f"tigesun_{name}"))
        ps = prompts(cfg, LENGTHS[name], seed=6)
        refs = [oracle(cfg, w, p) for p in ps]
        out[name] = (cfg, bs, folder, w, ps, refs, [allowance(cfg, w, p, r) for p, r in zip(ps, refs)])
    return out


def replayer(folder, dtype, bs, max_tokens, **more):
    from atomserve_b200.engine.replay import TraceReplayer

    return TraceReplayer(folder, dtype, max_tokens, bs, **more)


CASES = [(n, d) for n in TIGESUN for d in ("float32", "bfloat16")]


@pytest.mark.parametrize("name,dtype", CASES)
def test_whole_then_token_by_token_then_portions(models, name, dtype):
    cfg, bs, folder, _, ps, refs, tols = models[name]
    rp = replayer(folder, dtype, bs, max(-(-len(p) // 64) * 64 for p in ps))
    sizes = [2, 7, 3, 16, 2, 17, 5, 31, 2, 9, 1, 33]
    for i, (p, ref, tol) in enumerate(zip(ps, refs, tols)):
        n = len(p)
        judge(rp.step([dict(id=i, tokens=p, want=list(range(n)))], end=[i]), ref, dtype, f"{name} request {i} whole", tol)
        head = max(n - 40, 0)
        if head:
            judge(rp.step([dict(id=i, tokens=p[:head], want=[0, head - 1])], end=[]), ref[[0, head - 1]], dtype, f"{name} request {i} head", tol[[0, head - 1]])
        for j in range(head, n):
            logits = rp.step([dict(id=i, tokens=[p[j]], want=[0])], end=[i] if j == n - 1 else [])
            judge(logits, ref[j : j + 1], dtype, f"{name} request {i} position {j} alone", tol[j : j + 1])
        at, k = 0, i
        while at < n:
            m = min(sizes[k % len(sizes)], n - at)
            k += 1
            logits = rp.step([dict(id=i, tokens=p[at : at + m], want=list(range(m)))], end=[i] if at + m == n else [])
            judge(logits, ref[at : at + m], dtype, f"{name} request {i} portion {at}:{at + m}", tol[at : at + m])
            at += m


@pytest.mark.parametrize("name,dtype", CASES)
def test_mixed_requests_reusing_pages_and_slots(models, name, dtype):
    """Up to four live requests in four state slots, portions beside single tokens, in a pool so
    small that pages and slots freed by finished requests are taken again; every request appears
    four times, each equal to itself alone."""
    cfg, bs, folder, _, ps, refs, tols = models[name]
    ps3, refs3, tols3 = ps * 4, refs * 4, tols * 4
    biggest = sorted((-(-len(p) // 64) * 64 for p in ps3), reverse=True)
    rp = replayer(folder, dtype, bs, sum(biggest[:4]), max_live=4)
    rng = np.random.default_rng(11)
    for entries, end in mixed_trace(ps3, rng, largest=40):
        logits = rp.step([dict(id=e["id"], tokens=e["tokens"], want=e["want"]) for e in entries], end=end)
        row = 0
        for e in entries:
            n = len(e["tokens"])
            judge(logits[row : row + n], refs3[e["id"]][e["at"] : e["at"] + n], dtype, f"{name} request {e['id']} at {e['at']}",
                  tols3[e["id"]][e["at"] : e["at"] + n])
            row += n
    if rp.cache.groups:  # (a model of state-space layers alone keeps no pages, only slots)
        assert sum(len(p) for p in ps3) > rp.cache.num_blocks * bs, "the pool was large enough to never reuse a page"
    assert len(ps3) > 4


def test_a_place_asked_for_twice(models):
    """A single decoded token and a portion whose wanted places name one place twice: it is given twice."""
    cfg, bs, folder, _, ps, refs, _ = models["b"]
    rp = replayer(folder, "float32", bs, 128)
    p, ref = ps[0], refs[0]
    got = rp.step([dict(id=0, tokens=p[:20], want=[19, 3, 19])], end=[])
    judge(got, ref[[19, 3, 19]], "float32", "a portion", None)
    got = rp.step([dict(id=0, tokens=p[20:21], want=[0, 0])], end=[0])
    judge(got, ref[[20, 20]], "float32", "a single token", None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding(models, dtype):
    """400 tokens one by one after a short prompt: the windows pass over decoded tokens and pages
    they leave behind are given back, the states are carried through every step."""
    for name in ("a", "c"):
        cfg, bs, folder, w, _, _, _ = models[name]
        p = prompts(cfg, [420], seed=12)[0]
        ref = oracle(cfg, w, p)
        tol = allowance(cfg, w, p, ref)
        rp = replayer(folder, dtype, bs, 448)
        rp.step([dict(id="x", tokens=p[:20], want=[])], end=[])
        for j in range(20, len(p)):
            logits = rp.step([dict(id="x", tokens=[p[j]], want=[0])], end=[])
            if j % 9 == 0 or j > 410:
                judge(logits, ref[j : j + 1], dtype, f"{name} decode position {j}", tol[j : j + 1])


def test_the_stream_after_every_layer(models):
    """The float32 residual stream after each entry of the run order (a layer that runs another's
    tensors counts on its own) against the plain implementation's, in float32."""
    for name in ("a", "b"):
        cfg, bs, folder, w, ps, _, _ = models[name]
        p = ps[1]
        _, layers = plain.forward(cfg, w, p, return_layers=True)
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
        assert len(seen) == len(cfg["layers"])
        for i, (got, ref) in enumerate(zip(seen, layers)):
            assert float((got - ref).abs().max() / ref.abs().max()) < 2e-5, f"{name}: stream after layer {i}"


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

    cfg, bs, folder, w, _, _, _ = models[name]
    ps = prompts(cfg, [5, 17, 33], seed=3)
    expect = [plain.greedy_generate(cfg, w, p, 8) for p in ps]
    params = SamplingParams(max_tokens=8, **GREEDY)
    assert engine_for(folder, "float32", bs).generate(ps, params) == expect
    chunked = engine_for(folder, "float32", bs, max_num_batched_tokens=8, max_num_seqs=4)
    assert chunked.generate(ps, params) == expect
    assert chunked.num_steps > 8 + 3
    short = engine_for(folder, "float32", bs, num_blocks=7, max_model_len=7 * bs, enable_prefix_caching=False)
    n = bs + 8
    ps2 = prompts(cfg, [bs + 3, bs + 5, 2 * bs - 1], seed=5)
    assert short.generate(ps2, SamplingParams(max_tokens=n, **GREEDY)) == [plain.greedy_generate(cfg, w, p, n) for p in ps2]
    assert short.stats()["kv_blocks_used"] == 0


def test_greedy_generation_in_bfloat16_picks_near_best_tokens(models):
    from atomserve_b200.engine.sequence import SamplingParams

    cfg, bs, folder, w, _, _, _ = models["c"]
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
    """`python -m atomserve_b200` on a Tigesun folder written by the package's own random-weights
    writer from a configuration that round-trips through config.json."""
    import json
    import subprocess
    import sys

    from atomserve_b200.config.registry import config_from_dict
    from atomserve_b200.weights.random_init import write_model_folder

    arch, config = config_from_dict(TIGESUN["b"][0])
    folder = write_model_folder(config, 3, tmp_path / "m", "bfloat16")
    assert json.loads((folder / "config.json").read_text())["architecture"] == "Tigesun"
    done = subprocess.run([sys.executable, "-m", "atomserve_b200", str(folder), "--prompt-ids", "5,6,7", "--max-tokens", "6",
                           "--temperature", "0"], capture_output=True, text=True, timeout=600)  # fmt: skip
    assert done.returncode == 0, done.stderr[-2000:]
