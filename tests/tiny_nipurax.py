"""Small Nipurax configurations for the tests. They differ from one another in every size and
option: loops over a middle stretch of the layers, over the first layers, over all of them once, and
no loop; layers with and without a feed-forward; as many kv heads as heads, fewer, one; values wider
than the two maps of a head together, as wide, and narrower, also narrower than one map; rotations of
a whole map and of a part of it, none, stretched (with the band inside the frequencies, wholly above
and wholly below them) and plain; chunks of one token, shorter than a page, across page borders, equal
to a page and longer than the prompts; query factors that change every few tokens or never, scores
capped tightly, loosely and not at all; routers with no, one and several identity experts, one to
four choices, with and without a shared expert; a width and a vocabulary that are no multiples of 8.
Score scales are larger than 1 / sqrt(size), so that scores spread over many units and single keys
matter."""


def moe(experts, identity, top, ff, limit, scale, shared=None):
    out = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=dict(experts=experts, identity=identity, top=top, scale=scale))
    if shared is not None:
        out["shared"] = dict(ff=shared[0], limit=shared[1])
    return out


def diff_attention(heads, kv_heads, dim, vdim, scale, diff, chunk, rot=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, diff=diff)
    if chunk:
        m["mask"] = dict(size=chunk)
    if rot is not None:
        base, dims, scaling = rot
        m["rot"] = dict(base=base, dims=dims)
        if scaling is not None:
            m["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return dict(type="attention", mixer=m, mlp=mlp)


def sink_attention(heads, kv_heads, dim, vdim, scale, temp=None, softcap=None, mlp=None):
    m = dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale)
    if temp is not None:
        m["q_temp"] = dict(coef=temp[0], every=temp[1])
    if softcap is not None:
        m["softcap"] = softcap
    return dict(type="attention_2", mixer=m, mlp=mlp)


def _model(vocab, width, eps, mult, pairs, loop, layers):
    out = dict(architecture="Nipurax", vocab=vocab, width=width, norm=dict(eps=eps), residual_mult=mult,
               embedding=dict(bigram=dict(zip(("buckets", "mul_prev", "mul_cur"), pairs))), layers=list(layers))  # fmt: skip
    if loop is not None:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# a loop over the middle layers, three passes; a layer before it and one behind
NIPURAX_A = _model(300, 96, 1e-5, 0.4, (61, 31, 7), (1, 3, 3), [
    sink_attention(6, 3, 24, 16, 0.5, temp=(0.7, 7), softcap=5.0, mlp=moe(5, 1, 2, 40, 1.5, 1.5, shared=(56, 1.0))),
    diff_attention(4, 2, 12, 40, 0.6, 0.3, 10, rot=(100.0, 8, (4.0, 1.0, 4.0, 64)), mlp=moe(4, 0, 1, 24, 2.5, 1.0)),
    sink_attention(2, 1, 16, 16, 0.4, temp=(0.3, 16)),
    diff_attention(3, 3, 20, 24, 0.35, 0.6, 33, rot=(30.0, 20, None), mlp=moe(3, 2, 3, 32, 0.8, 2.5, shared=(16, 3.0))),
])  # fmt: skip
BLOCK_SIZE_A = 16

# no loop; chunks of one token and longer than every prompt; no query factor, no cap
NIPURAX_B = _model(257, 64, 1e-6, 1.0, (17, 3, 1000003), None, [
    diff_attention(2, 1, 8, 8, 0.9, 0.1, 1, rot=(50.0, 4, (16.0, 2.0, 3.0, 8)), mlp=moe(2, 3, 4, 16, 1.0, 0.7)),
    sink_attention(4, 4, 12, 20, 0.6),
    diff_attention(4, 1, 16, 32, 0.5, 0.8, 500, mlp=moe(6, 1, 2, 24, 2.0, 1.0, shared=(8, 0.5))),
    sink_attention(3, 1, 40, 8, 0.3, softcap=50.0, mlp=moe(3, 0, 3, 20, 5.0, 1.2, shared=(40, 2.0))),
    diff_attention(2, 2, 24, 16, 0.45, 0.5, None, rot=(1000.0, 12, (2.0, 100.0, 400.0, 64))),
])  # fmt: skip
BLOCK_SIZE_B = 8

# sizes at which the bfloat16 products and attention run this package's tensor-core kernels; the loop runs the
# first two layers twice
NIPURAX_C = _model(704, 256, 2e-6, 0.25, (1021, 211, 13), (0, 2, 2), [
    diff_attention(4, 2, 64, 128, 0.2, 0.4, 100, rot=(10000.0, 32, (6.0, 1.0, 3.0, 128)), mlp=moe(8, 2, 3, 128, 2.0, 2.0, shared=(192, 1.5))),
    sink_attention(8, 2, 128, 128, 0.15, temp=(0.5, 50), softcap=20.0, mlp=moe(6, 0, 2, 64, 1.5, 1.0)),
    sink_attention(4, 1, 64, 64, 0.25, temp=(0.2, 9), softcap=8.0),
    diff_attention(2, 2, 32, 64, 0.3, 0.7, 16, rot=(400000.0, 32, (2.0, 0.001, 0.01, 4096)), mlp=moe(4, 1, 1, 96, 1.0, 1.5, shared=(64, 1.0))),
])  # fmt: skip
BLOCK_SIZE_C = 16

# one layer of each kind, the whole model looped once; a width that is no multiple of 8; one expert and one identity expert
NIPURAX_D = _model(130, 100, 1e-5, 0.7, (1, 1, 1), (0, 2, 1), [
    diff_attention(1, 1, 10, 10, 0.7, 0.2, 5, rot=(10.0, 10, (32.0, 0.5, 2.0, 16)), mlp=moe(1, 1, 1, 12, 1.0, 1.0)),
    sink_attention(5, 5, 8, 12, 0.8, temp=(1.0, 1), softcap=3.0, mlp=moe(7, 4, 4, 8, 2.0, 0.5, shared=(20, 1.0))),
])  # fmt: skip
BLOCK_SIZE_D = 16

NIPURAX = {"a": (NIPURAX_A, BLOCK_SIZE_A), "b": (NIPURAX_B, BLOCK_SIZE_B), "c": (NIPURAX_C, BLOCK_SIZE_C),
           "d": (NIPURAX_D, BLOCK_SIZE_D)}  # fmt: skip
