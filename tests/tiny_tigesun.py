"""Small Tigesun configurations for the tests. They differ from one another in every size and
option: layer orders that start with each kind of mixer; layers with and without a feed-forward;
layers that run an earlier layer's tensors, next to it and far from it, several times; as many
kv heads as heads, fewer, one; key sizes other than value sizes; rotations of a whole head and of
a part of it, stretched (with the ramp inside the head's frequencies, wholly below them and wholly
above them) and plain; windows of one token, shorter than a page, across page borders, and longer
than the prompts; state-space layers with one group, several, and a group per head, with the
gated norm over the whole row, in parts, and a part per head, with one to five taps; a width, a
vocabulary and a latent size that are no multiples of 8; with and without a soft cap on the logits.
Score scales are larger than 1 / sqrt(size), so that scores spread over many units and single keys
matter."""


def _mlp(ff):
    return dict(kind="dense", ff=ff) if ff else None


def attention(heads, kv_heads, dim, vdim, scale, base, dims, scaling=None, ff=None):
    rot = dict(base=base, dims=dims)
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale, rot=rot), mlp=_mlp(ff))


def latent(heads, dim, vdim, kv_rank, window, scale, ff=None):
    return dict(type="latent_attention", mixer=dict(heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, scale=scale, mask=dict(size=window)),
                mlp=_mlp(ff))  # fmt: skip


def mamba2(heads, vdim, state, groups, conv, norm_groups, ff=None):
    return dict(type="mamba2", mixer=dict(heads=heads, vdim=vdim, state=state, groups=groups, conv=conv, norm_groups=norm_groups), mlp=_mlp(ff))


def again(layers, j):
    return dict(layers[j], weights_of=j)


def _model(vocab, width, eps, cap, layers, repeats):
    layers = list(layers)
    for j in repeats:
        layers.append(again(layers, j))
    out = dict(architecture="Tigesun", vocab=vocab, width=width, norm=dict(eps=eps), layers=layers)
    if cap:
        out["logit_softcap"] = cap
    return out


TIGESUN_A = _model(300, 96, 1e-5, 8.0, [
    mamba2(4, 16, 24, 2, 4, 4, ff=100),
    attention(6, 2, 24, 40, 0.45, 100.0, 16, scaling=(4.0, 64, 8.0, 1.0)),
    latent(3, 16, 24, 40, 20, 0.5, ff=72),
], repeats=[2, 0, 1, 2])  # fmt: skip
BLOCK_SIZE_A = 16

TIGESUN_B = _model(257, 64, 1e-6, None, [
    latent(2, 32, 8, 20, 1, 0.3, ff=40),
    attention(4, 4, 16, 16, 0.6, 50.0, 16),
    mamba2(5, 3, 8, 5, 1, 1),
    latent(5, 8, 24, 12, 500, 0.7),
    attention(2, 1, 40, 24, 0.35, 1000.0, 12, scaling=(16.0, 32, 64.0, 32.0), ff=64),
    mamba2(2, 24, 16, 1, 2, 2, ff=48),
], repeats=[])  # fmt: skip
BLOCK_SIZE_B = 8

# sizes at which the bfloat16 products and attention run this package's tensor-core kernels
TIGESUN_C = _model(704, 256, 2e-6, 30.0, [
    attention(8, 2, 128, 128, 0.2, 10000.0, 64, scaling=(8.0, 128, 16.0, 2.0), ff=512),
    mamba2(8, 64, 128, 1, 4, 1),
    latent(4, 64, 128, 64, 100, 0.2, ff=384),
    attention(4, 1, 64, 64, 0.3, 500000.0, 64, scaling=(2.0, 4096, 1.0, 0.01)),
    mamba2(4, 32, 64, 4, 3, 4, ff=256),
    latent(8, 128, 64, 128, 33, 0.15),
], repeats=[0, 1, 2])  # fmt: skip
BLOCK_SIZE_C = 16

# state-space layers only (no layer keeps pages), a width that is no multiple of 8, five taps
TIGESUN_D = _model(130, 100, 1e-5, 5.0, [mamba2(2, 20, 40, 2, 5, 1, ff=60), mamba2(6, 12, 10, 3, 3, 6)], repeats=[0])
BLOCK_SIZE_D = 16

# attention only: one layer's tensors run three times, each with pages of its own
TIGESUN_E = _model(140, 48, 1e-5, None, [attention(4, 2, 12, 20, 0.5, 30.0, 8, scaling=(32.0, 16, 2.0, 0.5), ff=56),
                                         attention(3, 3, 8, 8, 0.9, 300.0, 4)], repeats=[0, 0, 1])  # fmt: skip
BLOCK_SIZE_E = 8

# large heads and few of them: keys of 256 beside values of 64 and the other way round, latents of 256 and 320,
# a state of 256 under values of 128, eight taps, a single head with a single small state
TIGESUN_F = _model(500, 320, 1e-5, 20.0, [
    attention(2, 1, 256, 64, 0.08, 10000.0, 128, scaling=(4.0, 512, 16.0, 1.0), ff=640),
    latent(3, 192, 160, 256, 50, 0.07, ff=200),
    mamba2(2, 128, 256, 1, 8, 2),
    attention(5, 5, 32, 160, 0.2, 1e6, 32),
    latent(2, 48, 112, 320, 129, 0.1),
    mamba2(1, 8, 16, 1, 2, 1, ff=96),
], repeats=[1, 2])  # fmt: skip
BLOCK_SIZE_F = 16

TIGESUN = {"a": (TIGESUN_A, BLOCK_SIZE_A), "b": (TIGESUN_B, BLOCK_SIZE_B), "c": (TIGESUN_C, BLOCK_SIZE_C),
           "d": (TIGESUN_D, BLOCK_SIZE_D), "e": (TIGESUN_E, BLOCK_SIZE_E), "f": (TIGESUN_F, BLOCK_SIZE_F)}
