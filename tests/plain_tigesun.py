"""A plain, slow implementation of the Tigesun design for the tests: one function per mechanism,
float64 on the CPU, whole sequences at once, no cache, no batching. It shares no code with the package.

A model is (config dict, tensors dict name -> tensor). Tensor names: `embed`, `embed.norm`,
`l<i>.norm1`, `l<i>.norm1b`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.mix.*`, `l<i>.mlp.*`, `final.norm`.

`stored` (identity by default) is applied to everything that an engine may keep in 16 bits:
projections, convolution outputs, attention outputs, gated heads, a sublayer's normed input. With
`stored = lambda t: t.bfloat16().double()` the implementation shows what rounding alone does to a
model's logits; the tests measure the engine's bfloat16 error against that.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms(x: torch.Tensor, gain: torch.Tensor | None, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis, times the gain where there is one."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30, z, torch.log1p(torch.exp(torch.clamp(z, max=30))))


def scaled_rotary_tables(positions: torch.Tensor, rot: dict) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin [T, dims / 2] of a rotary encoding whose frequencies are stretched for long
    contexts: frequency i of dims / 2 is base^(-2i / dims); with `scaling` (factor, original, fast,
    slow) the slow frequencies are divided by `factor`, the fast ones kept, those between blended
    along a linear ramp over the index, and both tables are multiplied by 0.1 ln(factor) + 1."""
    dims, base = rot["dims"], rot["base"]
    half = dims // 2
    i = torch.arange(half, dtype=F64)
    f = base ** (-2.0 * i / dims)
    mag = 1.0
    s = rot.get("scaling")
    if s:
        def index_of(turns):
            return dims * math.log(s["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
        lo = max(math.floor(index_of(s["fast"])), 0)
        hi = min(math.ceil(index_of(s["slow"])), dims - 1)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        f = f / s["factor"] * ramp + f * (1 - ramp)
        mag = 0.1 * math.log(s["factor"]) + 1.0
    a = positions.to(F64)[:, None] * f[None, :]
    return torch.cos(a) * mag, torch.sin(a) * mag


def rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, dims: int) -> torch.Tensor:
    """x [T, heads, dim]: entry i < dims / 2 of a head pairs with entry i + dims / 2; the rest pass."""
    half = dims // 2
    u, v, rest = x[..., :half], x[..., half:dims], x[..., dims:]
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([u * c - v * s, v * c + u * s, rest], dim=-1)


def masked_softmax_attention(q, k, v, scale: float, window: int | None) -> torch.Tensor:
    """q [T, H, D], k [T, H, D], v [T, H, V] -> [T, H, V]; query i sees j <= i, and with a window
    only i - j < window."""
    T = q.shape[0]
    scores = torch.einsum("ihd,jhd->hij", q, k) * scale
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    seen = j <= i
    if window is not None:
        seen = seen & (i - j < window)
    scores = scores.masked_fill(~seen[None], float("-inf"))
    return torch.einsum("hij,jhv->ihv", torch.softmax(scores, dim=-1), v)


def attention_mixer(h, w: dict, m: dict, eps: float, stored=lambda t: t) -> torch.Tensor:
    """Grouped-query attention: per-head RMS norm of q and k with one gain for all heads, then the
    rotation, scores times `scale`, causal softmax, output projection."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = stored(h @ w["q"].T).view(T, H, D)
    k = stored(h @ w["k"].T).view(T, G, D)
    v = stored(h @ w["v"].T).view(T, G, V)
    q, k = rms(q, w["q.norm"], eps), rms(k, w["k.norm"], eps)
    rot = m.get("rot")
    if rot and rot["dims"]:
        cos, sin = scaled_rotary_tables(torch.arange(T), rot)
        q, k = rotate_half(q, cos, sin, rot["dims"]), rotate_half(k, cos, sin, rot["dims"])
    q, k = stored(q), stored(k)
    k = k.repeat_interleave(H // G, dim=1)
    v = v.repeat_interleave(H // G, dim=1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = stored(masked_softmax_attention(q, k, v, m["scale"], window))
    return o.reshape(T, H * V) @ w["o"].T


def latent_attention_mixer(h, w: dict, m: dict, eps: float, stored=lambda t: t) -> torch.Tensor:
    """Attention whose keys and values are up-projections of one normed latent per token, without
    positions, in a sliding window."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = stored(h @ w["q"].T).view(T, H, D)
    c = stored(rms(stored(h @ w["dkv"].T), w["dkv.norm"], eps))
    k = (c @ w["uk"].T).view(T, H, D)
    v = (c @ w["uv"].T).view(T, H, V)
    window = m["mask"]["size"] if m.get("mask") else None
    o = stored(masked_softmax_attention(q, k, v, m["scale"], window))
    return o.reshape(T, H * V) @ w["o"].T


def causal_conv(x: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """x [T, C], taps [C, K]: out[t, c] = bias[c] + sum_j taps[c, j] x[t - (K - 1) + j, c], zeros
    before the start (the last tap is the current token's)."""
    T, C = x.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=x.dtype), x])
    out = bias.expand(T, C).clone()
    for j in range(K):
        out = out + padded[j : j + T] * taps[:, j]
    return out


def mamba2_mixer(h, w: dict, m: dict, eps: float, stored=lambda t: t) -> torch.Tensor:
    """A selective state-space layer with a scalar decay per head, token by token."""
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = stored(h @ w["in"].T)
    z, xbc, dt = proj[:, :inner], proj[:, inner : 2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N :]
    xbc = stored(silu(causal_conv(xbc, w["conv"], w["conv.b"])))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner : inner + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N :].view(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + w["dt_bias"])
    decay = torch.exp(-torch.exp(w["A_log"]) * dt)  # [T, H]
    S = torch.zeros(H, N, P, dtype=F64)
    y = torch.empty(T, H, P, dtype=F64)
    for t in range(T):
        S = decay[t][:, None, None] * S + dt[t][:, None, None] * B[t][:, :, None] * x[t][:, None, :]
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + w["D"][:, None] * x[t]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = stored(rms(y.view(T, parts, inner // parts), None, eps).reshape(T, inner) * w["norm"])
    return y @ w["o"].T


def gated_mlp(h, w: dict, stored=lambda t: t) -> torch.Tensor:
    inner = stored(gelu_tanh(stored(h @ w["gate"].T) + w["gate.b"]) * (stored(h @ w["up"].T) + w["up.b"]))
    return inner @ w["down"].T + w["down.b"]


MIXERS = {"attention": attention_mixer, "latent_attention": latent_attention_mixer, "mamba2": mamba2_mixer}


def sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False, stored=lambda t: t):
    """Logits [T, vocab] of one sequence (and the stream after every layer)."""
    eps = config["norm"]["eps"]
    tensors = {k: v.double() for k, v in tensors.items()}
    x = rms(tensors["embed"][torch.tensor(tokens)], tensors["embed.norm"], eps)
    after = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{layer.get('weights_of', i)}."
        mix = MIXERS[layer["type"]](stored(rms(x, tensors[p + "norm1"], eps)), sub(tensors, p + "mix."), layer["mixer"], eps, stored)
        x = x + rms(mix, tensors[p + "norm1b"], eps)
        if layer.get("mlp") is not None:
            ff = gated_mlp(stored(rms(x, tensors[p + "norm2"], eps)), sub(tensors, p + "mlp."), stored)
            x = x + rms(ff, tensors[p + "norm2b"], eps)
        after.append(x)
    logits = stored(rms(x, tensors["final.norm"], eps)) @ tensors["embed"].T
    cap = config.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return (logits, torch.stack(after)) if return_layers else logits


def tensor_shapes(config: dict) -> dict[str, tuple]:
    """Name -> shape of every tensor of a model with this configuration."""
    d = config["width"]
    shapes = {"embed": (config["vocab"], d), "embed.norm": (d,), "final.norm": (d,)}
    for i, layer in enumerate(config["layers"]):
        if "weights_of" in layer:
            continue
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "norm1b"] = (d,)
        if layer["type"] == "attention":
            H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * D, d), p + "mix.k": (G * D, d), p + "mix.v": (G * V, d), p + "mix.q.norm": (D,),
                           p + "mix.k.norm": (D,), p + "mix.o": (d, H * V)})  # fmt: skip
        elif layer["type"] == "latent_attention":
            H, D, V, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
            shapes.update({p + "mix.q": (H * D, d), p + "mix.dkv": (r, d), p + "mix.dkv.norm": (r,), p + "mix.uk": (H * D, r),
                           p + "mix.uv": (H * V, r), p + "mix.o": (d, H * V)})  # fmt: skip
        else:
            H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
            inner, channels = H * P, H * P + 2 * G * N
            shapes.update({p + "mix.in": (2 * inner + 2 * G * N + H, d), p + "mix.conv": (channels, m["conv"]), p + "mix.conv.b": (channels,),
                           p + "mix.dt_bias": (H,), p + "mix.A_log": (H,), p + "mix.D": (H,), p + "mix.norm": (inner,),
                           p + "mix.o": (d, inner)})  # fmt: skip
        if layer.get("mlp") is not None:
            f = layer["mlp"]["ff"]
            shapes[p + "norm2"] = shapes[p + "norm2b"] = (d,)
            shapes.update({p + "mlp.gate": (f, d), p + "mlp.gate.b": (f,), p + "mlp.up": (f, d), p + "mlp.up.b": (f,),
                           p + "mlp.down": (d, f), p + "mlp.down.b": (d,)})  # fmt: skip
    return shapes


def random_checkpoint(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random float32 weights whose matrices are exact in bfloat16: matrices N(0, 1 / fan_in) (the
    embedding N(0, 1), convolution taps N(0, 1 / taps)), gains 1 + N(0, 0.1), biases N(0, 0.3),
    step biases spread over (-3, 1) and decay rates over exp(-1.5 .. 1.5), so that some heads forget
    within a few tokens and others keep hundreds."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith("dt_bias"):
            w[name] = torch.linspace(-3.0, 1.0, shape[0])[torch.randperm(shape[0], generator=g)]
        elif name.endswith("A_log"):
            w[name] = torch.linspace(-1.5, 1.5, shape[0])[torch.randperm(shape[0], generator=g)]
        elif name.endswith(".b"):
            w[name] = 0.3 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            w[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            std = 1.0 if name == "embed" else shape[1] ** -0.5
            w[name] = (torch.randn(shape, generator=g) * std).bfloat16().float()
    return w


def greedy_generate(config: dict, tensors: dict, prompt: list[int], n: int) -> list[int]:
    """The n tokens that follow `prompt` when the largest logit is taken each time (the whole
    sequence is run again for every token: slow and stateless)."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt) :]
