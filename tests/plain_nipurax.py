"""A plain, slow implementation of the Nipurax design: one function per mechanism, float64, whole
sequences at once, no cache. It shares no code with the package; the GPU tests compare the engine
with it.

Nipurax is a decoder over a residual stream x [n, width]:

  x0 = embed[tok] + bigram[row(prev, tok)]                 a hashed table of token pairs
  the layers of `loop` run `times` times with the same weights; each pass starts with
      x <- Win [x ; x0] + step[t]
  a layer:  x <- x + m (mixer(N1 x) + ff(N2 x)),  N an RMS norm with a gain
  mixers:   "attention"    two softmax maps per head over the same values, within chunks of the
                           sequence, partly rotated q and k; o = a1 - lambda a2, unit RMS, (1 - diff)
            "attention_2"  causal softmax with a capped score, a query factor that grows with
                           the logarithm of the position, and a sink in the denominator
  ff:       routed experts over a softmax router with selection offsets, identity experts and a
            shared expert, all of the clamped form g sigmoid(1.702 g) (u + 1)
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def rms_norm(x: torch.Tensor, gain: torch.Tensor | None, eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if gain is None else y * gain


def pair_rows(tokens: list[int], buckets: int, mul_prev: int, mul_cur: int) -> list[int]:
    """Row of the pair table for each token: a hash of (previous, current), and the table's last
    row for a token that has no previous one."""
    rows = []
    for i, t in enumerate(tokens):
        rows.append(buckets if i == 0 else (tokens[i - 1] * mul_prev + t * mul_cur) % buckets)
    return rows


def embedding(tokens: list[int], embed: torch.Tensor, pair_table: torch.Tensor, cfg: dict) -> torch.Tensor:
    b = cfg["embedding"]["bigram"]
    rows = pair_rows(tokens, b["buckets"], b["mul_prev"], b["mul_cur"])
    return embed[tokens].to(F64) + pair_table[rows].to(F64)


def rotary_frequencies(rot: dict) -> torch.Tensor:
    """f_i = base^(-2i / dims), then stretched by wavelength: short waves (below original / high)
    stay, long ones (above original / low) are divided by `factor`, and in between the two are
    mixed linearly in original / wavelength."""
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    s = rot.get("scaling")
    if s is None:
        return f
    out = f.clone()
    for i in range(dims // 2):
        wave = 2.0 * math.pi / float(f[i])
        if wave < s["original"] / s["high"]:
            continue
        if wave > s["original"] / s["low"]:
            out[i] = f[i] / s["factor"]
        else:
            mix = (s["original"] / wave - s["low"]) / (s["high"] - s["low"])
            out[i] = (1.0 - mix) * f[i] / s["factor"] + mix * f[i]
    return out


def rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, dims: int) -> torch.Tensor:
    """x [n, ..., size]: entries i and i + dims / 2 of the first `dims` turn by position * f_i."""
    if dims == 0:
        return x
    half = dims // 2
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [half]
    angle = (positions.to(F64)[:, None] * freqs[None, :]).reshape(shape)
    c, s = torch.cos(angle), torch.sin(angle)
    a, b = x[..., :half], x[..., half:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def visible(n: int, chunk: int | None) -> torch.Tensor:
    """[n, n] bool: query i sees key j <= i, and with chunks only inside i's own chunk."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    ok = j <= i
    if chunk:
        ok = ok & (i // chunk == j // chunk)
    return ok


def softmax_with_sink(scores: torch.Tensor, ok: torch.Tensor, sink: torch.Tensor | None) -> torch.Tensor:
    """scores [heads, n, n]; masked keys weigh nothing; a sink adds exp(sink_h) to the denominator."""
    scores = scores.masked_fill(~ok, -math.inf)
    top = scores.max(-1, keepdim=True).values
    if sink is not None:
        top = torch.maximum(top, sink.to(F64)[:, None, None])
    e = torch.exp(scores - top)
    denom = e.sum(-1, keepdim=True)
    if sink is not None:
        denom = denom + torch.exp(sink.to(F64)[:, None, None] - top)
    return e / denom


def keep(t: torch.Tensor) -> torch.Tensor:
    return t


def differential_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0, stored=keep) -> torch.Tensor:
    """`stored` (here and below): applied to what an engine may keep in 16 bits between kernels."""
    n = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + n)
    q = stored(h @ w["q"].to(F64).T).view(n, H, 2, d)
    k = stored(h @ w["k"].to(F64).T).view(n, G, 2, d)
    v = stored(h @ w["v"].to(F64).T).view(n, G, vd)
    rot = m.get("rot")
    if rot is not None and rot["dims"]:
        f = rotary_frequencies(rot)
        q, k = stored(rotate(q, pos, f, rot["dims"])), stored(rotate(k, pos, f, rot["dims"]))
    share = H // G
    k = k.repeat_interleave(share, dim=1)
    v = v.repeat_interleave(share, dim=1)
    ok = visible(n, m["mask"]["size"] if m.get("mask") else None)
    outs = []
    for j in range(2):
        scores = torch.einsum("ihd,jhd->hij", q[:, :, j], k[:, :, j]) * m["scale"]
        outs.append(stored(torch.einsum("hij,jhv->ihv", softmax_with_sink(scores, ok, None), v)))
    lam = (torch.exp((w["lq1"].to(F64) * w["lk1"].to(F64)).sum()) - torch.exp((w["lq2"].to(F64) * w["lk2"].to(F64)).sum())
           + m["diff"])  # fmt: skip
    o = outs[0] - lam * outs[1]
    o = stored(rms_norm(o, None, eps) * (1.0 - m["diff"]))
    return o.reshape(n, H * vd) @ w["o"].to(F64).T


def query_factor(pos: torch.Tensor, temp: dict | None) -> torch.Tensor:
    if temp is None:
        return torch.ones(pos.shape[0], dtype=F64)
    return 1.0 + temp["coef"] * torch.log(torch.floor((pos.to(F64) + 1.0) / temp["every"]) + 1.0)


def sink_attention(h: torch.Tensor, w: dict, m: dict, start: int = 0, stored=keep) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + n)
    q = stored(stored(h @ w["q"].to(F64).T).view(n, H, d) * query_factor(pos, m.get("q_temp"))[:, None, None])
    k = stored(h @ w["k"].to(F64).T).view(n, G, d).repeat_interleave(H // G, dim=1)
    v = stored(h @ w["v"].to(F64).T).view(n, G, vd).repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    p = softmax_with_sink(scores, visible(n, None), w.get("sink"))
    return stored(torch.einsum("hij,jhv->ihv", p, v)).reshape(n, H * vd) @ w["o"].to(F64).T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float, stored=keep) -> torch.Tensor:
    g = torch.clamp(h @ gate.to(F64).T, max=limit)
    u = torch.clamp(h @ up.to(F64).T, -limit, limit)
    return stored(g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.to(F64).T


def route(h: torch.Tensor, router: torch.Tensor, offsets: torch.Tensor, top: int, scale: float):
    """(chosen [n, top], weights [n, top]): softmax scores over all router outputs; the choice
    is by score + offset, the weight is the score itself times `scale`."""
    s = torch.softmax(h @ router.to(F64).T, dim=-1)
    chosen = torch.topk(s + offsets.to(F64), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * scale


def choice_margin(h: torch.Tensor, router: torch.Tensor, offsets: torch.Tensor, top: int) -> torch.Tensor:
    """[n]: by how much the last chosen expert's selection score leads the best one left out (inf where
    every expert is chosen). A small margin is a close call that rounding may decide otherwise."""
    c = torch.softmax(h @ router.to(F64).T, dim=-1) + offsets.to(F64)
    ranked = c.sort(-1, descending=True).values
    if top >= ranked.shape[1]:
        return torch.full((h.shape[0],), math.inf, dtype=F64)
    return ranked[:, top - 1] - ranked[:, top]


def routed_experts(h: torch.Tensor, w: dict, mlp: dict, stored=keep, margins: list | None = None) -> torch.Tensor:
    r = mlp["router"]
    E = r["experts"]
    chosen, weights = route(h, w["router"], w["correction"], r["top"], r["scale"])
    if margins is not None:
        margins.append(choice_margin(h, w["router"], w["correction"], r["top"]))
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0] if E else h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            if e >= E:  # an identity expert gives back what it was given
                out[t] += wt * h[t]
            else:
                out[t] += wt * clamped_expert(h[t : t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"]["limit"], stored)[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"], stored)
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix) :]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x: torch.Tensor, weights: dict, i: int, cfg: dict, stored=keep, margins: list | None = None) -> torch.Tensor:
    spec, eps = cfg["layers"][i], cfg["norm"]["eps"]
    h1 = stored(rms_norm(x, weights[f"l{i}.norm1"].to(F64), eps))
    w = sub(weights, f"l{i}.mix.")
    if spec["type"] == "attention":
        y = differential_attention(h1, w, spec["mixer"], eps, stored=stored)
    elif spec["type"] == "attention_2":
        y = sink_attention(h1, w, spec["mixer"], stored=stored)
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp") is not None:
        h2 = stored(rms_norm(x, weights[f"l{i}.norm2"].to(F64), eps))
        y = y + routed_experts(h2, sub(weights, f"l{i}.mlp."), spec["mlp"], stored, margins)
    return x + cfg["residual_mult"] * y


def run_order(cfg: dict) -> list[tuple[int, int | None]]:
    """(layer, pass number where the layer opens a pass of the loop)."""
    n, loop = len(cfg["layers"]), cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    order = [(i, None) for i in range(loop["start"])]
    for t in range(loop["times"]):
        order += [(i, t if i == loop["start"] else None) for i in range(loop["start"], loop["stop"])]
    return order + [(i, None) for i in range(loop["stop"], n)]


def forward(tokens: list[int], weights: dict, cfg: dict, streams: list | None = None, stored=keep,
            margins: list | None = None) -> torch.Tensor:
    """float64 logits [n, vocab]; `streams`, if a list, collects x after every layer run, and
    `margins` the routers' margins of choice per position (`choice_margin`), one entry per run."""
    x0 = embedding(tokens, weights["embed"], weights["bigram"], cfg)
    x = x0
    for i, opens in run_order(cfg):
        if opens is not None:
            x = stored(torch.cat([x, x0], dim=-1)) @ weights["loop.in"].to(F64).T + weights["loop.step"][opens].to(F64)
        x = layer(x, weights, i, cfg, stored, margins)
        if streams is not None:
            streams.append(x)
    x = stored(rms_norm(x, weights["final.norm"].to(F64), cfg["norm"]["eps"]))
    return x @ weights["head"].to(F64).T


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    d = cfg["width"]
    shapes = {"embed": (cfg["vocab"], d), "bigram": (cfg["embedding"]["bigram"]["buckets"] + 1, d)}
    if cfg.get("loop"):
        shapes["loop.in"], shapes["loop.step"] = (d, 2 * d), (cfg["loop"]["times"], d)
    for i, spec in enumerate(cfg["layers"]):
        p, m = f"l{i}.", spec["mixer"]
        maps = 2 if spec["type"] == "attention" else 1
        shapes[p + "norm1"] = (d,)
        shapes[p + "mix.q"] = (m["heads"] * maps * m["dim"], d)
        shapes[p + "mix.k"] = (m["kv_heads"] * maps * m["dim"], d)
        shapes[p + "mix.v"] = (m["kv_heads"] * m["vdim"], d)
        shapes[p + "mix.o"] = (d, m["heads"] * m["vdim"])
        if spec["type"] == "attention":
            for n in ("lq1", "lk1", "lq2", "lk2"):
                shapes[p + "mix." + n] = (m["dim"],)
        else:
            shapes[p + "mix.sink"] = (m["heads"],)
        mlp = spec.get("mlp")
        if mlp is None:
            continue
        shapes[p + "norm2"] = (d,)
        r, ff = mlp["router"], mlp["expert"]["ff"]
        for e in range(r["experts"]):
            shapes[f"{p}mlp.e{e}.gate"], shapes[f"{p}mlp.e{e}.up"], shapes[f"{p}mlp.e{e}.down"] = (ff, d), (ff, d), (d, ff)
        routed = r["experts"] + r.get("identity", 0)
        shapes[p + "mlp.router"], shapes[p + "mlp.correction"] = (routed, d), (routed,)
        if mlp.get("shared") is not None:
            s = mlp["shared"]["ff"]
            shapes[p + "mlp.shared.gate"], shapes[p + "mlp.shared.up"], shapes[p + "mlp.shared.down"] = (s, d), (s, d), (d, s)
    shapes["final.norm"], shapes["head"] = (d,), (cfg["vocab"], d)
    return shapes


def random_checkpoint(cfg: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random float32 weights whose matrices are exact in bfloat16: matrices N(0, 1 / fan_in) (the two
    embedding tables N(0, 1), routers N(0, 4 / fan_in) so that choices are seldom close), gains
    1 + N(0, 0.1), the vectors of lambda N(0, 0.3 / sqrt(dim)), sinks N(0, 1), selection offsets
    N(0, 0.05), pass vectors N(0, 0.3)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        last = name.rsplit(".", 1)[-1]
        if last in ("lq1", "lk1", "lq2", "lk2"):
            w[name] = torch.randn(shape, generator=g) * (0.3**0.5) * shape[0] ** -0.25
        elif last == "sink":
            w[name] = torch.randn(shape, generator=g)
        elif last == "correction":
            w[name] = 0.05 * torch.randn(shape, generator=g)
        elif name == "loop.step":
            w[name] = 0.3 * torch.randn(shape, generator=g)
        elif len(shape) == 1:
            w[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            std = 1.0 if name in ("embed", "bigram") else (2.0 if last == "router" else 1.0) * shape[1] ** -0.5
            w[name] = (torch.randn(shape, generator=g) * std).bfloat16().float()
    return w


def greedy_generate(tokens: list[int], weights: dict, cfg: dict, n: int) -> list[int]:
    """The n tokens that follow when the largest logit is taken each time (the whole sequence is
    run again for every token: slow and stateless)."""
    tokens = list(tokens)
    first = len(tokens)
    for _ in range(n):
        tokens.append(int(forward(tokens, weights, cfg)[-1].argmax()))
    return tokens[first:]
