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


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


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


def differential_attention(h: torch.Tensor, w: dict, m: dict, eps: float, start: int = 0) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + n)
    q = (h @ w["q"].to(F64).T).view(n, H, 2, d)
    k = (h @ w["k"].to(F64).T).view(n, G, 2, d)
    v = (h @ w["v"].to(F64).T).view(n, G, vd)
    rot = m.get("rot")
    if rot is not None and rot["dims"]:
        f = rotary_frequencies(rot)
        q, k = rotate(q, pos, f, rot["dims"]), rotate(k, pos, f, rot["dims"])
    share = H // G
    k = k.repeat_interleave(share, dim=1)
    v = v.repeat_interleave(share, dim=1)
    ok = visible(n, m["mask"]["size"] if m.get("mask") else None)
    outs = []
    for j in range(2):
        scores = torch.einsum("ihd,jhd->hij", q[:, :, j], k[:, :, j]) * m["scale"]
        outs.append(torch.einsum("hij,jhv->ihv", softmax_with_sink(scores, ok, None), v))
    lam = (torch.exp((w["lq1"].to(F64) * w["lk1"].to(F64)).sum()) - torch.exp((w["lq2"].to(F64) * w["lk2"].to(F64)).sum())
           + m["diff"])  # fmt: skip
    o = outs[0] - lam * outs[1]
    o = rms_norm(o, None, eps) * (1.0 - m["diff"])
    return o.reshape(n, H * vd) @ w["o"].to(F64).T


def query_factor(pos: torch.Tensor, temp: dict | None) -> torch.Tensor:
    if temp is None:
        return torch.ones(pos.shape[0], dtype=F64)
    return 1.0 + temp["coef"] * torch.log(torch.floor((pos.to(F64) + 1.0) / temp["every"]) + 1.0)


def sink_attention(h: torch.Tensor, w: dict, m: dict, start: int = 0) -> torch.Tensor:
    n = h.shape[0]
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(start, start + n)
    q = (h @ w["q"].to(F64).T).view(n, H, d) * query_factor(pos, m.get("q_temp"))[:, None, None]
    k = (h @ w["k"].to(F64).T).view(n, G, d).repeat_interleave(H // G, dim=1)
    v = (h @ w["v"].to(F64).T).view(n, G, vd).repeat_interleave(H // G, dim=1)
    scores = torch.einsum("ihd,jhd->hij", q, k) * m["scale"]
    cap = m.get("softcap")
    if cap:
        scores = cap * torch.tanh(scores / cap)
    p = softmax_with_sink(scores, visible(n, None), w.get("sink"))
    return torch.einsum("hij,jhv->ihv", p, v).reshape(n, H * vd) @ w["o"].to(F64).T


def clamped_expert(h: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ gate.to(F64).T, max=limit)
    u = torch.clamp(h @ up.to(F64).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ down.to(F64).T


def route(h: torch.Tensor, router: torch.Tensor, offsets: torch.Tensor, top: int, scale: float):
    """(chosen [n, top], weights [n, top]): softmax scores over all router outputs; the choice
    is by score + offset, the weight is the score itself times `scale`."""
    s = torch.softmax(h @ router.to(F64).T, dim=-1)
    chosen = torch.topk(s + offsets.to(F64), top, dim=-1).indices
    return chosen, torch.gather(s, 1, chosen) * scale


def routed_experts(h: torch.Tensor, w: dict, mlp: dict) -> torch.Tensor:
    r = mlp["router"]
    E = r["experts"]
    chosen, weights = route(h, w["router"], w["correction"], r["top"], r["scale"])
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0] if E else h.shape[1], dtype=F64)
    for t in range(h.shape[0]):
        for e, wt in zip(chosen[t].tolist(), weights[t]):
            if e >= E:  # an identity expert gives back what it was given
                out[t] += wt * h[t]
            else:
                out[t] += wt * clamped_expert(h[t : t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"]["limit"])[0]
    if mlp.get("shared") is not None:
        out = out + clamped_expert(h, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"])
    return out


def sub(weights: dict, prefix: str) -> dict:
    return {k[len(prefix) :]: v for k, v in weights.items() if k.startswith(prefix)}


def layer(x: torch.Tensor, weights: dict, i: int, cfg: dict) -> torch.Tensor:
    spec, eps = cfg["layers"][i], cfg["norm"]["eps"]
    h1 = rms_norm(x, weights[f"l{i}.norm1"].to(F64), eps)
    w = sub(weights, f"l{i}.mix.")
    if spec["type"] == "attention":
        y = differential_attention(h1, w, spec["mixer"], eps)
    elif spec["type"] == "attention_2":
        y = sink_attention(h1, w, spec["mixer"])
    else:
        raise ValueError(spec["type"])
    if spec.get("mlp") is not None:
        h2 = rms_norm(x, weights[f"l{i}.norm2"].to(F64), eps)
        y = y + routed_experts(h2, sub(weights, f"l{i}.mlp."), spec["mlp"])
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


def forward(tokens: list[int], weights: dict, cfg: dict, streams: list | None = None) -> torch.Tensor:
    """float64 logits [n, vocab]; `streams`, if a list, collects x after every layer run."""
    x0 = embedding(tokens, weights["embed"], weights["bigram"], cfg)
    x = x0
    for i, opens in run_order(cfg):
        if opens is not None:
            x = torch.cat([x, x0], dim=-1) @ weights["loop.in"].to(F64).T + weights["loop.step"][opens].to(F64)
        x = layer(x, weights, i, cfg)
        if streams is not None:
            streams.append(x)
    x = rms_norm(x, weights["final.norm"].to(F64), cfg["norm"]["eps"])
    return x @ weights["head"].to(F64).T
