"""Nipurax as a ModelSpec: a decoder over a float32 residual stream whose layers add mixer and
feed-forward side by side, x <- x + mult (mixer(N1 x) + ff(N2 x)), with RMS norms with a gain.
Mixers: "attention" (differential attention: two softmax maps a head over the same values, partly
rotated q and k with frequencies stretched by wavelength, within chunks of the sequence) and
"attention_2" (causal attention without positions in q and k, a query factor that grows with the
logarithm of the position, capped scores and a sink). The feed-forward is routed experts of the
clamped form with a softmax router, selection offsets, identity experts and a shared expert, or
absent. A stretch of layers may run several times with the same weights and a cache of its own
each time; every pass opens with x <- Win [x ; x0] + step[pass]. The embedding adds a hashed table
of token pairs. Layer i's tensors are `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.*`, `l<i>.mlp.*`; the
others `embed`, `bigram`, `loop.in`, `loop.step`, `final.norm`, `head`.

What the design fixes and the configuration therefore does not carry: the experts' form
g sigmoid(1.702 g) (u + 1) with g capped from above and u from both sides; the softmax router whose
weights are not renormalised; the ungated shared expert; the rotate-half pairing; the unit-RMS norm
of the maps' difference and its factor 1 - diff; the untied head.
"""

from __future__ import annotations

from atomserve_b200.config.nipurax_config import NipuraxConfig
from atomserve_b200.config.registry import register_architecture
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

EXPERT_SLOPE, EXPERT_SHIFT = 1.702, 1.0
SINK_NAMES = dict(q="q", k="k", v="v", o="o", sink="sink")


def _mixer(c: NipuraxConfig, layer: dict, prefix: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        rot, position = m.get("rot"), None
        if rot is not None and rot["dims"]:
            s = rot.get("scaling")
            if s is not None:
                position = PartSpec("band_scaled_rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"],
                                                               factor=s["factor"], original=s["original"], low=s["low"],
                                                               high=s["high"]))  # fmt: skip
            else:
                position = PartSpec("rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"]))
        mask = m.get("mask")
        return PartSpec("differential_attention", dict(num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                                       value_dim=m["vdim"], scale=m["scale"], diff=m["diff"], eps=c.norm_eps,
                                                       position=position, chunk=mask["size"] if mask else None), prefix)  # fmt: skip
    temp = m.get("q_temp")
    return PartSpec("gqa_attention", dict(num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                          value_dim=m["vdim"], scale=m["scale"], names=SINK_NAMES, sink=True,
                                          softcap=m.get("softcap"),
                                          query_temperature=(temp["coef"], temp["every"]) if temp else (0.0, 1)), prefix)  # fmt: skip


def _feed_forward(mlp: dict | None, prefix: str) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    r, shared = mlp["router"], mlp.get("shared")
    return PartSpec("routed_experts", dict(
        experts=r["experts"], top=r["top"], expert_ff=mlp["expert"]["ff"], limit=mlp["expert"]["limit"], scale=r["scale"],
        slope=EXPERT_SLOPE, shift=EXPERT_SHIFT, score="softmax", renormalise=False, identity=r.get("identity", 0),
        choice_offsets=True, shared_ff=shared["ff"] if shared else None, shared_limit=shared["limit"] if shared else None,
        shared_gated=False), prefix)  # fmt: skip


def build_spec(c: NipuraxConfig) -> ModelSpec:
    layers = []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        mlp = layer.get("mlp")
        layers.append(LayerSpec(
            block="parallel_residual",
            mixer=_mixer(c, layer, p + "mix."),
            feed_forward=_feed_forward(mlp, p + "mlp."),
            mixer_norm=PartSpec("scaled_rms_norm", dict(eps=c.norm_eps, mult=c.residual_mult, tensor=p + "norm1")),
            feed_forward_norm=(PartSpec("rms_norm", dict(eps=c.norm_eps, tensor=p + "norm2")) if mlp is not None else PartSpec("none")),
        ))  # fmt: skip
    schedule = [LayerCall(i, before=(0, opens) if opens is not None else None) for i, opens in c.run_order()]
    steps = (PartSpec("mix_with_input", dict(uses=c.loop["times"], tensor="loop.in", step_tensor="loop.step")),) if c.loop else ()
    return ModelSpec(
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("pair_hash_embedding", dict(vocab_size=c.vocab, buckets=c.bigram["buckets"], mul_prev=c.bigram["mul_prev"],
                                                       mul_cur=c.bigram["mul_cur"], tensor="embed", pair_tensor="bigram")),  # fmt: skip
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("stream_rms_norm", dict(eps=c.norm_eps, tensor="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, tied=False, tensor="head")),
        stream_steps=steps,
    )


register_architecture(NipuraxConfig.architecture, NipuraxConfig, build_spec)
