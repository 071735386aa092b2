"""Tigesun as a ModelSpec: a decoder over a float32 residual stream whose layers norm the input and
the output of each sublayer, x <- x + N1b(mixer(N1(x))), x <- x + N2b(ff(N2(x))), all RMS norms with
a gain. Mixers: "attention" (grouped-query, per-head q/k norms, a rotate-half rotary encoding with
optionally stretched frequencies), "latent_attention" (keys and values up-projected from one cached
latent per token, no positions, a sliding window) and "mamba2" (a selective state-space layer). A
layer may run an earlier layer's tensors with a cache or state of its own. Layer i's tensors are
`l<i>.norm1`, `l<i>.norm1b`, `l<i>.mix.*`, `l<i>.norm2`, `l<i>.norm2b`, `l<i>.mlp.*`; the embedding
is `embed` with its norm `embed.norm`, the last norm `final.norm`, and the head is the embedding.

What the design fixes and the configuration therefore does not carry: the feed-forward's gated
form, its tanh-form GELU and its biases; the plain (not one-plus) gains; the q/k norms before the
rotation and their sharing among heads; the rotate-half pairing; the gate before the state-space
layer's norm; the tied head.
"""

from __future__ import annotations

from atomserve_b200.config.registry import register_architecture
from atomserve_b200.config.tigesun_config import TigesunConfig
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

ATTENTION_NAMES = dict(q="q", k="k", v="v", o="o", q_norm="q.norm", k_norm="k.norm")


def _mixer(c: TigesunConfig, layer: dict, prefix: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "attention":
        rot, position = m.get("rot"), None
        if rot is not None and rot["dims"]:
            s = rot.get("scaling")
            if s is not None:
                position = PartSpec("scaled_rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"],
                                                          factor=s["factor"], original=s["original"], fast=s["fast"],
                                                          slow=s["slow"]))  # fmt: skip
            else:
                position = PartSpec("rotary", dict(head_dim=m["dim"], theta=rot["base"], rotary_dim=rot["dims"]))
        mask = m.get("mask")
        return PartSpec("gqa_attention", dict(num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                              value_dim=m["vdim"], qk_norm_eps=c.norm_eps, position=position, scale=m["scale"],
                                              window=mask["size"] if mask else None, names=ATTENTION_NAMES), prefix)  # fmt: skip
    if layer["type"] == "latent_attention":
        mask = m.get("mask")
        return PartSpec("latent_attention", dict(heads=m["heads"], dim=m["dim"], rot_dim=0, vdim=m["vdim"], kv_rank=m["kv_rank"],
                                                 scale=m["scale"], eps=c.norm_eps, position=None, gated=False,
                                                 window=mask["size"] if mask else None), prefix)  # fmt: skip
    return PartSpec("selective_state_space", dict(heads=m["heads"], vdim=m["vdim"], state=m["state"], groups=m["groups"],
                                                  conv=m["conv"], norm_groups=m["norm_groups"], eps=c.norm_eps), prefix)  # fmt: skip


def build_spec(c: TigesunConfig) -> ModelSpec:
    layers, index_of = [], {}
    for i, layer in enumerate(c.layers):
        if c.source_of(i) == i:
            p = f"l{i}."
            mlp = layer.get("mlp")
            index_of[i] = len(layers)
            layers.append(LayerSpec(
                block="sandwich_norm",
                mixer=_mixer(c, layer, p + "mix."),
                feed_forward=(PartSpec("gated_mlp", dict(intermediate_size=mlp["ff"], activation="gelu_tanh", biases=True), p + "mlp.")
                              if mlp is not None else PartSpec("none")),
                mixer_norm=PartSpec("sandwich_norm", dict(eps=c.norm_eps, tensor=p + "norm1", out_tensor=p + "norm1b")),
                feed_forward_norm=(PartSpec("sandwich_norm", dict(eps=c.norm_eps, tensor=p + "norm2", out_tensor=p + "norm2b"))
                                   if mlp is not None else PartSpec("none")),
            ))  # fmt: skip
    schedule = [LayerCall(index_of[c.source_of(i)]) for i in range(len(c.layers))]
    return ModelSpec(
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("normed_embedding", dict(vocab_size=c.vocab, eps=c.norm_eps, tensor="embed", norm_tensor="embed.norm")),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("stream_rms_norm", dict(eps=c.norm_eps, tensor="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, tied=True, softcap=c.logit_softcap)),
    )


register_architecture(TigesunConfig.architecture, TigesunConfig, build_spec)
