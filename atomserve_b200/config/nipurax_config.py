"""Typed configuration of the Nipurax design, read from its own config.json keys.

A Nipurax model is a list of layers around a float32 residual stream; a layer adds its mixer and its
feed-forward, both reading the same stream through norms of their own, times `residual_mult`. A
layer's mixer is "attention" (differential attention within chunks of the sequence, partly rotated)
or "attention_2" (causal attention with capped scores, a query factor that grows with the position
and a sink); its feed-forward is a mixture of experts or absent. `loop` names a stretch of layers
that runs several times with the same weights. The embedding adds a hashed table of token pairs.
Every size and every constant that may differ between models is a key; what the design fixes is
written in `models/nipurax.py`.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from atomserve_b200.config.gefilix_config import _need
from atomserve_b200.config.model_config import ModelConfigError

MIXERS = ("attention", "attention_2")


@dataclass(frozen=True)
class NipuraxConfig:
    vocab: int
    width: int
    layers: tuple[dict[str, Any], ...]
    norm_eps: float
    residual_mult: float
    bigram: dict[str, int]
    loop: dict[str, int] | None = None
    max_positions: int = 1 << 20  # no learned or tabulated positions: no limit of the design's own

    architecture = "Nipurax"

    @classmethod
    def from_dict(cls, raw: dict) -> "NipuraxConfig":
        name = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if name != cls.architecture:
            raise ModelConfigError(f"expected architecture {cls.architecture!r}, got {name!r}")
        _need(raw, ("vocab", "width", "layers", "norm", "residual_mult", "embedding"), "config.json")
        _need(raw["norm"], ("eps",), "config.json norm")
        _need(raw["embedding"], ("bigram",), "config.json embedding")
        _need(raw["embedding"]["bigram"], ("buckets", "mul_prev", "mul_cur"), "config.json embedding bigram")
        loop = raw.get("loop")
        if loop is not None:
            _need(loop, ("start", "stop", "times"), "config.json loop")
            loop = {k: int(loop[k]) for k in ("start", "stop", "times")}
        config = cls(
            vocab=int(raw["vocab"]),
            width=int(raw["width"]),
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float(raw["norm"]["eps"]),
            residual_mult=float(raw["residual_mult"]),
            bigram={k: int(raw["embedding"]["bigram"][k]) for k in ("buckets", "mul_prev", "mul_cur")},
            loop=loop,
            max_positions=int(raw.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def run_order(self) -> list[tuple[int, int | None]]:
        """(layer, the number of the pass it opens or None), in the order the layers run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, None) for i in range(n)]
        start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        order: list[tuple[int, int | None]] = [(i, None) for i in range(start)]
        for t in range(times):
            order += [(i, t if i == start else None) for i in range(start, stop)]
        return order + [(i, None) for i in range(stop, n)]

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ModelConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps >= 0:
            raise ModelConfigError("norm.eps must be >= 0")
        if self.bigram["buckets"] < 1 or self.bigram["mul_prev"] < 0 or self.bigram["mul_cur"] < 0:
            raise ModelConfigError("embedding.bigram needs buckets >= 1 and multipliers >= 0")
        if self.loop is not None:
            start, stop, times = self.loop["start"], self.loop["stop"], self.loop["times"]
            if not 0 <= start < stop <= len(self.layers) or times < 1:
                raise ModelConfigError(f"loop {start}..{stop} x {times} does not fit {len(self.layers)} layers")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] not in MIXERS:
                raise ModelConfigError(f"{where}: mixer type {layer['type']!r} is not one of {MIXERS}")
            _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where + " mixer")
            if m["heads"] < 1 or m["kv_heads"] < 1 or m["heads"] % m["kv_heads"]:
                raise ModelConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
            if layer["type"] == "attention":
                _need(m, ("diff",), where + " mixer")
                rot = m.get("rot")
                if rot is not None:
                    _need(rot, ("base", "dims"), where + " mixer rot")
                    if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["dim"]:
                        raise ModelConfigError(f"{where}: rot.dims {rot['dims']} must be even and at most dim {m['dim']}")
                    if rot.get("scaling") is not None:
                        _need(rot["scaling"], ("factor", "low", "high", "original"), where + " mixer rot scaling")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), where + " mixer mask")
                    if m["mask"]["size"] < 1:
                        raise ModelConfigError(f"{where}: mask.size must be positive")
            else:
                if m.get("q_temp") is not None:
                    _need(m["q_temp"], ("coef", "every"), where + " mixer q_temp")
                    if m["q_temp"]["every"] < 1:
                        raise ModelConfigError(f"{where}: q_temp.every must be positive")
                if m.get("softcap") is not None and not m["softcap"] > 0:
                    raise ModelConfigError(f"{where}: softcap must be positive")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind", "expert", "router"), where + " mlp")
            if mlp["kind"] != "moe":
                raise ModelConfigError(f"{where}: mlp kind {mlp['kind']!r} is not 'moe'")
            _need(mlp["expert"], ("ff", "limit"), where + " mlp expert")
            r = mlp["router"]
            _need(r, ("experts", "top", "scale"), where + " mlp router")
            if r["experts"] < 1 or r.get("identity", 0) < 0 or not 1 <= r["top"] <= r["experts"] + r.get("identity", 0):
                raise ModelConfigError(f"{where}: cannot choose {r['top']} of {r['experts']} + {r.get('identity', 0)} experts")
            if r["top"] > 32:
                raise ModelConfigError(f"{where}: at most 32 experts a token")
            if mlp.get("shared") is not None:
                _need(mlp["shared"], ("ff", "limit"), where + " mlp shared")

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        out = {
            "architecture": self.architecture,
            "embedding": {"bigram": dict(self.bigram)},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out
