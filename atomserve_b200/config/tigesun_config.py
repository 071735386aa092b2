"""Typed configuration of the Tigesun design, read from its own config.json keys.

A Tigesun model is a list of layers around a float32 residual stream; each layer norms the input and
the output of its mixer and then of its feed-forward (if it has one). A layer's mixer is "attention"
(grouped-query attention with per-head q/k norms and a rotary encoding whose frequencies may be
stretched), "latent_attention" (attention over a cached latent in a sliding window, no positions) or
"mamba2" (a selective state-space layer). A layer with `weights_of: j` runs layer j's tensors with a
cache or state of its own. Every size and every constant that may differ between models is a key;
what the design fixes is written in `models/tigesun.py`.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from atomserve_b200.config.gefilix_config import _need
from atomserve_b200.config.model_config import ModelConfigError

MIXERS = ("attention", "latent_attention", "mamba2")


@dataclass(frozen=True)
class TigesunConfig:
    vocab: int
    width: int
    layers: tuple[dict[str, Any], ...]
    norm_eps: float
    logit_softcap: float | None = None
    max_positions: int = 1 << 20  # no learned or tabulated positions: no limit of the design's own

    architecture = "Tigesun"

    @classmethod
    def from_dict(cls, raw: dict) -> "TigesunConfig":
        name = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if name != cls.architecture:
            raise ModelConfigError(f"expected architecture {cls.architecture!r}, got {name!r}")
        _need(raw, ("vocab", "width", "layers", "norm"), "config.json")
        _need(raw["norm"], ("eps",), "config.json norm")
        cap = raw.get("logit_softcap")
        config = cls(
            vocab=int(raw["vocab"]),
            width=int(raw["width"]),
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float(raw["norm"]["eps"]),
            logit_softcap=float(cap) if cap else None,
            max_positions=int(raw.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def source_of(self, i: int) -> int:
        """The layer whose tensors layer i runs (through any chain of `weights_of`)."""
        seen = {i}
        while self.layers[i].get("weights_of") is not None:
            i = int(self.layers[i]["weights_of"])
            if i in seen:
                raise ModelConfigError(f"layer {i}: weights_of runs in a circle")
            seen.add(i)
        return i

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ModelConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps >= 0:
            raise ModelConfigError("norm.eps must be >= 0")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ModelConfigError("logit_softcap must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer.get("weights_of") is not None:
                j = layer["weights_of"]
                if not isinstance(j, int) or not 0 <= j < len(self.layers) or j == i:
                    raise ModelConfigError(f"{where}: weights_of must name another layer")
                j = self.source_of(i)
                if any(layer.get(k) != self.layers[j].get(k) for k in ("type", "mixer", "mlp")):
                    raise ModelConfigError(f"{where}: a layer that runs layer {j}'s tensors must have layer {j}'s sizes")
            if layer["type"] == "attention":
                _need(m, ("heads", "kv_heads", "dim", "vdim", "scale"), where + " mixer")
                if m["heads"] % m["kv_heads"]:
                    raise ModelConfigError(f"{where}: {m['heads']} heads are not a multiple of {m['kv_heads']} kv heads")
                rot = m.get("rot")
                if rot is not None:
                    _need(rot, ("base", "dims"), where + " mixer rot")
                    if rot["dims"] % 2 or not 0 <= rot["dims"] <= m["dim"]:
                        raise ModelConfigError(f"{where}: rot.dims {rot['dims']} must be even and at most dim {m['dim']}")
                    if rot.get("scaling") is not None:
                        _need(rot["scaling"], ("factor", "original", "fast", "slow"), where + " mixer rot scaling")
            elif layer["type"] == "latent_attention":
                _need(m, ("heads", "dim", "vdim", "kv_rank", "scale"), where + " mixer")
                if m.get("mask") is not None:
                    _need(m["mask"], ("size",), where + " mixer mask")
                    if m["mask"]["size"] < 1:
                        raise ModelConfigError(f"{where}: mask.size must be positive")
            elif layer["type"] == "mamba2":
                _need(m, ("heads", "vdim", "state", "groups", "conv", "norm_groups"), where + " mixer")
                if m["heads"] % m["groups"] or (m["heads"] * m["vdim"]) % m["norm_groups"] or m["conv"] < 1:
                    raise ModelConfigError(f"{where}: heads must be a multiple of groups, heads * vdim of norm_groups, conv >= 1")
            else:
                raise ModelConfigError(f"{where}: mixer type {layer['type']!r} is not one of {MIXERS}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind", "ff"), where + " mlp")
            if mlp["kind"] != "dense":
                raise ModelConfigError(f"{where}: mlp kind {mlp['kind']!r} is not 'dense'")

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        out = {
            "architecture": self.architecture,
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.logit_softcap is not None:
            out["logit_softcap"] = self.logit_softcap
        return out
