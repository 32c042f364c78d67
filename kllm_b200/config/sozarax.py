"""``SozaraxConfig``: the keys of a Sozarax ``config.json`` as the engine reads them.

    architecture   "Sozarax"
    vocab, width   sizes of the embedding
    embedding      {scale}: every embedded row is multiplied by it
    norm           {eps}: of every RMS norm of the model
    layers         a list; each entry {type, mixer, mlp}:
                   type "wkv":        mixer {heads, dim}
                   type "attention":  mixer {heads, kv_heads, dim, vdim, scale, q_temp {coef, every}}
                   mlp null | {kind "dense", ff} | {kind "moe", expert {ff}, router {experts, top}}
    loop           {start, stop, times}: layers start .. stop-1 run ``times`` times in a row
                   (absent: every layer once)

Everything a model of this design may vary is read from here; nothing is defaulted to the
values of one particular model.  ``q_temp`` may be absent (no temperature on the queries).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigError, ModelConfig, take_float, take_int


def _obj(d, key, where="config.json"):
    v = d.get(key)
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: '{key}' must be an object")
    return v


@dataclass(frozen=True)
class WkvMixerConfig:
    heads: int
    dim: int

    def to_dict(self):
        return {"heads": self.heads, "dim": self.dim}


@dataclass(frozen=True)
class AttentionMixerConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp_coef: float          # 0: no temperature
    q_temp_every: int

    def to_dict(self):
        d = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim, "scale": self.scale}
        if self.q_temp_coef != 0.0:
            d["q_temp"] = {"coef": self.q_temp_coef, "every": self.q_temp_every}
        return d


@dataclass(frozen=True)
class MlpConfig:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense layer, or of one expert
    experts: int = 0
    top: int = 0

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "expert": {"ff": self.ff}, "router": {"experts": self.experts, "top": self.top}}


@dataclass(frozen=True)
class LayerConfig:
    type: str                   # "wkv" | "attention"
    mixer: object
    mlp: Optional[MlpConfig]

    def to_dict(self):
        return {"type": self.type, "mixer": self.mixer.to_dict(), "mlp": self.mlp.to_dict() if self.mlp else None}


@dataclass(frozen=True)
class SozaraxConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[LayerConfig, ...]
    loop_start: int
    loop_stop: int
    loop_times: int

    @classmethod
    def from_dict(cls, d: dict) -> "SozaraxConfig":
        vocab = take_int(d, "vocab", minimum=1)
        width = take_int(d, "width", minimum=1)
        scale = take_float(_obj(d, "embedding"), "scale")
        eps = take_float(_obj(d, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"config.json: layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{where} must be an object")
            kind, m = L.get("type"), _obj(L, "mixer", where)
            if kind == "wkv":
                mixer = WkvMixerConfig(take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1))
            elif kind == "attention":
                heads, kv = take_int(m, "heads", minimum=1), take_int(m, "kv_heads", minimum=1)
                if heads % kv:
                    raise ConfigError(f"{where}: {heads} heads are not a multiple of {kv} kv_heads")
                qt = m.get("q_temp")
                coef, every = 0.0, 1
                if qt is not None:
                    coef, every = take_float(qt, "coef"), take_int(qt, "every", minimum=1)
                mixer = AttentionMixerConfig(heads, kv, take_int(m, "dim", minimum=1), take_int(m, "vdim", minimum=1),
                                             take_float(m, "scale"), coef, every)
            else:
                raise ConfigError(f"{where}: unknown layer type {kind!r} (wkv, attention)")
            ml, mlp = L.get("mlp"), None
            if ml is not None:
                if not isinstance(ml, dict):
                    raise ConfigError(f"{where}: 'mlp' must be an object or null")
                if ml.get("kind") == "dense":
                    mlp = MlpConfig("dense", take_int(ml, "ff", minimum=1))
                elif ml.get("kind") == "moe":
                    r = _obj(ml, "router", where)
                    mlp = MlpConfig("moe", take_int(_obj(ml, "expert", where), "ff", minimum=1),
                                    take_int(r, "experts", minimum=1), take_int(r, "top", minimum=1))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"{where}: top {mlp.top} of {mlp.experts} experts")
                else:
                    raise ConfigError(f"{where}: unknown mlp kind {ml.get('kind')!r} (dense, moe)")
            layers.append(LayerConfig(kind, mixer, mlp))
        loop = d.get("loop")
        start, stop, times = 0, 0, 1
        if loop is not None:
            if not isinstance(loop, dict):
                raise ConfigError("config.json: 'loop' must be an object")
            start, stop = take_int(loop, "start", minimum=0), take_int(loop, "stop", minimum=0)
            times = take_int(loop, "times", minimum=1)
            if not (start <= stop <= len(layers)):
                raise ConfigError(f"config.json: loop {start}..{stop} does not lie within the {len(layers)} layers")
        return cls(architecture="Sozarax", vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps,
                   layers=tuple(layers), loop_start=start, loop_stop=stop, loop_times=times)

    def layer_order(self):
        """Indices of the layers in the order they run."""
        n = len(self.layers)
        a, b = self.loop_start, self.loop_stop
        return list(range(a)) + list(range(a, b)) * self.loop_times + list(range(b, n))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": [L.to_dict() for L in self.layers]}
        if self.loop_stop > self.loop_start:
            d["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return d
