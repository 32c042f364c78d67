"""``NutizenConfig``: the keys of a Nutizen ``config.json`` as the engine reads them.

    architecture   "Nutizen"
    vocab, width   sizes of the embedding
    embedding      {scale}: every embedded row is multiplied by it
    norm           {eps}: of every RMS norm of the model
    streams        number of residual streams (absent: one plain residual stream)
    layers         a list; each entry {type "latent_attention", mixer, mlp}:
                   mixer {heads, dim, vdim, q_rank, kv_rank, scale, mask {size}, kv_from}
                       mask absent: every earlier key is visible; kv_from j (optional): the layer
                       has no key/value latent of its own and reads the one layer j caches
                   mlp null | {kind "dense", ff}
                       | {kind "moe", expert {ff, limit}, router {experts, top}, shared {ff, limit} | absent}

Everything a model of this design may vary is read from here; nothing is defaulted to the
values of one particular model.
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
class LatentMixerConfig:
    heads: int
    dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    window: Optional[int]       # None: no window
    kv_from: Optional[int]      # None: the layer has a key/value latent of its own

    def to_dict(self):
        d = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "q_rank": self.q_rank, "kv_rank": self.kv_rank,
             "scale": self.scale}
        if self.window is not None:
            d["mask"] = {"size": self.window}
        if self.kv_from is not None:
            d["kv_from"] = self.kv_from
        return d


@dataclass(frozen=True)
class NutizenMlpConfig:
    kind: str                   # "dense" | "moe"
    ff: int                     # of the dense layer, or of one expert
    limit: float = 0.0          # of an expert's activation
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert
    shared_limit: float = 0.0

    def to_dict(self):
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        d = {"kind": "moe", "expert": {"ff": self.ff, "limit": self.limit},
             "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            d["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return d


@dataclass(frozen=True)
class NutizenLayerConfig:
    mixer: LatentMixerConfig
    mlp: Optional[NutizenMlpConfig]

    def to_dict(self):
        return {"type": "latent_attention", "mixer": self.mixer.to_dict(),
                "mlp": self.mlp.to_dict() if self.mlp else None}


def _limit(d, where):
    v = take_float(d, "limit")
    if v <= 0:
        raise ConfigError(f"{where}: 'limit' must be positive, got {v}")
    return v


@dataclass(frozen=True)
class NutizenConfig(ModelConfig):
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    streams: int                # 0: one plain residual stream
    layers: Tuple[NutizenLayerConfig, ...]

    @classmethod
    def from_dict(cls, d: dict) -> "NutizenConfig":
        vocab = take_int(d, "vocab", minimum=1)
        width = take_int(d, "width", minimum=1)
        scale = take_float(_obj(d, "embedding"), "scale")
        eps = take_float(_obj(d, "norm"), "eps")
        if eps <= 0:
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps}")
        streams = 0 if d.get("streams") is None else take_int(d, "streams", minimum=1)
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"config.json: layers[{i}]"
            if not isinstance(L, dict):
                raise ConfigError(f"{where} must be an object")
            if L.get("type") != "latent_attention":
                raise ConfigError(f"{where}: unknown layer type {L.get('type')!r} (latent_attention)")
            m = _obj(L, "mixer", where)
            mask = m.get("mask")
            window = None
            if mask is not None:
                if not isinstance(mask, dict):
                    raise ConfigError(f"{where}: 'mask' must be an object")
                window = take_int(mask, "size", minimum=1)
            src = m.get("kv_from")
            if src is not None:
                src = take_int(m, "kv_from", minimum=0)
            mixer = LatentMixerConfig(take_int(m, "heads", minimum=1), take_int(m, "dim", minimum=1),
                                      take_int(m, "vdim", minimum=1), take_int(m, "q_rank", minimum=1),
                                      take_int(m, "kv_rank", minimum=1), take_float(m, "scale"), window, src)
            if src is not None:
                if src >= i or layers[src].mixer.kv_from is not None:
                    raise ConfigError(f"{where}: kv_from {src} must name an earlier layer with a latent of its own")
                if layers[src].mixer.kv_rank != mixer.kv_rank:
                    raise ConfigError(f"{where}: kv_rank {mixer.kv_rank} differs from layer {src}'s "
                                      f"{layers[src].mixer.kv_rank}")
            ml, mlp = L.get("mlp"), None
            if ml is not None:
                if not isinstance(ml, dict):
                    raise ConfigError(f"{where}: 'mlp' must be an object or null")
                if ml.get("kind") == "dense":
                    mlp = NutizenMlpConfig("dense", take_int(ml, "ff", minimum=1))
                elif ml.get("kind") == "moe":
                    ex, r = _obj(ml, "expert", where), _obj(ml, "router", where)
                    sh = ml.get("shared")
                    if sh is not None and not isinstance(sh, dict):
                        raise ConfigError(f"{where}: 'shared' must be an object or null")
                    mlp = NutizenMlpConfig("moe", take_int(ex, "ff", minimum=1), _limit(ex, where),
                                           take_int(r, "experts", minimum=1), take_int(r, "top", minimum=1),
                                           take_int(sh, "ff", minimum=1) if sh else 0, _limit(sh, where) if sh else 0.0)
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"{where}: top {mlp.top} of {mlp.experts} experts")
                else:
                    raise ConfigError(f"{where}: unknown mlp kind {ml.get('kind')!r} (dense, moe)")
            layers.append(NutizenLayerConfig(mixer, mlp))
        return cls(architecture="Nutizen", vocab=vocab, width=width, embedding_scale=scale, norm_eps=eps,
                   streams=streams, layers=tuple(layers))

    def to_dict(self) -> dict:
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
             "layers": [L.to_dict() for L in self.layers]}
        if self.streams:
            d["streams"] = self.streams
        return d
