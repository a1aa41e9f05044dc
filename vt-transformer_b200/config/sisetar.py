"""Configuration of the Sisetar decoder ("Sisetar").

Its config.json is nested: ``layers`` lists the layers one by one, each with the ``type`` of its mixer
("gla": gated linear attention; "parallel": softmax attention on chunks beside a delta-rule recurrence), the
mixer's sizes and constants under ``mixer``, and its feed-forward under ``mlp`` (null: the layer has none).
Every size and every constant that can differ between two models of the design is read from there; nothing
is taken from a tensor's shape except the rank of the two low-rank gates, which the file does not name.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig, architecture_name


@dataclass(frozen=True)
class SisetarGLA:
    """Gated linear attention: ``heads`` heads with keys of ``dim`` and values of ``vdim``; the decay is
    sigmoid(.)^(1 / tau)."""
    heads: int
    dim: int
    vdim: int
    tau: float


@dataclass(frozen=True)
class SisetarAttention:
    """Softmax attention: ``heads`` query heads over ``kv_heads`` key/value heads, keys of ``dim``, values of
    ``vdim``; the first ``rot_dims`` dimensions of a head are rotated with base ``rot_base``; position i sees
    j <= i with i // chunk == j // chunk."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    rot_dims: int
    rot_base: float
    scale: float
    chunk: int


@dataclass(frozen=True)
class SisetarDelta:
    """Generalized delta rule: ``heads`` heads with keys and values of ``dim``."""
    heads: int
    dim: int


@dataclass(frozen=True)
class SisetarParallel:
    left: SisetarAttention
    right: SisetarDelta
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class SisetarLayer:
    type: str                           # "gla" or "parallel"
    mixer: Any                          # SisetarGLA or SisetarParallel
    ff: Optional[int]                   # inner size of the dense feed-forward; None: no feed-forward


@dataclass(frozen=True)
class SisetarConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[SisetarLayer, ...]
    embedding_scale: float
    logit_scale: float
    logit_softcap: float                # 0: none
    norm_eps: float

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "SisetarConfig":
        r = KeyReader(data, where)
        arch = architecture_name(data, where)
        layers_raw = r.raw("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a list with one entry for each layer")
        layers = tuple(_layer(entry, f"{where}: layers[{i}]") for i, entry in enumerate(layers_raw))
        emb = KeyReader(_obj(r.raw("embedding", default={}), f"{where}: embedding"), f"{where}: embedding")
        norm = KeyReader(_obj(r.raw("norm"), f"{where}: norm"), f"{where}: norm")
        cfg = cls(architecture=arch, vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1),
                  layers=layers, embedding_scale=emb.number("scale", default=1.0),
                  logit_scale=r.number("logit_scale", default=1.0),
                  logit_softcap=r.number("logit_softcap", default=0.0) or 0.0,
                  norm_eps=norm.number("eps", positive=True))
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.width % 8:
            raise ConfigError(f"{where}: 'width' {self.width} is not supported: the matrix kernels read rows in "
                              f"16-byte pieces, so it must be a multiple of 8")
        if self.logit_softcap < 0:
            raise ConfigError(f"{where}: 'logit_softcap' must not be negative")
        for i, layer in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            att = layer.mixer.left if layer.type == "parallel" else None
            if att is not None:
                if att.heads % att.kv_heads:
                    raise ConfigError(f"{at}: left 'heads' {att.heads} is not a multiple of 'kv_heads' {att.kv_heads}")
                if att.rot_dims % 2 or att.rot_dims > att.dim:
                    raise ConfigError(f"{at}: left 'rot.dims' {att.rot_dims} must be even and at most 'dim' {att.dim}")
                if att.dim > 256 or att.vdim > 256:
                    raise ConfigError(f"{at}: left 'dim' and 'vdim' above 256 are not supported by the attention kernel")

    def to_dict(self) -> Dict[str, Any]:
        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "gla":
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "tau": m.tau}
            else:
                a, d = m.left, m.right
                mixer = {"left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim,
                                  "rot": {"dims": a.rot_dims, "base": a.rot_base}, "scale": a.scale,
                                  "mask": {"size": a.chunk}},
                         "right": {"heads": d.heads, "dim": d.dim},
                         "left_scale": m.left_scale, "right_scale": m.right_scale}
            layers.append({"type": layer.type, "mixer": mixer,
                           "mlp": None if layer.ff is None else {"kind": "dense", "ff": layer.ff}})
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": layers,
                "embedding": {"scale": self.embedding_scale}, "logit_scale": self.logit_scale,
                "logit_softcap": self.logit_softcap, "norm": {"eps": self.norm_eps}}


def _obj(v, where: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: expected an object")
    return v


def _layer(entry, where: str) -> SisetarLayer:
    r = KeyReader(_obj(entry, where), where)
    kind = r.string("type")
    m = KeyReader(_obj(r.raw("mixer"), f"{where}.mixer"), f"{where}.mixer")
    if kind == "gla":
        mixer = SisetarGLA(heads=m.integer("heads", minimum=1), dim=m.integer("dim", minimum=1),
                           vdim=m.integer("vdim", minimum=1), tau=m.number("tau", positive=True))
    elif kind == "parallel":
        lw, rw = f"{where}.mixer.left", f"{where}.mixer.right"
        left = KeyReader(_obj(m.raw("left"), lw), lw)
        right = KeyReader(_obj(m.raw("right"), rw), rw)
        rot = KeyReader(_obj(left.raw("rot"), lw + ".rot"), lw + ".rot")
        mask = KeyReader(_obj(left.raw("mask"), lw + ".mask"), lw + ".mask")
        heads = left.integer("heads", minimum=1)
        att = SisetarAttention(heads=heads, kv_heads=left.integer("kv_heads", default=heads, minimum=1),
                               dim=left.integer("dim", minimum=1), vdim=left.integer("vdim", minimum=1),
                               rot_dims=rot.integer("dims", minimum=0), rot_base=rot.number("base", positive=True),
                               scale=left.number("scale"), chunk=mask.integer("size", minimum=1))
        delta = SisetarDelta(heads=right.integer("heads", minimum=1), dim=right.integer("dim", minimum=1))
        mixer = SisetarParallel(left=att, right=delta, left_scale=m.number("left_scale", default=1.0),
                                right_scale=m.number("right_scale", default=1.0))
    else:
        raise ConfigError(f"{where}: layer type '{kind}' is not known; known are 'gla' and 'parallel'")
    mlp = r.raw("mlp", default=None)
    ff = None
    if mlp is not None:
        f = KeyReader(_obj(mlp, f"{where}.mlp"), f"{where}.mlp")
        if f.string("kind", default="dense") != "dense":
            raise ConfigError(f"{where}.mlp: feed-forward kind '{mlp.get('kind')}' is not known; known is 'dense'")
        ff = f.integer("ff", minimum=1)
    return SisetarLayer(type=kind, mixer=mixer, ff=ff)
