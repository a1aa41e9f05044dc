"""Configuration of the Vegilix decoder ("Vegilix").

Its config.json is nested: ``layers`` lists the layers one by one, each with the ``type`` of its mixer
("attention": differential softmax attention under a sliding window that keeps the first tokens;
"retention": linear attention with a fixed decay for each head), the mixer's sizes and constants under ``mixer``,
and its feed-forward under ``mlp`` (a mixture of experts with a shared expert, or null).  ``loop`` names a span of
layers that runs several times in a row with the same weights.  Every size and every constant that can differ
between two models of the design is read from there.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, KeyReader, ModelConfig, architecture_name


@dataclass(frozen=True)
class RotationScaling:
    """Frequencies whose wavelength is above original/low are divided by ``factor``, those below original/high are
    kept, and those between are blended."""
    factor: float
    low: float
    high: float
    original: float


@dataclass(frozen=True)
class VegilixRotation:
    dims: int
    base: float
    scaling: Optional[RotationScaling] = None


@dataclass(frozen=True)
class VegilixAttention:
    """Differential attention: ``heads`` query heads over ``kv_heads`` key/value heads; every head has two maps of
    queries and keys of ``dim`` over one set of values of ``vdim``.  Position i sees j <= i with i - j < ``window`` (None:
    all) or j < ``keep_first``."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    rot: VegilixRotation
    scale: float
    diff: float
    window: Optional[int]
    keep_first: int


@dataclass(frozen=True)
class VegilixRetention:
    """Retention: ``heads`` heads with keys of ``dim`` and values of ``vdim``; head h's state decays by ``decay[h]`` a token."""
    heads: int
    dim: int
    vdim: int
    rot: VegilixRotation
    decay: Tuple[float, ...]


@dataclass(frozen=True)
class VegilixExperts:
    """``experts`` gated feed-forwards of inner size ``ff`` of which a token uses ``top``; ``shared_ff``: the inner size of
    the expert that every token uses (None: there is none)."""
    experts: int
    top: int
    ff: int
    shared_ff: Optional[int]


@dataclass(frozen=True)
class VegilixLayer:
    type: str                           # "attention" or "retention"
    mixer: Any                          # VegilixAttention or VegilixRetention
    mlp: Optional[VegilixExperts]


@dataclass(frozen=True)
class VegilixConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[VegilixLayer, ...]
    norm_eps: float
    residual_mult: float
    loop_start: int
    loop_stop: int
    loop_times: int                     # 1: no span is repeated

    def run_order(self) -> Tuple[int, ...]:
        """The layers in the order in which a token passes them."""
        n = len(self.layers)
        return (tuple(range(self.loop_start)) + tuple(range(self.loop_start, self.loop_stop)) * self.loop_times
                + tuple(range(self.loop_stop, n)))

    # ---- reading -------------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any], where: str = "config.json") -> "VegilixConfig":
        r = KeyReader(data, where)
        arch = architecture_name(data, where)
        layers_raw = r.raw("layers")
        if not isinstance(layers_raw, list) or not layers_raw:
            raise ConfigError(f"{where}: key 'layers' must be a list with one entry for each layer")
        layers = tuple(_layer(entry, f"{where}: layers[{i}]") for i, entry in enumerate(layers_raw))
        norm = KeyReader(_obj(r.raw("norm"), f"{where}: norm"), f"{where}: norm")
        loop_raw = r.raw("loop", default=None)
        start, stop, times = 0, 0, 1
        if loop_raw is not None:
            lp = KeyReader(_obj(loop_raw, f"{where}: loop"), f"{where}: loop")
            start, stop = lp.integer("start", minimum=0), lp.integer("stop", minimum=0)
            times = lp.integer("times", default=1, minimum=1)
        cfg = cls(architecture=arch, vocab=r.integer("vocab", minimum=1), width=r.integer("width", minimum=1), layers=layers,
                  norm_eps=norm.number("eps", positive=True), residual_mult=r.number("residual_mult", default=1.0),
                  loop_start=start, loop_stop=stop, loop_times=times)
        cfg.validate(where)
        return cfg

    def validate(self, where: str = "config.json") -> None:
        if self.width % 8:
            raise ConfigError(f"{where}: 'width' {self.width} is not supported: the matrix kernels read rows in "
                              f"16-byte pieces, so it must be a multiple of 8")
        if not 0 <= self.loop_start <= self.loop_stop <= len(self.layers):
            raise ConfigError(f"{where}: loop: 'start' {self.loop_start} and 'stop' {self.loop_stop} must lie within the "
                              f"{len(self.layers)} layers, start <= stop")
        for i, layer in enumerate(self.layers):
            at = f"{where}: layers[{i}]"
            m = layer.mixer
            if m.rot.dims % 2 or m.rot.dims > m.dim:
                raise ConfigError(f"{at}: 'rot.dims' {m.rot.dims} must be even and at most 'dim' {m.dim}")
            if layer.type == "attention":
                if m.heads % m.kv_heads:
                    raise ConfigError(f"{at}: 'heads' {m.heads} is not a multiple of 'kv_heads' {m.kv_heads}")
                if m.dim > 256 or m.vdim > 256:
                    raise ConfigError(f"{at}: 'dim' and 'vdim' above 256 are not supported by the attention kernel")
            else:
                if len(m.decay) != m.heads:
                    raise ConfigError(f"{at}: 'decay' lists {len(m.decay)} numbers for {m.heads} heads")
                if m.dim > 1024:
                    raise ConfigError(f"{at}: 'dim' above 1024 is not supported by the scan kernel")
            if layer.mlp is not None and not 1 <= layer.mlp.top <= layer.mlp.experts:
                raise ConfigError(f"{at}: router 'top' {layer.mlp.top} must lie between 1 and 'experts' {layer.mlp.experts}")
            if layer.mlp is not None and layer.mlp.experts > 1024:
                raise ConfigError(f"{at}: more than 1024 experts are not supported by the routing kernel")

    def to_dict(self) -> Dict[str, Any]:
        def rot(r: VegilixRotation):
            out = {"dims": r.dims, "base": r.base}
            if r.scaling is not None:
                s = r.scaling
                out["scaling"] = {"factor": s.factor, "low": s.low, "high": s.high, "original": s.original}
            return out

        layers = []
        for layer in self.layers:
            m = layer.mixer
            if layer.type == "attention":
                mask = {"keep_first": m.keep_first}
                if m.window is not None:
                    mask["size"] = m.window
                mixer = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "rot": rot(m.rot),
                         "scale": m.scale, "diff": m.diff, "mask": mask}
            else:
                mixer = {"heads": m.heads, "dim": m.dim, "vdim": m.vdim, "rot": rot(m.rot), "decay": list(m.decay)}
            mlp = None
            if layer.mlp is not None:
                f = layer.mlp
                mlp = {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.ff},
                       "shared": None if f.shared_ff is None else {"ff": f.shared_ff}}
            layers.append({"type": layer.type, "mixer": mixer, "mlp": mlp})
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "layers": layers,
               "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult}
        if self.loop_times > 1 or self.loop_stop > self.loop_start:
            out["loop"] = {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}
        return out


def _obj(v, where: str) -> Dict[str, Any]:
    if not isinstance(v, dict):
        raise ConfigError(f"{where}: expected an object")
    return v


def _rotation(raw, where: str) -> VegilixRotation:
    if raw is None:
        return VegilixRotation(dims=0, base=10000.0)
    r = KeyReader(_obj(raw, where), where)
    scaling = None
    sc = r.raw("scaling", default=None)
    if sc is not None:
        s = KeyReader(_obj(sc, where + ".scaling"), where + ".scaling")
        scaling = RotationScaling(factor=s.number("factor", positive=True), low=s.number("low"), high=s.number("high"),
                                  original=s.number("original", positive=True))
        if scaling.high == scaling.low:
            raise ConfigError(f"{where}.scaling: 'high' and 'low' must differ")
    return VegilixRotation(dims=r.integer("dims", minimum=0), base=r.number("base", positive=True), scaling=scaling)


def _layer(entry, where: str) -> VegilixLayer:
    r = KeyReader(_obj(entry, where), where)
    kind = r.string("type")
    mw = f"{where}.mixer"
    m = KeyReader(_obj(r.raw("mixer"), mw), mw)
    if kind == "attention":
        heads = m.integer("heads", minimum=1)
        window, keep = None, 0
        mask_raw = m.raw("mask", default=None)
        if mask_raw is not None:
            mask = KeyReader(_obj(mask_raw, mw + ".mask"), mw + ".mask")
            window = mask.integer("size", default=None, minimum=1)
            keep = mask.integer("keep_first", default=0, minimum=0)
        dim = m.integer("dim", minimum=1)
        mixer = VegilixAttention(heads=heads, kv_heads=m.integer("kv_heads", default=heads, minimum=1), dim=dim,
                                 vdim=m.integer("vdim", default=dim, minimum=1), rot=_rotation(m.raw("rot", default=None), mw + ".rot"),
                                 scale=m.number("scale", default=dim ** -0.5), diff=m.number("diff"), window=window, keep_first=keep)
    elif kind == "retention":
        decay = m.raw("decay")
        if not isinstance(decay, list) or not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
            raise ConfigError(f"{mw}: key 'decay' must be a list of numbers, one for each head")
        dim = m.integer("dim", minimum=1)
        mixer = VegilixRetention(heads=m.integer("heads", minimum=1), dim=dim, vdim=m.integer("vdim", default=dim, minimum=1),
                                 rot=_rotation(m.raw("rot", default=None), mw + ".rot"), decay=tuple(float(d) for d in decay))
    else:
        raise ConfigError(f"{where}: layer type '{kind}' is not known; known are 'attention' and 'retention'")
    mlp_raw = r.raw("mlp", default=None)
    mlp = None
    if mlp_raw is not None:
        fw = f"{where}.mlp"
        f = KeyReader(_obj(mlp_raw, fw), fw)
        if f.string("kind", default="moe") != "moe":
            raise ConfigError(f"{fw}: feed-forward kind '{mlp_raw.get('kind')}' is not known; known is 'moe'")
        router = KeyReader(_obj(f.raw("router"), fw + ".router"), fw + ".router")
        exp = KeyReader(_obj(f.raw("expert"), fw + ".expert"), fw + ".expert")
        shared_raw = f.raw("shared", default=None)
        shared_ff = None
        if shared_raw is not None:
            shared_ff = KeyReader(_obj(shared_raw, fw + ".shared"), fw + ".shared").integer("ff", minimum=1)
        mlp = VegilixExperts(experts=router.integer("experts", minimum=1), top=router.integer("top", minimum=1),
                             ff=exp.integer("ff", minimum=1), shared_ff=shared_ff)
    return VegilixLayer(type=kind, mixer=mixer, mlp=mlp)
