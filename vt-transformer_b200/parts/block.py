"""The arrangement of parts in a layer."""
from __future__ import annotations

from .base import Block, build_part, register_part


@register_part("block", "prenorm")
class PreNormBlock(Block):
    """x += mixer(norm1(x)); x += ffn(norm2(x))
    (the order of v1/models/qwen2-7b/inference_fp16.dag:287-345).  The two sums are formed
    in 32-bit inside the next norm (``ResidualStream``)."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        self.norm1 = build_part("norm", spec.norm1, prefix + spec.norm1_name, rt)
        self.mixer = build_part("mixer", spec.mixer, prefix + spec.mixer_prefix, rt)
        self.norm2 = self.ffn = None
        if spec.ffn is not None:            # a layer without a feed-forward has the first sublayer only
            self.norm2 = build_part("norm", spec.norm2, prefix + spec.norm2_name, rt)
            self.ffn = build_part("feed_forward", spec.ffn, prefix + spec.ffn_prefix, rt)
        self.parts = tuple(p for p in (self.norm1, self.mixer, self.norm2, self.ffn) if p is not None)

    def cache_spec(self):
        return self.mixer.cache_spec()

    @property
    def graph_safe(self):
        return all(p.graph_safe for p in self.parts)

    def param_specs(self):
        out = {}
        for p in self.parts:
            out.update(p.param_specs())
        return out

    def load(self, get) -> None:
        for p in self.parts:
            p.load(get)

    def weight_bytes(self) -> int:
        return sum(p.weight_bytes() for p in self.parts)

    def first_product(self):
        return self.mixer.first_product()

    def link(self, then) -> None:
        if self.ffn is None:
            self.mixer.then = then
            return
        self.mixer.then = self.ffn.first_product()
        self.ffn.then = then

    def forward(self, stream, ctx, cache):
        h = stream.normed(self.norm1)
        stream.add(self.mixer.forward(h, ctx, cache))
        if self.ffn is None:
            return
        h = stream.normed(self.norm2)
        stream.add(self.ffn.forward(h, ctx))


@register_part("block", "sandwich")
class SandwichBlock(PreNormBlock):
    """x += m * post1(mixer(norm1(x))); x += m * post2(ffn(norm2(x))): every sublayer's result is normed (root mean
    square, weight) and multiplied by m before the residual sum.  The norm that reads the stream next does all of it
    in one pass: it norms and scales the pending result in 32-bit, adds it, and norms the sum."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if spec.post1 is None or (spec.ffn is not None and spec.post2 is None):
            raise ValueError("sandwich block: a norm for each sublayer's result (post1, post2)")
        for n in (spec.post1, spec.post2):
            if n is not None and n.kind != "rmsnorm":
                raise ValueError(f"sandwich block: the norm of a sublayer's result is a root-mean-square norm, not '{n.kind}'")
        self.post1 = build_part("norm", spec.post1, prefix + spec.post1_name, rt)
        self.post2 = build_part("norm", spec.post2, prefix + spec.post2_name, rt) if spec.ffn is not None else None
        self.parts = self.parts + tuple(p for p in (self.post1, self.post2) if p is not None)

    def forward(self, stream, ctx, cache):
        s = self.spec
        h = stream.normed(self.norm1)
        stream.add(self.mixer.forward(h, ctx, cache), post=(self.post1.weighted(), s.post1.eps, s.residual_mult))
        if self.ffn is None:
            return
        h = stream.normed(self.norm2)
        stream.add(self.ffn.forward(h, ctx), post=(self.post2.weighted(), s.post2.eps, s.residual_mult))
