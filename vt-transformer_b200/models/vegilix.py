"""Vegilix as a ``ModelSpec``: a decoder whose layers mix tokens either by differential softmax attention (two maps a
head over one set of values, under a sliding window that keeps the first tokens) or by retention (linear attention
with a fixed decay for each head), with a norm before and after each sublayer, a scaled residual sum, a mixture of
experts with a shared expert as the feed-forward, and a span of layers that may run several times with the same
weights, each pass with a cache or state of its own.

Tensor names: ``embed``, ``final.norm``, ``head``, and for layer i ``l<i>.norm1``, ``l<i>.norm1b``, ``l<i>.norm2``,
``l<i>.norm2b``, ``l<i>.mix.*`` and ``l<i>.mlp.*``."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.vegilix import VegilixConfig
from ..parts.specs import (BlockSpec, DifferentialAttentionSpec, EmbeddingSpec, ExpertsSpec, HeadSpec, ModelSpec, NormSpec,
                           PositionSpec, RetentionSpec, RunSpec)


def _position(rot) -> PositionSpec:
    if not rot.dims:
        return PositionSpec(kind="none")
    sc = rot.scaling
    return PositionSpec(kind="rotary_computed", dim=rot.dims, base=rot.base,
                        scaling=None if sc is None else (sc.factor, sc.low, sc.high, sc.original))


def vegilix_model_spec(cfg: VegilixConfig) -> ModelSpec:
    norm = NormSpec(size=cfg.width, eps=cfg.norm_eps, kind="rmsnorm", weight_suffix="", one_plus=True)
    blocks = []
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "attention":
            mixer = DifferentialAttentionSpec(hidden=cfg.width, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim, v_dim=m.vdim,
                                              scale=m.scale, diff=m.diff, window=m.window, keep_first=m.keep_first,
                                              norm_eps=cfg.norm_eps, position=_position(m.rot))
        else:
            mixer = RetentionSpec(hidden=cfg.width, heads=m.heads, dim=m.dim, v_dim=m.vdim, decay=m.decay, norm_eps=cfg.norm_eps,
                                  position=_position(m.rot))
        f = layer.mlp
        ffn = None if f is None else ExpertsSpec(hidden=cfg.width, experts=f.experts, top=f.top, inter=f.ff, shared_inter=f.shared_ff)
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=None if ffn is None else norm, prefix=f"l{i}.",
                                mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1", norm2_name="norm2", kind="sandwich",
                                post1=norm, post2=None if ffn is None else norm, post1_name="norm1b", post2_name="norm2b",
                                residual_mult=cfg.residual_mult))
    # every run of a layer has a cache slot of its own: a layer of a repeated span keeps keys or a state for each pass
    order = tuple(RunSpec(block=b, cache=slot) for slot, b in enumerate(cfg.run_order()))
    embedding = EmbeddingSpec(vocab=cfg.vocab, hidden=cfg.width, name="embed")
    head = HeadSpec(vocab=cfg.vocab, hidden=cfg.width, norm=norm, norm_name="final.norm", name="head")
    return ModelSpec(vocab=cfg.vocab, hidden=cfg.width, blocks=tuple(blocks), order=order, embedding=embedding, head=head,
                     max_positions=0)


register_architecture("Vegilix", VegilixConfig, vegilix_model_spec, replace=True)
