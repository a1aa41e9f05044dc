"""Sisetar as a ``ModelSpec``: a decoder whose layers mix tokens either by gated linear attention or by softmax
attention on chunks beside a delta-rule recurrence, with layer norms, a PolyNorm feed-forward on some layers, a
scaled embedding and a tied, scaled and soft-capped output.

Tensor names: ``embed``, ``final.norm``, and for layer i ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*`` (under
``.left`` and ``.right`` for the two branches of a parallel mixer) and ``l<i>.mlp.*``."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.sisetar import SisetarConfig
from ..parts.specs import (AttentionSpec, BlockSpec, DeltaRuleSpec, EmbeddingSpec, GatedLinearAttentionSpec, HeadSpec,
                           ModelSpec, NormSpec, ParallelSpec, PolyNormMLPSpec, PositionSpec, RunSpec)


def sisetar_model_spec(cfg: SisetarConfig) -> ModelSpec:
    norm = NormSpec(size=cfg.width, eps=cfg.norm_eps, kind="layernorm", weight_suffix="")
    blocks, order, slot = [], [], 0
    for i, layer in enumerate(cfg.layers):
        m = layer.mixer
        if layer.type == "gla":
            mixer = GatedLinearAttentionSpec(hidden=cfg.width, heads=m.heads, dim=m.dim, v_dim=m.vdim, tau=m.tau,
                                             norm_eps=cfg.norm_eps)
            caches = 1
        else:
            a, d = m.left, m.right
            left = AttentionSpec(hidden=cfg.width, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, v_dim=a.vdim,
                                 qkv_bias=False, out_bias=False, scale=a.scale, chunk=a.chunk, qk_norm_eps=cfg.norm_eps,
                                 position=PositionSpec(kind="rotary_computed", dim=a.rot_dims, base=a.rot_base),
                                 names=("q", "k", "v", "o"), weight_suffix="")
            right = DeltaRuleSpec(hidden=cfg.width, heads=d.heads, dim=d.dim, norm_eps=cfg.norm_eps)
            mixer = ParallelSpec(branches=(left, right), scales=(m.left_scale, m.right_scale), prefixes=("left.", "right."))
            caches = 2
        ffn = None if layer.ff is None else PolyNormMLPSpec(hidden=cfg.width, inter=layer.ff, eps=cfg.norm_eps)
        blocks.append(BlockSpec(mixer=mixer, ffn=ffn, norm1=norm, norm2=None if ffn is None else norm, prefix=f"l{i}.",
                                mixer_prefix="mix.", ffn_prefix="mlp.", norm1_name="norm1", norm2_name="norm2"))
        # a run names one cache slot for everything its mixer keeps: pages of keys and values, a recurrent state
        order.append(RunSpec(block=i, cache=slot if caches == 1 else tuple(range(slot, slot + caches))))
        slot += caches
    embedding = EmbeddingSpec(vocab=cfg.vocab, hidden=cfg.width, name="embed", scale=cfg.embedding_scale)
    head = HeadSpec(vocab=cfg.vocab, hidden=cfg.width, norm=norm, norm_name="final.norm", name="head", tied_to="embed",
                    logit_scale=cfg.logit_scale, logit_cap=cfg.logit_softcap)
    return ModelSpec(vocab=cfg.vocab, hidden=cfg.width, blocks=tuple(blocks), order=tuple(order), embedding=embedding,
                     head=head, max_positions=0)


register_architecture("Sisetar", SisetarConfig, sisetar_model_spec, replace=True)
