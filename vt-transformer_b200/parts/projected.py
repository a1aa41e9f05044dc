"""Mixers of the shape  projections of h -> a core on the projected values -> one output projection,  and the
mixer that runs several of them side by side.

Such a mixer says which matrices it multiplies its input with (``in_matrices``), how wide what its core leaves for
the output projection is (``inner_size``), and with which matrix that is projected (``out_matrix``).  Alone it runs
one product over its packed input matrices, its core, and the output product.  Side by side (``ParallelMixer``) the
branches share both products: one over all branches' input matrices, and one over their output matrices packed along
the inner dimension, so that sum_i scale_i * O_i core_i costs one product whose inputs the cores have scaled.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .base import Mixer, build_part, register_part

PACK = 8    # column ranges of packed products start at multiples of 8 (16 bytes of bfloat16)


def _round_up(n: int, to: int = PACK) -> int:
    return -(-n // to) * to


def pack_rows(mats: List[torch.Tensor]):
    """The matrices [n_i, k] one below the other, each padded with zero rows to a multiple of 8.  Returns the packed
    matrix and the first row of each."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.float() for m in mats]
    parts, starts, at = [], [], 0
    for m in mats:
        starts.append(at)
        parts.append(m)
        pad = _round_up(m.shape[0]) - m.shape[0]
        if pad:
            parts.append(torch.zeros((pad, m.shape[1]), dtype=m.dtype, device=m.device))
        at += m.shape[0] + pad
    return torch.cat(parts, dim=0).contiguous(), starts


def pack_columns(mats: List[torch.Tensor]):
    """The matrices [n, k_i] side by side, each padded with zero columns to a multiple of 8."""
    if len({m.dtype for m in mats}) > 1:
        mats = [m.float() for m in mats]
    parts, starts, at = [], [], 0
    for m in mats:
        starts.append(at)
        parts.append(m)
        pad = _round_up(m.shape[1]) - m.shape[1]
        if pad:
            parts.append(torch.zeros((m.shape[0], pad), dtype=m.dtype, device=m.device))
        at += m.shape[1] + pad
    return torch.cat(parts, dim=1).contiguous(), starts, at


class ProjectedMixer(Mixer):
    """``in_matrices()``: after ``load``, the matrices [n_i, hidden] of the projections the core reads, in the order
    in which ``core`` finds their results: result i starts at column ``cols[i]`` of ``y``.
    ``core(y, cols, ctx, cache, out, out_col, out_scale)``: y [T, N] holds the projections; the core writes
    out_scale * (what the output projection multiplies) into out[:, out_col : out_col + inner_size()].
    ``out_matrix()``: [hidden, inner_size()]."""

    graph_safe = True
    standalone = True       # False for a branch of a ``ParallelMixer``, which packs its branches' matrices itself

    def in_matrices(self) -> List[torch.Tensor]:
        raise NotImplementedError

    def inner_size(self) -> int:
        raise NotImplementedError

    def out_matrix(self) -> torch.Tensor:
        raise NotImplementedError

    def core(self, y, cols, ctx, cache, out, out_col: int, out_scale: float) -> None:
        raise NotImplementedError

    # ---- alone ---------------------------------------------------------------------------
    def pack(self) -> None:
        """Packs the matrices for a run of this mixer alone (a ``ParallelMixer`` packs its branches' itself)."""
        if not self.standalone:
            return
        self.w_in, self.cols = pack_rows(self.in_matrices())
        self.w_out, _, self.k_out = pack_columns([self.out_matrix()])
        self.release_unpacked()

    def release_unpacked(self) -> None:
        """Drops the single matrices once a packed copy exists."""

    def weight_bytes(self) -> int:
        return sum(m.numel() * m.element_size() for m in (self.w_in, self.w_out)) + self.extra_weight_bytes()

    def extra_weight_bytes(self) -> int:
        return 0

    def first_product(self):
        return self.rt.ops.product_hint(self.w_in, "linear")

    def forward(self, h, ctx, cache):
        ops = self.rt.ops
        T = h.shape[0]
        y = torch.empty((T, self.w_in.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_in, None, y)
        padded = self.k_out != self.inner_size()
        act = (torch.zeros if padded else torch.empty)((T, self.k_out), dtype=h.dtype, device=h.device)
        self.core(y, self.cols, ctx, cache, act, 0, 1.0)
        return ops.linear_to_stream(act, self.w_out, None, then=self.then)


@register_part("mixer", "parallel")
class ParallelMixer(Mixer):
    """sum_i scales[i] * branches[i](h): every branch a ``ProjectedMixer``.  One product over all branches' input
    matrices, the cores one after the other (each scaling what it leaves by its branch's scale, in 32-bit, before
    the one rounding), one product over the output matrices packed along the inner dimension.  What the branches
    keep between steps is handed on as a tuple, one entry for each branch that keeps something."""

    def __init__(self, spec, prefix, rt):
        super().__init__(spec, prefix, rt)
        if not (len(spec.branches) == len(spec.scales) == len(spec.prefixes)) or not spec.branches:
            raise ValueError("parallel mixer: one scale and one prefix for each branch")
        self.branches = [build_part("mixer", b, prefix + p, rt) for b, p in zip(spec.branches, spec.prefixes)]
        for b in self.branches:
            b.standalone = False
            if not isinstance(b, ProjectedMixer):
                raise ValueError(f"parallel mixer: branch '{b.spec.kind}' is no projected mixer (projections, core, "
                                 f"output projection); only those can share the two products")

    @property
    def graph_safe(self):
        return all(b.graph_safe for b in self.branches)

    def cache_spec(self):
        specs = [b.cache_spec() for b in self.branches]
        kept = tuple(s for s in specs if s is not None)
        return kept if kept else None

    def param_specs(self):
        out = {}
        for b in self.branches:
            out.update(b.param_specs())
        return out

    def load(self, get) -> None:
        mats, counts = [], []
        for b in self.branches:
            b.load(get)
            m = b.in_matrices()
            mats += m
            counts.append(len(m))
        self.w_in, cols = pack_rows(mats)
        self.cols, at = [], 0
        for n in counts:
            self.cols.append(cols[at:at + n])
            at += n
        self.w_out, self.out_cols, self.k_out = pack_columns([b.out_matrix() for b in self.branches])
        self.padded = self.k_out != sum(b.inner_size() for b in self.branches)
        for b in self.branches:
            b.release_unpacked()

    def weight_bytes(self) -> int:
        return (sum(m.numel() * m.element_size() for m in (self.w_in, self.w_out))
                + sum(b.extra_weight_bytes() for b in self.branches))

    def first_product(self):
        return self.rt.ops.product_hint(self.w_in, "linear")

    def forward(self, h, ctx, cache):
        ops = self.rt.ops
        T = h.shape[0]
        y = torch.empty((T, self.w_in.shape[0]), dtype=h.dtype, device=h.device)
        ops.linear(h, self.w_in, None, y)
        act = (torch.zeros if self.padded else torch.empty)((T, self.k_out), dtype=h.dtype, device=h.device)
        views = list(cache) if isinstance(cache, (tuple, list)) else ([cache] if cache is not None else [])
        for b, cols, col, scale in zip(self.branches, self.cols, self.out_cols, self.spec.scales):
            view = views.pop(0) if b.cache_spec() is not None else None
            b.core(y, cols, ctx, view, act, col, float(scale))
        return ops.linear_to_stream(act, self.w_out, None, then=self.then)
