"""Configurations, weights and scenarios of the Vegilix tests.  Every scenario runs the engine (``ModelRunner.step`` or
``LLM.generate``) and compares with the plain implementation (tests/plain/vegilix_plain.py); each takes the device and
dtype, so the host-side tests run it on the CPU with the stand-in kernels and the GPU tests on cuda:0 with the real ones."""
from __future__ import annotations

import copy
import json
import os
import random
from typing import Callable, Dict, List

import numpy as np
import torch

import helpers
from plain import vegilix_plain as plain
from sisetar_cases import rewritten, runner_for, step_all  # noqa: F401  (the same helpers serve both designs)


def _att(heads, kv_heads, dim, vdim, rot, base, scale, diff, size, keep, scaling=None, mlp=None):
    r = {"dims": rot, "base": base}
    if scaling:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mask = {"keep_first": keep}
    if size is not None:
        mask["size"] = size
    return {"type": "attention", "mixer": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": r, "scale": scale,
                                           "diff": diff, "mask": mask}, "mlp": mlp}


def _ret(heads, dim, vdim, rot, base, decay, mlp=None):
    return {"type": "retention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base},
                                           "decay": decay}, "mlp": mlp}


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": None if shared is None else {"ff": shared}}


def _model(vocab, width, layers, loop=None, mult=1.0, eps=1e-5):
    out = {"architecture": "Vegilix", "vocab": vocab, "width": width, "layers": layers, "norm": {"eps": eps}, "residual_mult": mult}
    if loop:
        out["loop"] = dict(zip(("start", "stop", "times"), loop))
    return out


# Configurations that differ from one another in every size and constant: grouped and ungrouped query heads, one head,
# values wider and narrower than keys and as wide, a rotation of the whole head, of a part and of nothing, with and
# without scaled frequencies (wavelengths on all three sides of the scaling's bounds), windows below and above a page,
# with and without kept first tokens and without a window, experts whose inner size is no multiple of 8, top of 1 and of
# all experts, with and without the shared expert, layers without a feed-forward, a repeated span in the middle, at the
# start, over all layers and none, decays of exactly 1 and far below, residual multipliers of 1 and others.
CONFIGS: Dict[str, dict] = {
    "mix": _model(300, 64, [_ret(3, 24, 40, 24, 500.0, [0.9, 0.97, 1.0], mlp=_moe(5, 2, 20, 36)),
                            _att(4, 2, 24, 40, 12, 3000.0, 0.21, 0.25, 21, 3, scaling=(4.0, 1.0, 3.0, 64), mlp=_moe(6, 3, 24, None)),
                            _att(2, 2, 40, 16, 40, 100.0, 0.15, 0.4, 9, 0),
                            _ret(1, 16, 16, 8, 10000.0, [0.875], mlp=_moe(3, 1, 50, 16))],
                  loop=(1, 3, 2), mult=0.6),
    "wide": _model(257, 72, [_att(6, 1, 72, 136, 0, 10000.0, 0.1, 0.1, None, 0, mlp=_moe(4, 4, 40, 24)),
                             _ret(2, 136, 72, 64, 50.0, [0.99, 0.5]), _att(1, 1, 16, 8, 16, 7.0, 0.3, 0.5, 70, 17, mlp=_moe(2, 1, 64, 8))],
                   loop=(0, 3, 3), mult=1.0, eps=1e-6),
    "attention_alone": _model(128, 48, [_att(4, 2, 16, 24, 8, 777.0, 0.25, 0.2, 11, 2, scaling=(8.0, 1.0, 4.0, 32))], mult=0.8),
    "retention_alone": _model(128, 48, [_ret(3, 20, 28, 10, 300.0, [0.8, 0.95, 0.99])], mult=1.3),
    "experts_alone": _model(128, 48, [_ret(1, 8, 8, 0, 10.0, [0.5], mlp=_moe(7, 3, 28, 12))], mult=0.9),
    # sizes that the tensor-core kernel of the differential attention takes (bfloat16): windows of several blocks of
    # 64 keys and below one, kept first tokens within a block and over more than one, grouped heads
    "tensor": _model(200, 64, [_att(4, 2, 32, 64, 16, 1e4, 0.18, 0.3, 150, 5, scaling=(8.0, 1.0, 4.0, 128), mlp=_moe(3, 3, 24, 16)),
                               _att(2, 1, 64, 128, 64, 500.0, 0.125, 0.2, 40, 70), _ret(2, 16, 16, 16, 1e4, [0.9, 0.95]),
                               _att(2, 2, 64, 64, 32, 1e5, 0.125, 0.35, None, 0)], loop=(0, 2, 2), mult=0.8),
    "tensor_wide": _model(160, 64, [_att(3, 1, 128, 256, 64, 1e4, 0.09, 0.3, 50, 2, mlp=_moe(2, 2, 16, None)),
                                    _att(2, 2, 128, 128, 128, 300.0, 0.09, 0.15, None, 0)], mult=0.8),
    "tensor_alone": _model(128, 64, [_att(4, 2, 32, 64, 16, 1e4, 0.18, 0.3, 100, 3)], mult=0.9),
    "looped_start": _model(128, 48, [_att(2, 1, 16, 16, 16, 1e4, 0.25, 0.3, 18, 1, mlp=_moe(3, 2, 16, 16)),
                                     _ret(2, 16, 24, 16, 1e4, [0.9, 0.99], mlp=_moe(3, 2, 16, 16))], loop=(0, 1, 3), mult=0.7),
}
SIGMA = {"tensor": 0.15, "tensor_wide": 0.12, "tensor_alone": 0.25, "mix": 0.15, "wide": 0.12, "attention_alone": 0.25, "retention_alone": 0.2, "experts_alone": 0.2, "looped_start": 0.2}
SEED = {n: 300 + i for i, n in enumerate(CONFIGS)}
LENGTHS = {"tensor": [1, 70, 150, 330, 260], "tensor_wide": [2, 90, 200], "tensor_alone": [3, 130, 270], "mix": [1, 9, 40, 71, 130], "wide": [3, 33, 90, 152], "attention_alone": [2, 30, 77], "retention_alone": [1, 25, 66],
           "experts_alone": [4, 19, 50], "looped_start": [5, 48, 97]}


def every_expert(name: str) -> str:
    """The name of the configuration ``name`` with every router's ``top`` set to its number of experts."""
    return name + "+all"


def for_dtype(name: str, dtype: str) -> str:
    """The configuration that a test of the whole model runs in ``dtype``.  In bfloat16 the rounding of the activations
    decides a router's close call (two logits a few percent apart) the other way now and then; the token then runs other
    experts, and through keys, values and states every later position of a deep model moves by more than rounding
    explains.  So the deep models run in bfloat16 with every expert chosen (the weights still come from the router's
    softmax), and the choice among experts is tested in 32-bit on the same kernels and in bfloat16 on the model of one
    layer, where a close call touches its own position only and is left out."""
    return name if dtype == "float32" else every_expert(name)


def config_of(name: str) -> dict:
    base = name[:-len("+all")] if name.endswith("+all") else name
    cfg = copy.deepcopy(CONFIGS[base])
    if name.endswith("+all"):
        for layer in cfg["layers"]:
            if layer["mlp"] is not None:
                layer["mlp"]["router"]["top"] = layer["mlp"]["router"]["experts"]
    return cfg


def make_folder(name: str, folder: str) -> str:
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    base = name[:-len("+all")] if name.endswith("+all") else name
    return write_random_model(config_from_dict(config_of(name)), folder, seed=SEED[base], sigma=SIGMA[base])


def prompts_for(name: str, seed: int = 0, lengths=None) -> List[List[int]]:
    name = name[:-len("+all")] if name.endswith("+all") else name
    rng = random.Random(900 + seed)
    vocab = CONFIGS[name]["vocab"]
    return [[rng.randrange(vocab) for _ in range(n)] for n in (lengths or LENGTHS[name])]


def tol(dtype: str, ref: torch.Tensor, alone: bool = False) -> float:
    """The bound on |logit - plain logit|, as a part of the spread of the model's plain logits.  32-bit differs by
    rounding and the order of sums only (measured on a B200: up to 1.5e-5 of the spread; the bound is 5e-5).  bfloat16
    rounds the activations to 8 bits at every part: models of one layer (``alone``) measured up to 0.035 of the spread
    (bound 0.1), the deep ones up to 0.25 (bound 0.35)."""
    spread = max(1.0, float(ref.double().std()))
    return (5e-5 if dtype == "float32" else (0.1 if alone else 0.35)) * spread


def outliers_allowed(dtype: str, n: int) -> int:
    """Positions of ``n`` that may lie beyond the bound.  None in 32-bit.  In bfloat16 one in fifty (at least one): the
    design norms each head's result without a weight, so where a head's result nearly cancels (the first token of a
    retention head whose q . k is close to zero) rounding decides its sign, and that position's logits move by more than
    rounding elsewhere does."""
    return 0 if dtype == "float32" else max(1, n // 50)


_close = {}
CLOSE_CALL = 0.03       # a router's margin, as a part of its largest logit, below which bfloat16 rounding may choose otherwise


def close_calls(folder, tokens, dtype) -> set:
    """The positions at which a router of the plain model makes a close call.  In bfloat16 the rounding of the
    activations may decide such a call the other way, which moves that position's logits by more than rounding does (later
    positions meet the token's changed keys, values or state diluted among all the others): comparisons in bfloat16 leave
    these positions out.  In 32-bit every position counts."""
    if dtype == "float32":
        return set()
    key = (folder, tuple(tokens))
    if key not in _close:
        margins = []
        plain.forward(plain.read_config(folder), helpers._plain_weights(folder), list(tokens), margins=margins)
        found = set()
        for m in margins:
            found |= set(int(i) for i in torch.nonzero(m < CLOSE_CALL).flatten())
        _close[key] = found
    return _close[key]


def within(got: torch.Tensor, folder, tokens, dtype, alone: bool = False) -> None:
    """``got`` [T, vocab] against the plain logits of ``tokens``, position by position except at close calls."""
    ref = helpers.plain_logits(folder, tokens)
    keep = [i for i in range(len(tokens)) if i not in close_calls(folder, tokens, dtype)]
    assert bool(torch.isfinite(got).all()) and 3 * len(keep) >= len(tokens)
    d = (got[keep].double() - ref[keep]).abs().max(dim=1).values
    over = int((d > tol(dtype, ref, alone)).sum())
    assert over <= (0 if alone else outliers_allowed(dtype, len(keep))), (over, float(d.max()), tol(dtype, ref, alone))


def compare(folder, prompts, trace, got, dtype, alone: bool = False) -> float:
    worst, counted, total, over = 0.0, 0, 0, []
    for n in sorted(trace.expect):
        exp = trace.expect[n]
        assert got[n].shape[0] == len(exp), f"step {n}: {got[n].shape[0]} rows, {len(exp)} wanted"
        for i, (r, pos) in enumerate(exp):
            ref = helpers.plain_logits(folder, prompts[r])
            total += 1
            if pos in close_calls(folder, prompts[r], dtype):
                assert np.isfinite(got[n][i]).all()
                continue
            counted += 1
            d = float(np.abs(got[n][i].astype(np.float64) - ref[pos].numpy()).max())
            bound = tol(dtype, ref, alone)
            assert np.isfinite(d)
            if d > bound:
                over.append(f"step {n}, request {r} (length {len(prompts[r])}), position {pos}: |dlogit| {d:.3e} > {bound:.1e} "
                            f"(entries {[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
            else:
                worst = max(worst, d / bound)
    assert len(over) <= (0 if alone else outliers_allowed(dtype, counted)), over
    assert 3 * counted >= total, f"only {counted} of {total} positions are free of a router's close call: the test compares too little"
    return worst


def replay(folder, prompts, family, device, dtype, page_size=16, sizes=None, tail=20, alone: bool = False) -> float:
    """One way of cutting the requests into steps, with no more pages than the live requests need (so that pages and
    state rows are used again), against the plain implementation.  Returns the worst error as a part of its bound."""
    make = {"whole": helpers.trace_whole, "tail": lambda p: helpers.trace_tail(p, tail=tail),
            "portions": (lambda p: helpers.trace_portions(p, sizes=sizes)) if sizes else helpers.trace_portions,
            "mixed": lambda p: helpers.trace_mixed(p, max_live=3, seed=5)}[family]
    trace = make(prompts)
    pages = max(1, helpers.tokens_needed(trace, round_to=page_size) // page_size)
    runner = runner_for(folder, device, dtype, num_pages=pages, max_requests=3 if family == "mixed" else 1, page_size=page_size)
    got = helpers.run_trace_inproc(runner, trace)
    worst = compare(folder, prompts, trace, got, dtype, alone)
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    assert runner.cache.free_rows == runner.cache.max_requests
    runner.cache.check()
    return worst


def sharpen_attention(t: Dict[str, torch.Tensor], factor: float = 4.0) -> None:
    """Scales the weights of the query norms so that a position's attention lies on a few keys: a key that is wrongly
    seen or wrongly hidden then moves the logits far beyond rounding."""
    for n in t:
        if n.endswith("mix.q.norm"):
            t[n] = (t[n].float() * factor).to(t[n].dtype)


def greedy_generation(folder, name, device, dtype, n_new=12):
    """Greedy generation through the entry point and its scheduler (portions of prompts beside decoding requests)."""
    from vt_transformer_b200 import LLM, SamplingParams
    prompts = prompts_for(name)[1:4]
    llm = LLM(folder, dtype=dtype, device=device, max_running_reqs=3, num_pages=24, max_seq_len=192, page_size=16,
              max_extend_tokens=40, chunk_size=24)
    outs = llm.generate(prompts, SamplingParams(temperature=0.0, max_tokens=n_new, ignore_eos=True))
    cfg, w = plain.read_config(folder), helpers._plain_weights(folder)
    for p, o in zip(prompts, outs):
        assert len(o) == n_new
        ref = plain.forward(cfg, w, list(p) + o)
        close = close_calls(folder, list(p) + o, dtype)
        for i, tok in enumerate(o):
            if len(p) - 1 + i in close:
                continue
            row = ref[len(p) - 1 + i]
            # the token is the plain argmax, or (two logits closer than the rounding) its plain logit is within the bound
            assert float(row.max() - row[tok]) <= 2 * tol(dtype, ref), (len(p), i, tok)
    llm.runner.cache.check()
    assert llm.stats["free_pages"] == [24] * len(llm.runner.cache.groups)
    return outs
