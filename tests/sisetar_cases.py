"""Configurations, weights and scenarios of the Sisetar tests.  Every scenario runs the engine (``ModelRunner.step`` or
``LLM.generate``) and compares with the plain implementation (tests/plain/sisetar_plain.py); each takes the device and
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
from plain import sisetar_plain as plain


def _gla(heads, dim, vdim, tau, ff=None):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _par(heads, kv_heads, dim, vdim, rot, base, scale, chunk, rheads, rdim, ls, rs, ff=None):
    return {"type": "parallel",
            "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "rot": {"dims": rot, "base": base},
                               "scale": scale, "mask": {"size": chunk}},
                      "right": {"heads": rheads, "dim": rdim}, "left_scale": ls, "right_scale": rs},
            "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _model(vocab, width, layers, emb=1.0, logit_scale=1.0, cap=0.0, eps=1e-5):
    return {"architecture": "Sisetar", "vocab": vocab, "width": width, "layers": layers, "embedding": {"scale": emb},
            "logit_scale": logit_scale, "logit_softcap": cap, "norm": {"eps": eps}}


# Configurations that differ from one another in every size and constant: head counts of 1, grouped and ungrouped
# query heads, values wider and narrower than keys, a rotation of the whole head, of a part and of nothing, chunks
# smaller and larger than a page, feed-forwards on either kind of layer and on none, scales of 1 and others, with and
# without the soft cap; head sizes below 32, between 32 and 64, between 64 and 128 and above 128 (each a shape of its
# own of the scan kernel), sizes that are no multiples of 8, 16 or 32.
CONFIGS: Dict[str, dict] = {
    "mix": _model(300, 64, [_par(4, 4, 32, 48, 32, 100.0, 0.3, 7, 2, 40, 1.0, 1.0, ff=96), _gla(3, 24, 40, 4.0, ff=72),
                            _gla(1, 32, 32, 1.0), _par(4, 1, 40, 16, 8, 5000.0, 0.11, 33, 1, 16, 0.5, 2.0, ff=50)],
                  emb=3.0, logit_scale=0.7, cap=8.0),
    "wide": _model(257, 72, [_gla(2, 136, 72, 8.0), _par(2, 1, 72, 20, 0, 10000.0, 0.2, 50, 1, 160, 1.5, 0.6, ff=40),
                             _gla(1, 72, 100, 2.0)], emb=1.0, logit_scale=1.0, cap=0.0, eps=1e-6),
    # values as wide as keys at head sizes that the tensor-core attention kernels take (32: mma.sync tiles and the
    # single-token kernel; 64 with four query heads a group: tcgen05 for portions of 32 tokens and more)
    "square": _model(200, 64, [_par(4, 2, 32, 32, 16, 1000.0, 0.2, 21, 1, 24, 1.3, 0.7, ff=48), _gla(2, 16, 16, 2.0)], emb=2.0, cap=6.0),
    "square64": _model(200, 64, [_par(4, 1, 64, 64, 64, 1e4, 0.125, 100, 1, 16, 1.0, 1.0)], emb=2.0),
    "gla_only": _model(128, 48, [_gla(2, 20, 28, 3.0), _gla(2, 20, 28, 3.0, ff=56)], emb=2.0, cap=5.0),
    "gla_alone": _model(128, 48, [_gla(3, 16, 24, 2.0)], emb=2.0),
    "attention_alone": _model(128, 48, [_par(3, 1, 24, 40, 12, 777.0, 0.25, 9, 1, 8, 1.0, 0.0)], emb=2.0),
    "delta_alone": _model(128, 48, [_par(1, 1, 8, 8, 4, 777.0, 0.25, 9, 2, 36, 0.0, 1.0)], emb=2.0),
    "ffn_alone": _model(128, 48, [_gla(1, 8, 8, 2.0, ff=88)], emb=2.0),
}
SIGMA = {"mix": 0.15, "wide": 0.12, "square": 0.2, "square64": 0.2, "gla_only": 0.2, "gla_alone": 0.2, "attention_alone": 0.25, "delta_alone": 0.2,
         "ffn_alone": 0.2}
SEED = {n: 100 + i for i, n in enumerate(CONFIGS)}
LENGTHS = {"mix": [1, 9, 40, 71, 130], "wide": [3, 33, 90, 52], "gla_only": [2, 30, 77], "square": [1, 19, 64, 110],
           "square64": [5, 150, 260, 64]}


def make_folder(name: str, folder: str) -> str:
    from vt_transformer_b200.config import config_from_dict
    from vt_transformer_b200.weights import write_random_model
    return write_random_model(config_from_dict(copy.deepcopy(CONFIGS[name])), folder, seed=SEED[name], sigma=SIGMA[name])


def rewritten(folder: str, out: str, change: Callable[[Dict[str, torch.Tensor]], None], config: Callable[[dict], None] = None) -> str:
    """A copy of a model folder whose tensors (and configuration) ``change`` has altered."""
    from safetensors import safe_open
    from safetensors.torch import save_file
    os.makedirs(out, exist_ok=True)
    tensors = {}
    with safe_open(os.path.join(folder, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            tensors[n] = f.get_tensor(n).clone()
    change(tensors)
    save_file({n: t.contiguous() for n, t in tensors.items()}, os.path.join(out, "model.safetensors"))
    with open(os.path.join(folder, "config.json")) as f:
        c = json.load(f)
    if config is not None:
        config(c)
    with open(os.path.join(out, "config.json"), "w") as f:
        json.dump(c, f)
    return out


def prompts_for(name: str, seed: int = 0, lengths=None) -> List[List[int]]:
    rng = random.Random(500 + seed)
    vocab = CONFIGS[name]["vocab"]
    return [[rng.randrange(vocab) for _ in range(n)] for n in (lengths or LENGTHS[name])]


def tol(dtype: str, ref: torch.Tensor) -> float:
    """The bound on |logit - plain logit|, as a part of the spread of the model's plain logits.  Measured on a B200 over
    the configurations above and the four ways of cutting (the cut changes nothing: a configuration's worst error is
    the same in all four).  32-bit, rounding and the order of sums only: 1.4e-6 to 8.2e-6 of the spread; the bound is
    5e-5.  bfloat16, activations rounded to 8 bits at every part: 0.019 to 0.094 of the spread (the largest where a
    layer norm follows a small residual); the bound is three times the worst, 0.3."""
    spread = max(1.0, float(ref.double().std()))
    return (5e-5 if dtype == "float32" else 0.3) * spread


def runner_for(folder, device, dtype, num_pages, max_requests=4, page_size=16):
    from vt_transformer_b200.engine.runner import ModelRunner
    return ModelRunner.from_folder(folder, dtype=dtype, device=device, page_size=page_size, num_pages=num_pages,
                                   max_requests=max_requests, max_seq_len=None)


def compare(folder, prompts, trace, got, dtype) -> float:
    worst = 0.0
    for n in sorted(trace.expect):
        exp = trace.expect[n]
        assert got[n].shape[0] == len(exp), f"step {n}: {got[n].shape[0]} rows, {len(exp)} wanted"
        for i, (r, pos) in enumerate(exp):
            ref = helpers.plain_logits(folder, prompts[r])
            d = float(np.abs(got[n][i].astype(np.float64) - ref[pos].numpy()).max())
            bound = tol(dtype, ref)
            assert np.isfinite(d) and d <= bound, (
                f"step {n}, request {r} (length {len(prompts[r])}), position {pos}: |dlogit| {d:.3e} > {bound:.1e} "
                f"(entries {[(e['id'], len(e['tokens'])) for e in trace.steps[n]['entries']]})")
            worst = max(worst, d / bound)
    return worst


def replay(folder, prompts, family, device, dtype, page_size=16, sizes=None) -> float:
    """One way of cutting the requests into steps, with no more pages than the live requests need (so that pages and
    state rows are used again), against the plain implementation.  Returns the worst error as a part of its bound."""
    make = {"whole": helpers.trace_whole, "tail": lambda p: helpers.trace_tail(p, tail=20),
            "portions": (lambda p: helpers.trace_portions(p, sizes=sizes)) if sizes else helpers.trace_portions,
            "mixed": lambda p: helpers.trace_mixed(p, max_live=3, seed=5)}[family]
    trace = make(prompts)
    pages = max(1, helpers.tokens_needed(trace, round_to=page_size) // page_size)
    runner = runner_for(folder, device, dtype, num_pages=pages, max_requests=3 if family == "mixed" else 1, page_size=page_size)
    got = helpers.run_trace_inproc(runner, trace)
    worst = compare(folder, prompts, trace, got, dtype)
    assert runner.cache.free_pages() == [g.pool.num_pages for g in runner.cache.groups]
    assert runner.cache.free_rows == runner.cache.max_requests
    return worst


def step_all(runner, row, tokens, cuts):
    """The logits of every position of ``tokens``, run through ``runner`` in portions of the sizes ``cuts`` (cycled)."""
    from vt_transformer_b200.engine.batch import StepEntry
    out, at, i = [], 0, 0
    while at < len(tokens):
        k = min(cuts[i % len(cuts)], len(tokens) - at)
        out.append(runner.step([StepEntry(row, tokens[at:at + k], list(range(k)))]).double().cpu())
        at, i = at + k, i + 1
    runner.check_status()
    return torch.cat(out)


def sharpen_attention(t: Dict[str, torch.Tensor], factor: float = 4.0) -> None:
    """Scales the query projections of the softmax attention so that a position's weight lies on a few keys: a key
    that is wrongly seen or wrongly hidden then moves the logits far beyond rounding."""
    for n in t:
        if n.endswith("left.q"):
            t[n] = (t[n].float() * factor).to(t[n].dtype)


def remember_everything(t: Dict[str, torch.Tensor]) -> None:
    """Decays of (nearly) one and a removal rate of (nearly) zero: what the first tokens wrote into a recurrent state
    still decides the output hundreds of tokens later."""
    for n in t:
        if n.endswith("mix.a2.b"):
            t[n] = torch.full_like(t[n], 9.0)
        if n.endswith("right.w0") or n.endswith("right.a.b"):
            t[n] = torch.full_like(t[n], -9.0)


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
        for i, tok in enumerate(o):
            row = ref[len(p) - 1 + i]
            # the token is the plain argmax, or (two logits closer than the rounding) its plain logit is within the bound
            assert float(row.max() - row[tok]) <= 2 * tol(dtype, ref), (len(p), i, tok)
    llm.runner.cache.check()
    assert llm.stats["free_pages"] == [24] * len(llm.runner.cache.groups)
    return outs
