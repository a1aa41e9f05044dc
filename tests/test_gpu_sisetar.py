"""Sisetar on the GPU: every mechanism alone and the whole model, through the engine's step and entry point, against
the plain implementation (tests/plain/sisetar_plain.py)."""
import json
import os

import pytest
import torch

import helpers
import sisetar_cases as cases
from plain import sisetar_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["bfloat16", "float32"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def sisetar_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"sisetar_{name}")))
        return made[name]
    return get


def _logits(folder, tokens):
    return helpers.plain_logits(folder, tokens)


# ----------------------------------------------------------------------------- kernels against the plain functions


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("hidden", [48, 200, 4104])
def test_layer_norm_kernel(dtype, hidden):
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn((7, hidden), generator=g) * 3 + 5.0          # a mean far from zero: E[x^2] - mean^2 would lose digits
    d = (torch.randn((7, hidden), generator=g)).to(dtype)
    w = 1 + 0.2 * torch.randn(hidden, generator=g)
    rows = torch.tensor([5, 0, 3], dtype=torch.int32)
    xd, out = x.to(DEV), torch.empty((3, hidden), dtype=dtype, device=DEV)
    ops.layernorm(xd, w.to(DEV), 1e-5, out, delta=d.to(DEV), rows=rows.to(DEV))
    v = x.double() + d.double()
    ref = plain.layer_norm(v[rows.long()], w.double(), 1e-5)
    assert float((out.double().cpu() - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 4e-2)
    assert float((xd.cpu().double()[rows.long()] - v[rows.long()]).abs().max()) <= 1e-6      # the sum went back into the stream
    assert torch.equal(xd.cpu()[[1, 2, 4, 6]], x[[1, 2, 4, 6]])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_polynorm_kernel(dtype):
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(3)
    z = (torch.randn((5, 136), generator=g) * 2).to(dtype)
    coef = torch.tensor([0.7, -0.4, 0.2, 0.05])
    out = torch.empty_like(z, device=DEV)
    ops.polynorm(z.to(DEV), coef.to(DEV), 1e-5, out)
    zz = z.double()
    ref = 0.7 * plain.rms(zz, 1e-5) - 0.4 * plain.rms(zz * zz, 1e-5) + 0.2 * plain.rms(zz ** 3, 1e-5) + 0.05
    assert float((out.double().cpu() - ref).abs().max()) <= (1e-5 if dtype == torch.float32 else 3e-2)


# ----------------------------------------------------------------------------- each mechanism alone, in a model of one layer


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gla_alone", "attention_alone", "delta_alone", "ffn_alone"])
def test_each_mechanism_alone(sisetar_folders, name, dtype):
    folder = sisetar_folders(name)
    prompts = cases.prompts_for(name, lengths=[1, 12, 45])
    for family in ("whole", "tail", "portions"):
        cases.replay(folder, prompts, family, DEV, dtype)


# ----------------------------------------------------------------------------- the whole model, cut in every way


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "wide", "gla_only"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(sisetar_folders, name, family, dtype):
    cases.replay(sisetar_folders(name), cases.prompts_for(name), family, DEV, dtype)


@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
@pytest.mark.parametrize("name", ["square", "square64"])
def test_chunks_through_the_tensor_core_attention_kernels(sisetar_folders, name, family):
    """Values as wide as keys: in bfloat16 the attention runs the kernels of the plain attention with the chunk as one
    more bound of the keys (32-bit runs the general kernel: the same cases, as the oracle's check of the configuration)."""
    from vt_transformer_b200 import ops
    folder = sisetar_folders(name)
    before = ops.launches
    cases.replay(folder, cases.prompts_for(name), family, DEV, "bfloat16", sizes=(40, 3, 64, 2, 150))
    cases.replay(folder, cases.prompts_for(name), family, DEV, "float32", sizes=(40, 3, 64, 2, 150))
    assert ops.launches > before


def test_keys_at_a_chunks_edge_through_the_tensor_core_kernels(sisetar_folders, tmp_path):
    """The marked token just inside and just outside the asking position's chunk of 100, where a tile of 128 rows and a
    block of 128 keys straddle the chunk's edge; prompt portions (tcgen05, mma.sync) and single tokens."""
    folder = cases.rewritten(sisetar_folders("square64"), str(tmp_path / "sharp64"), lambda t: cases.sharpen_attention(t, 6.0))
    base = cases.prompts_for("square64", lengths=[330])[0]
    ask, start = 317, 300
    marked = max(range(0, 200, 7), key=lambda tok: _sensitivity(folder, base, ask, start, tok))
    runner = cases.runner_for(folder, DEV, "bfloat16", num_pages=24, max_requests=1)
    seen = {}
    for where in (start, start - 1):
        ids = list(base)
        ids[where] = marked
        ref = _logits(folder, ids)
        seen[where] = ref[ask]
        for cuts in ([len(ids)], [ask, 1, 1, 1], [150, 149, 1, 1, 16], [299, 31]):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= cases.tol("bfloat16", ref), (where, cuts)
    assert float((seen[start] - seen[start - 1]).abs().max()) > 3 * cases.tol("bfloat16", _logits(folder, base))


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_two_tokens_and_pages_of_64(sisetar_folders, dtype):
    folder = sisetar_folders("mix")
    cases.replay(folder, cases.prompts_for("mix")[1:4], "portions", DEV, dtype, sizes=(2,))
    cases.replay(folder, cases.prompts_for("mix"), "mixed", DEV, dtype, page_size=64)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests_equal_each_alone_and_rows_are_used_again(sisetar_folders, dtype):
    """Three requests of different lengths stepped together, one of them sitting a step out; then the same rows and
    pages serve other requests.  In 32-bit the logits are those of each request alone, bit for bit."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = sisetar_folders("mix")
    runner = cases.runner_for(folder, DEV, dtype, num_pages=16, max_requests=3)
    for turn in range(2):
        prompts = cases.prompts_for("mix", seed=turn, lengths=[50, 7, 23])
        alone = []
        for p in prompts:
            row = runner.admit()
            alone.append(cases.step_all(runner, row, p, [len(p)]))
            runner.release(row)
        rows = [runner.admit() for _ in prompts]
        done, got = [0, 0, 0], [[], [], []]
        step = 0
        while any(d < len(p) for d, p in zip(done, prompts)):
            entries, who = [], []
            for i, p in enumerate(prompts):
                if done[i] < len(p) and not (i == 1 and step == 1):
                    k = min([9, 1, 4][(i + step) % 3], len(p) - done[i])
                    entries.append(StepEntry(rows[i], p[done[i]:done[i] + k], list(range(k))))
                    who.append((i, k))
                    done[i] += k
            logits, at = runner.step(entries).double().cpu(), 0
            for i, k in who:
                got[i].append(logits[at:at + k])
                at += k
            step += 1
        runner.check_status()
        for i, p in enumerate(prompts):
            ref = _logits(folder, p)
            assert float((torch.cat(got[i]) - ref).abs().max()) <= cases.tol(dtype, ref)
            if dtype == "float32":
                assert torch.equal(torch.cat(got[i]), alone[i]), "logits depend on what else is in the batch"
        for r in rows:
            runner.release(r)
        runner.cache.check()


# ----------------------------------------------------------------------------- edges of chunks, far keys, first tokens


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_just_inside_and_just_outside_a_chunk(sisetar_folders, tmp_path, dtype):
    """Attention alone, sharpened so that one key can carry a position's weight.  A marked token stands once just
    inside the asking position's chunk and once just outside it: the plain logits of the two differ far beyond the
    bound, and the engine gives each its own, in a prompt's portion and decoded alone, with pages of 16 whose
    borders lie inside the chunks of 9."""
    folder = cases.rewritten(sisetar_folders("attention_alone"), str(tmp_path / "sharp"), lambda t: cases.sharpen_attention(t, 6.0))
    chunk = cases.CONFIGS["attention_alone"]["layers"][0]["mixer"]["left"]["mask"]["size"]
    base = cases.prompts_for("attention_alone", lengths=[6 * chunk + 3])[0]
    ask = 5 * chunk + 4                     # asks from the middle of the sixth chunk
    start = 5 * chunk
    marked = max(range(128), key=lambda tok: _sensitivity(folder, base, ask, start, tok))
    runner = cases.runner_for(folder, DEV, dtype, num_pages=8, max_requests=1)
    seen = {}
    for where in (start, start - 1, ask, start + 1):
        ids = list(base)
        ids[where] = marked
        ref = _logits(folder, ids)
        seen[where] = ref[ask]
        for cuts in ([len(ids)], [ask, 1, 1, 1], [start - 1, 1, 1, 2, 3], [2]):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= cases.tol(dtype, ref), (where, cuts)
    gap = float((seen[start] - seen[start - 1]).abs().max())
    assert gap > 3 * cases.tol(dtype, _logits(folder, base)), gap      # the test would see a chunk that is one token off


def _sensitivity(folder, base, ask, where, tok):
    ids = list(base)
    ids[where] = tok
    return float((_logits(folder, ids)[ask] - _logits(folder, base)[ask]).abs().max())


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["gla_alone", "delta_alone"])
def test_a_token_far_back_still_decides_a_recurrent_state(sisetar_folders, tmp_path, name, dtype):
    """Decays of nearly one: what token 2 wrote into the state decides the logits 400 tokens later.  The prompt runs
    in portions, its end token by token; the plain logits with another token 2 differ far beyond the bound."""
    folder = cases.rewritten(sisetar_folders(name), str(tmp_path / "long"), cases.remember_everything)
    ids = cases.prompts_for(name, lengths=[420])[0]
    other = list(ids)
    other[2] = (ids[2] + 17) % 128
    ref, ref_other = _logits(folder, ids), _logits(folder, other)
    # (one token among hundreds moves the logits by a hundredth of their spread: far beyond the 32-bit bound, which is
    # the run that would show a lost state; the bfloat16 run checks the same path against its own, wider bound)
    assert float((ref[-1] - ref_other[-1]).abs().max()) > 100 * cases.tol("float32", ref)
    runner = cases.runner_for(folder, DEV, dtype, num_pages=30, max_requests=2)
    for tokens, want in ((ids, ref), (other, ref_other)):
        row = runner.admit()
        got = cases.step_all(runner, row, tokens, [150, 37, 200] + [1] * 40)
        runner.release(row)
        assert float((got - want).abs().max()) <= cases.tol(dtype, want)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(sisetar_folders, dtype):
    """A request of one token, then 150 tokens decoded one by one (through the captured graphs of single-token
    steps, over page borders and chunk borders), beside a second request that joins and leaves."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = sisetar_folders("mix")
    a, b = cases.prompts_for("mix", seed=9, lengths=[151, 40])
    runner = cases.runner_for(folder, DEV, dtype, num_pages=14, max_requests=2)
    ra = runner.admit()
    got_a, got_b, rb = [], [], None
    for i, tok in enumerate(a):
        entries = [StepEntry(ra, [tok], [0])]
        if 30 <= i < 30 + len(b):
            if rb is None:
                rb = runner.admit()
            entries.append(StepEntry(rb, [b[i - 30]], [0]))
        logits = runner.step(entries).double().cpu()
        got_a.append(logits[0])
        if len(entries) == 2:
            got_b.append(logits[1])
            if i - 30 == len(b) - 1:
                runner.release(rb)
    runner.check_status()
    for got, ids in ((got_a, a), (got_b, b)):
        ref = _logits(folder, ids)
        assert float((torch.stack(got) - ref).abs().max()) <= cases.tol(dtype, ref)
    assert runner._graphs, "single-token steps did not run as captured graphs"


# ----------------------------------------------------------------------------- the entry point


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "gla_only"])
def test_greedy_generation_through_the_entry_point(sisetar_folders, name, dtype):
    cases.greedy_generation(sisetar_folders(name), name, DEV, dtype)


def test_trace_replay_command(sisetar_folders, tmp_path):
    folder = sisetar_folders("mix")
    prompts = cases.prompts_for("mix")
    trace = helpers.trace_mixed(prompts, max_live=4, seed=2)
    got = helpers.run_trace_cli(folder, trace, "float32", str(tmp_path / "out"), helpers.tokens_needed(trace, 64))
    cases.compare(folder, prompts, trace, got, "float32")
