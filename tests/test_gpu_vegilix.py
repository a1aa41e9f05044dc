"""Vegilix on the GPU: every mechanism alone and the whole model, through the engine's step and entry point, against
the plain implementation (tests/plain/vegilix_plain.py)."""
import pytest
import torch

import helpers
import vegilix_cases as cases
from plain import vegilix_plain as plain

pytestmark = pytest.mark.gpu
DTYPES = ["bfloat16", "float32"]
DEV = "cuda:0"


@pytest.fixture(scope="module")
def vegilix_folders(tmp_path_factory):
    made = {}

    def get(name):
        if name not in made:
            made[name] = cases.make_folder(name, str(tmp_path_factory.mktemp(f"vegilix_{name}")))
        return made[name]
    return get


def _logits(folder, tokens):
    return helpers.plain_logits(folder, tokens)


def _sensitivity(folder, base, ask, where, tok):
    ids = list(base)
    ids[where] = tok
    return float((_logits(folder, ids)[ask] - _logits(folder, base)[ask]).abs().max())


# ----------------------------------------------------------------------------- kernels against the plain functions


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("hidden", [48, 200, 4104])
@pytest.mark.parametrize("shares", [0, 3])
def test_norm_kernel_norms_the_delta_before_the_sum(dtype, hidden, shares):
    """x <- x + m * norm_b(delta); out = norm_a(x): the delta as a tensor and as the unadded shares of a product."""
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(hidden + shares)
    x = torch.randn((7, hidden), generator=g) * 3
    wa, wb = 0.2 * torch.randn(hidden, generator=g), 0.2 * torch.randn(hidden, generator=g)
    rows = torch.tensor([5, 0, 3], dtype=torch.int32)
    if shares:
        parts = torch.randn((shares, 7, hidden), generator=g) * 2
        d, delta = parts.double().sum(0), ops.SplitSum(parts.to(DEV))
    else:
        delta = (torch.randn((7, hidden), generator=g) * 2).to(dtype)
        d, delta = delta.double(), delta.to(DEV)
    xd, out = x.to(DEV), torch.empty((3, hidden), dtype=dtype, device=DEV)
    ops.rmsnorm(xd, (1 + wa).to(DEV), 1e-5, out, delta=delta, rows=rows.to(DEV), post=((1 + wb).to(DEV), 1e-5, 0.7))
    v = x.double() + 0.7 * plain.norm(d, wb.double(), 1e-5)
    ref = plain.norm(v[rows.long()], wa.double(), 1e-5)
    assert float((out.double().cpu() - ref).abs().max()) <= (2e-5 if dtype == torch.float32 else 4e-2)
    assert float((xd.cpu().double()[rows.long()] - v[rows.long()]).abs().max()) <= 2e-6      # the sum went back into the stream
    assert torch.equal(xd.cpu()[[1, 2, 4, 6]], x[[1, 2, 4, 6]])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("experts,top,inter", [(5, 2, 24), (1, 1, 8), (40, 40, 16), (130, 7, 8), (3, 1, 12)])
def test_routing_kernel(dtype, experts, top, inter):
    from vt_transformer_b200 import ops
    g = torch.Generator().manual_seed(experts)
    T, extra = 9, 16
    z = torch.randn((T, experts), generator=g) * 2
    z[0, :] = 0.5                                            # all equal: the lowest indices are picked
    act = torch.randn((T, experts * inter + extra), generator=g).to(dtype)
    got = act.clone().to(DEV)
    ops.route_experts(z.to(DEV), top, got, inter)
    ref = act.double().clone()
    for t in range(T):
        order = sorted(range(experts), key=lambda e: (-float(z[t, e]), e))[:top]
        w = torch.zeros(experts, dtype=torch.float64)
        w[order] = torch.softmax(z[t, order].double(), dim=0)
        ref[t, :experts * inter] = (ref[t, :experts * inter].view(experts, inter) * w[:, None]).reshape(-1)
    assert float((got.double().cpu() - ref).abs().max()) <= (1e-5 if dtype == torch.float32 else 3e-2)
    assert torch.equal(got.cpu()[:, experts * inter:], act[:, experts * inter:])     # the shared expert's columns stay
    # the same with the logits formed in the kernel from input rows and a router's matrix: rows that point along one
    # router row each, so that no choice is a close call
    width = 64
    router = torch.randn((experts, width), generator=g)
    order = [[(3 * t + 5 * k) % experts for k in range(experts)] for t in range(T)]
    x = torch.stack([sum((top + 2.0 - min(k, top + 1)) * router[order[t][k]] / router[order[t][k]].norm() ** 2 for k in range(min(top + 1, experts)))
                     for t in range(T)]).to(dtype)
    z2 = x.double() @ router.double().t()
    got2, ids, wts = act.clone().to(DEV), torch.empty((T, top), dtype=torch.int32, device=DEV), torch.empty((T, top), device=DEV)
    ops.route_experts(None, top, got2, inter, x=x.to(DEV), router=router.to(DEV))
    ops.route_topk(None, top, ids, wts, x=x.to(DEV), router=router.to(DEV))
    ref2 = act.double().clone()
    for t in range(T):
        picks = sorted(range(experts), key=lambda e: (-float(z2[t, e]), e))[:top]
        w = torch.zeros(experts, dtype=torch.float64)
        w[picks] = torch.softmax(z2[t, picks], dim=0)
        ref2[t, :experts * inter] = (ref2[t, :experts * inter].view(experts, inter) * w[:, None]).reshape(-1)
        if experts > top + 1:           # the margins between the first top + 1 logits are wide by construction
            assert ids[t].tolist() == picks
            assert float((wts[t].double().cpu() - w[picks]).abs().max()) <= (1e-5 if dtype == torch.float32 else 2e-2)
    if experts > top + 1:
        assert float((got2.double().cpu() - ref2).abs().max()) <= (1e-5 if dtype == torch.float32 else 6e-2)


# ----------------------------------------------------------------------------- each mechanism alone, in a model of one layer


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["attention_alone", "retention_alone", "experts_alone"])
def test_each_mechanism_alone(vegilix_folders, name, dtype):
    folder = vegilix_folders(name)
    prompts = cases.prompts_for(name, lengths=[1, 12, 45])
    for family in ("whole", "tail", "portions"):
        cases.replay(folder, prompts, family, DEV, dtype, alone=name != "experts_alone")


# ----------------------------------------------------------------------------- the whole model, cut in every way


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "wide", "looped_start"])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_equal_the_plain_implementation(vegilix_folders, name, family, dtype):
    cases.replay(vegilix_folders(cases.for_dtype(name, dtype)), cases.prompts_for(name), family, DEV, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("segments", [(8, 3), (16, 8), (33, 2)])
def test_long_retention_walks_cut_into_segments(vegilix_folders, monkeypatch, segments, dtype):
    """A sequence that brings many tokens has its retention walk cut into segments that run side by side (the later ones
    from zeros; the states carried and the outputs completed afterwards): forced here for short sequences, with segment
    lengths that are no multiples of the staged batches of 16 tokens or of the tiles of 32."""
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "RETENTION_SEGMENT_MIN", segments[0])
    monkeypatch.setattr(ops, "RETENTION_SEGMENTS", segments[1])
    for name in ("retention_alone", "wide", "mix"):
        folder = vegilix_folders(name if name == "retention_alone" else cases.for_dtype(name, dtype))
        for family in ("whole", "portions", "mixed"):
            cases.replay(folder, cases.prompts_for(name), family, DEV, dtype, sizes=(40, 3, 70, 2, 150), alone=name == "retention_alone")


def test_the_cut_walk_leaves_the_state_of_the_walk_in_one_piece(vegilix_folders, monkeypatch):
    """A prompt of 300 tokens in one step, cut into 8 segments, then 20 tokens decoded from the state it left: the decoded
    logits equal the plain ones (the carried state is the walk's), in 32-bit."""
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "RETENTION_SEGMENT_MIN", 32)
    folder = vegilix_folders("retention_alone")
    ids = cases.prompts_for("retention_alone", lengths=[320])[0]
    runner = cases.runner_for(folder, DEV, "float32", num_pages=1, max_requests=1)
    row = runner.admit()
    got = cases.step_all(runner, row, ids, [300] + [1] * 20)
    runner.release(row)
    ref = _logits(folder, ids)
    assert float((got - ref).abs().max()) <= cases.tol("float32", ref, alone=True)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "wide", "experts_alone"])
def test_tokens_grouped_by_expert(vegilix_folders, monkeypatch, name, dtype):
    """Portions with many picks group their tokens by expert (the experts' products over slices of sorted rows) instead of
    running every expert on every token: forced here for every portion, also those in which an expert gets no token."""
    from vt_transformer_b200 import ops
    monkeypatch.setattr(ops, "EXPERTS_GROUPED_MIN_PICKS", 1)
    folder = vegilix_folders(cases.for_dtype(name, dtype) if name != "experts_alone" else name)
    before = ops.launches
    for family in ("whole", "portions", "mixed"):
        cases.replay(folder, cases.prompts_for(name), family, DEV, dtype)
    assert ops.launches > before


@pytest.mark.parametrize("page_size", [16, 64])
@pytest.mark.parametrize("family", ["whole", "tail", "portions", "mixed"])
def test_cuts_through_the_tensor_core_attention_kernel(vegilix_folders, family, page_size):
    """Sizes that the tensor-core kernel of the differential attention takes: bfloat16 runs it for prompt portions and
    for single tokens (32-bit runs the plain kernel: the same cases, as the oracle's check of the configuration)."""
    from vt_transformer_b200 import ops
    assert ops.backend().attention_diff_supports(32, 64, 4, 2) and ops.backend().attention_diff_supports(64, 128, 2, 1)
    sizes = (40, 3, 64, 2, 150)
    cases.replay(vegilix_folders("tensor"), cases.prompts_for("tensor"), family, DEV, "bfloat16", sizes=sizes, page_size=page_size, tail=70)
    if page_size == 16:
        cases.replay(vegilix_folders("tensor"), cases.prompts_for("tensor"), family, DEV, "float32", sizes=sizes, tail=70)
    # heads of 128 with values of 256 and of 128, three query heads a head of values
    assert ops.backend().attention_diff_supports(128, 256, 3, 1) and ops.backend().attention_diff_supports(128, 128, 2, 2)
    cases.replay(vegilix_folders("tensor_wide"), cases.prompts_for("tensor_wide"), family, DEV, "bfloat16", sizes=sizes, page_size=page_size, tail=70)


def test_the_windows_edge_and_the_kept_first_tokens_through_the_tensor_core_kernel(vegilix_folders, tmp_path):
    """A window of 100 that keeps the first 3 tokens, asked from position 250: the marked token just inside and just
    outside the window (where a block of 64 keys straddles its edge), at the last kept position and the first that is not
    kept (in a block of its own before the window's); prompt portions and single tokens."""
    folder = cases.rewritten(vegilix_folders("tensor_alone"), str(tmp_path / "sharp_tc"), lambda t: cases.sharpen_attention(t, 6.0))
    mask = cases.CONFIGS["tensor_alone"]["layers"][0]["mixer"]["mask"]
    size, keep = mask["size"], mask["keep_first"]
    base = cases.prompts_for("tensor_alone", lengths=[262])[0]
    ask = 250
    inside, outside = ask - size + 1, ask - size
    marked = max(range(0, 128, 2), key=lambda tok: _sensitivity(folder, base, ask, inside, tok))
    kept_mark = max(range(0, 128, 2), key=lambda tok: _sensitivity(folder, base, ask, keep - 1, tok))
    runner = cases.runner_for(folder, DEV, "bfloat16", num_pages=20, max_requests=1)
    seen = {}
    for where, tok in ((inside, marked), (outside, marked), (keep - 1, kept_mark), (keep, kept_mark)):
        ids = list(base)
        ids[where] = tok
        ref = _logits(folder, ids)
        seen[where] = ref[ask]
        for cuts in ([len(ids)], [ask, 1, 1, 1], [150, 99, 1, 1, 11], [200, 31]):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= cases.tol("bfloat16", ref, alone=True), (where, cuts)
    bound = cases.tol("bfloat16", _logits(folder, base), alone=True)
    assert float((seen[inside] - seen[outside]).abs().max()) > 3 * bound
    assert float((seen[keep - 1] - seen[keep]).abs().max()) > 3 * bound


@pytest.mark.parametrize("dtype", DTYPES)
def test_portions_of_two_tokens_and_pages_of_64(vegilix_folders, dtype):
    folder = vegilix_folders(cases.for_dtype("mix", dtype))
    cases.replay(folder, cases.prompts_for("mix")[1:4], "portions", DEV, dtype, sizes=(2,))
    cases.replay(folder, cases.prompts_for("mix"), "mixed", DEV, dtype, page_size=64)
    cases.replay(folder, cases.prompts_for("mix"), "tail", DEV, dtype, page_size=64, tail=40)


@pytest.mark.parametrize("dtype", DTYPES)
def test_batches_of_unequal_requests_equal_each_alone_and_rows_are_used_again(vegilix_folders, dtype):
    """Three requests of different lengths stepped together, one of them sitting a step out; then the same rows and
    pages serve other requests.  In 32-bit the logits are those of each request alone, bit for bit."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = vegilix_folders(cases.for_dtype("mix", dtype))
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
            cases.within(torch.cat(got[i]), folder, p, dtype)
            if dtype == "float32":
                assert torch.equal(torch.cat(got[i]), alone[i]), "logits depend on what else is in the batch"
        for r in rows:
            runner.release(r)
        runner.cache.check()


# ----------------------------------------------------------------------------- edges of the window, first tokens, far keys


@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_at_the_windows_edge_and_among_the_kept_first_tokens(vegilix_folders, tmp_path, dtype):
    """Attention alone (a window of 11 that keeps the first 2 tokens, pages of 16), sharpened so that one key can carry a
    position's weight.  A marked token stands just inside and just outside the asking position's window, and at the last
    kept position and the first that is not kept: the plain logits of each pair differ far beyond the bound, and the
    engine gives each its own, in a prompt's portion and decoded alone."""
    folder = cases.rewritten(vegilix_folders("attention_alone"), str(tmp_path / "sharp"), lambda t: cases.sharpen_attention(t, 6.0))
    mask = cases.CONFIGS["attention_alone"]["layers"][0]["mixer"]["mask"]
    size, keep = mask["size"], mask["keep_first"]
    base = cases.prompts_for("attention_alone", lengths=[70])[0]
    ask = 53
    inside, outside = ask - size + 1, ask - size
    marked = max(range(128), key=lambda tok: _sensitivity(folder, base, ask, inside, tok))
    kept_mark = max(range(128), key=lambda tok: _sensitivity(folder, base, ask, keep - 1, tok))
    runner = cases.runner_for(folder, DEV, dtype, num_pages=8, max_requests=1)
    seen = {}
    for where, tok in ((inside, marked), (outside, marked), (ask, marked), (keep - 1, kept_mark), (keep, kept_mark)):
        ids = list(base)
        ids[where] = tok
        ref = _logits(folder, ids)
        seen[where] = ref[ask]
        for cuts in ([len(ids)], [ask, 1, 1, 1], [outside, 1, 1, 2, 3], [2], [keep, 1, 1, 40]):
            row = runner.admit()
            got = cases.step_all(runner, row, ids, cuts)
            runner.release(row)
            assert float((got - ref).abs().max()) <= cases.tol(dtype, ref, alone=True), (where, cuts)
    bound = cases.tol(dtype, _logits(folder, base), alone=True)
    # the test would see a window, or a count of kept tokens, that is one token off
    assert float((seen[inside] - seen[outside]).abs().max()) > 3 * bound
    assert float((seen[keep - 1] - seen[keep]).abs().max()) > 3 * bound


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_hundreds_of_tokens_back(vegilix_folders, tmp_path, dtype):
    """Attention alone without a window, sharpened: a marked token at position 3 decides the logits at position 389,
    across 24 pages; in portions, and with the asking tokens decoded one by one."""
    def no_window(c):
        c["layers"][0]["mixer"]["mask"] = {"keep_first": 0}
    folder = cases.rewritten(vegilix_folders("attention_alone"), str(tmp_path / "far"), lambda t: cases.sharpen_attention(t, 4.0),
                             config=no_window)
    base = cases.prompts_for("attention_alone", lengths=[392])[0]
    ask, where = 389, 3
    marked = max(range(0, 128, 3), key=lambda tok: _sensitivity(folder, base, ask, where, tok))
    ids = list(base)
    ids[where] = marked
    ref = _logits(folder, ids)
    assert float((ref[ask] - _logits(folder, base)[ask]).abs().max()) > 3 * cases.tol(dtype, ref, alone=True)
    runner = cases.runner_for(folder, DEV, dtype, num_pages=26, max_requests=1)
    for cuts in ([len(ids)], [150, 37, 190] + [1] * 15, [380] + [1] * 12):
        row = runner.admit()
        got = cases.step_all(runner, row, ids, cuts)
        runner.release(row)
        assert float((got - ref).abs().max()) <= cases.tol(dtype, ref, alone=True), cuts


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_token_far_back_still_decides_a_retention_state(vegilix_folders, tmp_path, dtype):
    """Decays of nearly one and of one: what token 2 wrote into the state decides the logits 400 tokens later.  The
    prompt runs in portions, its end token by token; the plain logits with another token 2 differ far beyond the bound."""
    def slow(c):
        c["layers"][0]["mixer"]["decay"] = [0.999, 1.0, 0.9995]
    folder = cases.rewritten(vegilix_folders("retention_alone"), str(tmp_path / "long"), lambda t: None, config=slow)
    ids = cases.prompts_for("retention_alone", lengths=[420])[0]
    other = list(ids)
    other[2] = (ids[2] + 17) % 128
    ref, ref_other = _logits(folder, ids), _logits(folder, other)
    assert float((ref[-1] - ref_other[-1]).abs().max()) > 100 * cases.tol("float32", ref)
    runner = cases.runner_for(folder, DEV, dtype, num_pages=1, max_requests=2)
    for tokens, want in ((ids, ref), (other, ref_other)):
        row = runner.admit()
        got = cases.step_all(runner, row, tokens, [150, 37, 200] + [1] * 40)
        runner.release(row)
        assert float((got - want).abs().max()) <= cases.tol(dtype, want, alone=True)


@pytest.mark.parametrize("dtype", DTYPES)
def test_first_tokens_and_long_decoding(vegilix_folders, dtype):
    """A request of one token, then 150 tokens decoded one by one (through the captured graphs of single-token
    steps, over page borders, past the window and the kept first tokens), beside a second request that joins and leaves."""
    from vt_transformer_b200.engine.batch import StepEntry
    folder = vegilix_folders(cases.for_dtype("mix", dtype))
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
        cases.within(torch.stack(got), folder, ids, dtype)
    assert runner._graphs, "single-token steps did not run as captured graphs"


# ----------------------------------------------------------------------------- the entry point


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mix", "looped_start"])
def test_greedy_generation_through_the_entry_point(vegilix_folders, name, dtype):
    cases.greedy_generation(vegilix_folders(cases.for_dtype(name, dtype)), name, DEV, dtype)


def test_trace_replay_command(vegilix_folders, tmp_path):
    folder = vegilix_folders("mix")
    prompts = cases.prompts_for("mix")
    trace = helpers.trace_mixed(prompts, max_live=4, seed=2)
    got = helpers.run_trace_cli(folder, trace, "float32", str(tmp_path / "out"), helpers.tokens_needed(trace, 64))
    cases.compare(folder, prompts, trace, got, "float32")


def test_generate_from_the_command_line_greedy_and_sampled(vegilix_folders):
    """The command line's generation with the design's folder: greedy tokens equal the plain argmax; sampled tokens
    (temperature, top-k, top-p) come out the same for the same seed, and lie among the plain model's likely tokens."""
    import os
    import subprocess
    import sys
    folder = vegilix_folders("looped_start")
    prompts = cases.prompts_for("looped_start")[:2]
    base = [sys.executable, "-m", "vt_transformer_b200", "generate", "--model", folder, "--dtype", "float32", "--max-tokens", "6",
            "--ignore-eos", "--num-pages", "16", "--max-seq-len", "128", "--page-size", "16"]
    for p in prompts:
        base += ["--prompt-ids", ",".join(str(t) for t in p)]
    run = lambda extra: subprocess.run(base + extra, capture_output=True, text=True, timeout=600,
                                       env=dict(os.environ, PYTHONPATH=helpers.ROOT), cwd=helpers.ROOT)
    res = run(["--temperature", "0"])
    assert res.returncode == 0, res.stderr[-3000:]
    lines = [[int(t) for t in l.split()] for l in res.stdout.splitlines() if l.strip()]
    assert len(lines) == 2 and all(len(l) == 6 for l in lines)
    for p, o in zip(prompts, lines):
        ref = _logits(folder, list(p) + o)
        for i, tok in enumerate(o):
            row = ref[len(p) - 1 + i]
            assert float(row.max() - row[tok]) <= 2 * cases.tol("float32", ref)
    sampled = [run(["--temperature", "0.8", "--top-k", "5", "--top-p", "0.9", "--seed", "3"]) for _ in range(2)]
    assert all(r.returncode == 0 for r in sampled) and sampled[0].stdout == sampled[1].stdout
    for p, l in zip(prompts, [[int(t) for t in l.split()] for l in sampled[0].stdout.splitlines() if l.strip()]):
        ref = _logits(folder, list(p) + l)
        for i, tok in enumerate(l):
            assert tok in torch.topk(ref[len(p) - 1 + i], 5).indices.tolist()
