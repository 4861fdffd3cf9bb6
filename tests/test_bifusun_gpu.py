"""Bifusun on the GPU against the plain statement in ``tests/plain/bifusun_plain.py``: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, batches of unequal requests, pages and state slots that are used again, keys
far back, at page borders and at a sequence's first positions, long decoding, greedy generation through the engine, and the new
kernels against their formulas."""


import pytest
import torch

import bifusun_util as BU
from plain import bifusun_plain as BP
from util import Replay

pytestmark = pytest.mark.gpu

DEV = "cuda"


CLOSE_CALL = 0.01
"""bfloat16 rows at which some router of the plain model decided by less than this are not compared: a sigmoid score that differs by a
rounding step may choose another expert there, for no fault. (32-bit compares every row.)"""


def close(got, want, dtype, what, margins=None):
    """32-bit: every row within 2e-4 of the row's spread. bfloat16: within 8e-2, except that one row in twenty may be off by up to
    0.5: the matrix memory divides by max(|n . q|, exp(-m)), and where n . q passes near zero a rounding step of q or k moves the
    output by much more than a step (the rows are the same ones whatever the cutting and whoever else is in the batch)."""
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    d = (got - want) - (got - want).mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-6)
    if dtype == "float32":
        assert err.max() <= 2e-4, f"{what}: row {int(err.argmax())} is off by {err.max():.2e} of the row's spread (limit 2e-04)"
        return
    if margins is not None:
        clear = margins >= CLOSE_CALL
        assert clear.float().mean() >= 0.5 or len(clear) < 12, f"{what}: most rows are close calls of a router; the test compares too little"
        err = torch.where(clear, err, torch.zeros_like(err))
    over = int((err > 8e-2).sum())
    assert err.max() <= 0.5 and over <= len(err) // 20, (
        f"{what}: {over} of {len(err)} rows are off by more than 8e-02 of the row's spread, row {int(err.argmax())} by {err.max():.2e}")


def runner_for(folder, dtype, *, page_size=8, num_pages=64, max_requests=4):
    from oxr_inference_b200.engine.runtime import ModelRunner

    return ModelRunner.from_folder(folder, dtype=dtype, page_size=page_size, num_pages=num_pages, max_requests=max_requests)


def feed(runner, rc, ids, lo, hi, want=None):
    from oxr_inference_b200.engine.batch import StepEntry

    assert runner.cache.reserve(rc, hi)
    return StepEntry(rc, ids[lo:hi], list(range(hi - lo)) if want is None else want)


def run_cut(runner, ids, cuts):
    """One request alone, cut into portions; logits of every position."""
    rc = runner.cache.open("r")
    rows, at = [], 0
    for c in cuts:
        rows.append(runner.step([feed(runner, rc, ids, at, at + c)]))
        at += c
    assert at == len(ids)
    runner.check()
    runner.cache.close(rc)
    return torch.cat(rows)


# ------------------------------------------------------------------------------------------------ each mechanism alone
A, M = BU.attention_layer, BU.mlstm_layer
SINGLE = {
    "filter_only": BU.model_config([A(every=0)]),
    "filter_of_five_taps": BU.model_config([A(conv=5, every=0, heads=3, kv_heads=3, dim=8, vdim=40)]),
    "temperature_only": BU.model_config([A(conv=0, every=4, coef=1.5)]),
    "temperature_every_position": BU.model_config([A(conv=2, every=1, coef=0.3)]),
    "biases_only": BU.model_config([A(conv=0, every=0)]),
    "values_blended": BU.model_config([A(v_mix=True), A(v_mix=True, conv=2), A(), A(v_mix=True, every=0)]),
    "tiled_sizes": BU.model_config([A(dim=32, vdim=32, heads=6, kv_heads=2)]),
    "tiled_sizes_many_heads": BU.model_config([A(dim=16, vdim=16, heads=20, kv_heads=1, scale=0.2)]),
    "tma_sizes_blended": BU.model_config([A(dim=64, vdim=64, heads=4, kv_heads=2, scale=0.12, v_mix=True), A(dim=64, vdim=64, heads=2, kv_heads=2, scale=0.12, v_mix=True)]),
    "tma_sizes_128": BU.model_config([A(dim=128, vdim=128, heads=2, kv_heads=1, scale=0.09)], width=64),
    "values_narrower_than_keys": BU.model_config([A(dim=64, vdim=16, heads=4, kv_heads=2, scale=0.11, v_mix=True), A(dim=64, vdim=16, heads=2, kv_heads=2, scale=0.11, v_mix=True)]),
    "values_wider_than_keys": BU.model_config([A(dim=32, vdim=64, heads=4, kv_heads=1, scale=0.2)]),
    "values_three_times_the_keys": BU.model_config([A(dim=16, vdim=48, heads=2, kv_heads=2, conv=2)]),
    "matrix_memory": BU.model_config([M()]),
    "matrix_memory_wide_keys": BU.model_config([M(heads=1, dim=70, vdim=40, cap=4.0)]),
    "matrix_memory_many_heads": BU.model_config([M(heads=5, dim=8, vdim=8, cap=30.0)], width=40),
    "matrix_memory_256_keys": BU.model_config([M(heads=1, dim=256, vdim=33)]),
    "experts": BU.model_config([M(heads=1, dim=8, vdim=8, mlp=BU.moe())]),
    "experts_one_group": BU.model_config([M(heads=1, dim=8, vdim=8, mlp=BU.moe(count=0, top=3))]),
    "experts_groups_of_one": BU.model_config([M(heads=1, dim=8, vdim=8, mlp=BU.moe(experts=5, count=5, keep=3, top=2))]),
    "experts_top_one": BU.model_config([M(heads=1, dim=8, vdim=8, mlp=BU.moe(experts=8, count=2, keep=1, top=1, scale=0.6))]),
    "experts_all_chosen": BU.model_config([M(heads=1, dim=8, vdim=8, mlp=BU.moe(experts=4, count=2, keep=2, top=4))]),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism(name, dtype, tmp_path):
    cfg = SINGLE[name]
    folder = BU.make_folder(tmp_path, cfg, name, seed=5)
    ids = BU.tokens(cfg, 61, seed=1)
    want = BU.plain_logits(folder, ids)
    r = runner_for(folder, dtype)
    mg = BU.router_margins(folder, ids)
    close(run_cut(r, ids, [61]), want, dtype, f"{name}, whole prompt", mg)
    close(run_cut(r, ids, [29] + [1] * 32), want, dtype, f"{name}, 29 tokens then one by one", mg)
    close(run_cut(r, ids, [2, 3, 2, 11, 2, 17, 1, 2, 21]), want, dtype, f"{name}, portions", mg)


# ------------------------------------------------------------------------------------------------ whole models, every cutting
MODELS = {"P": BU.MODEL_P, "Q": BU.MODEL_Q, "R": BU.MODEL_R}


@pytest.fixture(scope="module", params=[(m, d) for m in sorted(MODELS) for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def model(request, tmp_path_factory):
    name, dtype = request.param
    folder = BU.make_folder(tmp_path_factory.mktemp(f"bifusun_{name}_{dtype}"), MODELS[name], name, seed=11)
    return name, dtype, folder, runner_for(folder, dtype, page_size=8, num_pages=40)


def test_whole_prompt_equals_token_by_token(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    for n in (1, 2, 9, 75):
        ids = BU.tokens(cfg, n, seed=2)
        want = BU.plain_logits(folder, ids)
        mg = BU.router_margins(folder, ids)
        close(run_cut(r, ids, [n]), want, dtype, f"{name}: whole prompt of {n}", mg)
        close(run_cut(r, ids, [1] * n), want, dtype, f"{name}: {n} tokens one by one", mg)


def test_portions_of_several_sizes(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = BU.tokens(cfg, 120, seed=3)
    want = BU.plain_logits(folder, ids)
    for cuts in ([2] * 60, [7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 8, 18], [33, 33, 33, 21], [119, 1]):
        close(run_cut(r, ids, cuts), want, dtype, f"{name}: portions {cuts[:4]}...", BU.router_margins(folder, ids))


def test_long_decoding(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = BU.tokens(cfg, 260, seed=4)
    close(run_cut(r, ids, [4] + [1] * 256), BU.plain_logits(folder, ids), dtype, f"{name}: 256 decoded tokens", BU.router_margins(folder, ids))


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model):
    """Four live requests at most, 40 pages of 8 tokens: the lengths below need far more over time, so pages and state slots come
    back and are handed out again; every request's logits equal those it gets alone."""
    name, dtype, folder, r = model
    cfg = MODELS[name]
    lengths = [97, 3, 64, 30, 1, 121, 45, 18, 70]
    todo = [(f"q{i}", BU.tokens(cfg, n, seed=20 + i)) for i, n in enumerate(lengths)]
    live, got, used_slots = {}, {}, []
    step = 0
    while todo or live:
        while todo and len(live) < 4:
            key, ids = todo.pop(0)
            rc = r.cache.open(key)
            assert rc is not None
            used_slots.append(rc.state_slot)
            live[key] = [rc, ids, 0]
        entries, order = [], []
        for k, (key, (rc, ids, at)) in enumerate(sorted(live.items())):
            if (step + k) % 3 == 0 and at > 0 and len(live) > 1:
                continue                                   # a request may sit a step out
            left = len(ids) - at
            c = 1 if at >= len(ids) // 2 else min(left, [2, 5, 16, 3, 29][(step + k) % 5])   # portions first, then single tokens
            if r.cache.free_pages * 8 < c + 8:
                continue
            entries.append(feed(r, rc, ids, at, at + c))
            order.append((key, c))
        if not entries:   # everything sat out or lacked pages: let the longest go on alone
            key, (rc, ids, at) = max(live.items(), key=lambda kv: kv[1][2])
            entries, order = [feed(r, rc, ids, at, at + 1)], [(key, 1)]
        out = r.step(entries)
        row = 0
        for key, c in order:
            got.setdefault(key, []).append(out[row:row + c])
            row += c
            live[key][2] += c
            if live[key][2] == len(live[key][1]):
                r.cache.close(live.pop(key)[0])
        step += 1
    r.check()
    r.cache.check()
    assert len(used_slots) > len(set(used_slots)), "no state slot was used twice"
    for i, n in enumerate(lengths):
        ids = BU.tokens(cfg, n, seed=20 + i)
        close(torch.cat(got[f"q{i}"]), BU.plain_logits(folder, ids), dtype, f"{name}: request {i} of {n} tokens in the mix", BU.router_margins(folder, ids))


def test_far_keys_and_long_memory(tmp_path):
    """A prompt of 700 tokens with peaked attention and forget gates that lean open: the last logits rest on keys and state from
    hundreds of tokens back, across dozens of pages; in 32-bit a lost one shows."""
    cfg = BU.MODEL_Q
    folder = BU.make_folder(tmp_path, cfg, "far", seed=3, sharpen=16.0)
    ids = BU.tokens(cfg, 700, seed=9)
    want = BU.plain_logits(folder, ids)
    r = runner_for(folder, "float32", page_size=16, num_pages=50)
    close(run_cut(r, ids, [650] + [1] * 50), want, "float32", "650 tokens, then 50 one by one")
    close(run_cut(r, ids, [255, 257, 2, 186]), want, "float32", "portions that end beside page borders")
    b = runner_for(folder, "bfloat16", page_size=16, num_pages=50)
    close(run_cut(b, ids, [650] + [1] * 50), want, "bfloat16", "bfloat16: 650 tokens, then 50 one by one", BU.router_margins(folder, ids))


def test_replay_program_runs_the_design(tmp_path):
    cfg = BU.MODEL_R
    folder = BU.make_folder(tmp_path, cfg, "R", seed=11)
    ids_a, ids_b = BU.tokens(cfg, 50, seed=7), BU.tokens(cfg, 9, seed=8)
    r = Replay(folder, "float32", tmp_path / "out", max_tokens=128, page_size=16)
    got = r.step([{"id": "a", "tokens": ids_a[:31], "want": [0, 30]}, {"id": "b", "tokens": ids_b[:2], "want": []}])
    close(got, BU.plain_logits(folder, ids_a)[[0, 30]], "float32", "replay: first step")
    assert r.step([{"id": "b", "tokens": ids_b[2:8], "want": []}]) is None
    got = r.step([{"id": "a", "tokens": ids_a[31:], "want": [18]}, {"id": "b", "tokens": ids_b[8:], "want": [0]}], end=["a", "b"])
    close(got, torch.stack([BU.plain_logits(folder, ids_a)[49], BU.plain_logits(folder, ids_b)[8]]), "float32", "replay: last step")
    assert r.close() == 0


# ------------------------------------------------------------------------------------------------ greedy generation through the engine
@pytest.mark.parametrize("graphs", [False, True])
@pytest.mark.parametrize("which", ["P", "Q"])
def test_greedy_generation_through_the_engine(which, graphs, tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = MODELS[which]
    folder = BU.make_folder(tmp_path, cfg, which, seed=11)
    plain_cfg, w = BP.read_model(folder, torch.float64)
    prompts = [BU.tokens(cfg, n, seed=30 + n) for n in (5, 23, 1, 40, 12, 9)]
    engine = Engine(folder, EngineSettings(dtype="float32", num_pages=48, page_size=8, max_running=3, max_step_tokens=32, prefill_chunk=16,
                                           cuda_graphs=graphs))
    done = engine.generate(prompts, SamplingParams(max_tokens=14, ignore_eos=True))
    compared = 0
    for prompt, c in zip(prompts, done):
        want, gaps = BP.greedy(plain_cfg, w, prompt, 14)
        for a, b, gap in zip(c.token_ids, want, gaps):
            if gap < 1e-3:
                break          # a near-tie: from here on the two may differ for no fault
            assert a == b, f"prompt of {len(prompt)}: generated {c.token_ids}, the plain implementation {want}"
            compared += 1
    assert compared >= 60
    if graphs:
        assert engine.counters["graph_steps"] > 0


def test_command_line_generates_with_the_design(tmp_path):
    import json
    import subprocess
    import sys

    import util

    cfg = BU.MODEL_R
    folder = BU.make_folder(tmp_path, cfg, "R", seed=14)
    plain_cfg, w = BP.read_model(folder, torch.float64)
    cmd = [sys.executable, "-m", "oxr_inference_b200", "--model", str(folder), "--prompt-ids", "5,17,3", "--prompt-ids", "9 8 7 6 11 2",
           "--max-tokens", "6", "--dtype", "float32", "--num-pages", "32", "--max-running", "4", "--ignore-eos"]
    res = subprocess.run(cmd, capture_output=True, text=True, cwd=str(util.ROOT), timeout=600)
    assert res.returncode == 0, res.stderr
    rows = [json.loads(line) for line in res.stdout.strip().splitlines() if line.startswith("{")]
    for row, prompt in zip(rows, ([5, 17, 3], [9, 8, 7, 6, 11, 2])):
        want, gaps = BP.greedy(plain_cfg, w, prompt, 6)
        for a, b, gap in zip(row["token_ids"], want, gaps):
            if gap < 1e-3:
                break
            assert a == b, f"the command line generated {row['token_ids']}, the plain implementation {want}"
    assert len(rows) == 2


def test_bfloat16_generation_with_graphs_equals_eager(tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = BU.MODEL_Q
    folder = BU.make_folder(tmp_path, cfg, "Q", seed=12)
    prompts = [BU.tokens(cfg, n, seed=40 + n) for n in (17, 3, 30, 8)]
    out = []
    for graphs in (False, True):
        engine = Engine(folder, EngineSettings(dtype="bfloat16", num_pages=48, page_size=16, max_running=4, cuda_graphs=graphs))
        out.append([c.token_ids for c in engine.generate(prompts, SamplingParams(max_tokens=10, ignore_eos=True))])
    assert out[0] == out[1]


# ------------------------------------------------------------------------------------------------ the kernels against their formulas
SHORT_STEPS = ([11, 7], ([1, 2], [3, 1], [1, 1], [1, 3], [1, 0], [4, 0]))     # with the transposed filter, steps of single tokens roll their tails inline
LONG_STEPS = ([70, 50, 9], ([41, 19, 4], [29, 31, 5]))   # steps of 64 and 65 tokens: the kernel that walks over neighbouring tokens; borders inside a walk


@pytest.mark.parametrize("steps", [SHORT_STEPS, LONG_STEPS], ids=["short", "long"])
@pytest.mark.parametrize("transposed", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [0, 1, 2, 3, 4, 5])
def test_filter_kernel_with_tails_across_steps(dtype, taps, transposed, steps):
    """Two requests whose tokens arrive in unequal portions (down to one token, fewer than the filter's taps): biases, filter,
    temperature, blend, cache rows and the rolled tails against the formulas over the whole sequences. With the filter also handed over
    transposed, bfloat16 runs the 16-byte kernel."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(taps)
    H, KV, DK, DV, P = 3, 1, 8, 16, 4
    cq, ck, cv = H * DK, KV * DK, KV * DV
    C = cq + ck + cv
    lens, step_list = steps
    proj = [torch.randn(n, C + 8, generator=g).to(dtype) for n in lens]          # 8 columns that are not ours
    first = [torch.randn(n, cv, generator=g).to(dtype) for n in lens]
    conv = torch.randn(C, taps, generator=g) if taps else None
    bias = torch.randn(C, generator=g)
    lam, coef, every = 0.3, 0.7, 3
    want = []
    for u, f in zip(proj, first):
        y = u[:, :C].double() + bias.double()
        if taps:
            y = BP.short_convolution(y, conv.double())
        q = y[:, :cq] * BP.query_temperature(len(u), coef, every, torch.float64)[:, None]
        v = (1 - lam) * y[:, cq + ck:] + lam * f.double()
        want.append((q, y[:, cq:cq + ck], v))
    per = (max(lens) + P - 1) // P          # pages a request takes
    pages = per * len(lens)
    k_pool = torch.zeros(pages, P, KV, DK, dtype=dtype, device=DEV)
    v_pool = torch.zeros(pages, P, KV, DV, dtype=dtype, device=DEV)
    tails = torch.zeros(len(lens) + 1, max(1, C * max(taps - 1, 0)) + 2, device=DEV)   # slot rows longer than the tail: a strided view
    status = ops.new_status(DEV)
    slot_of = [[(r * per + j // P) * P + j % P for j in range(n)] for r, n in enumerate(lens)]
    at = [0] * len(lens)
    got_q = [[] for _ in lens]
    top_slot = len(lens)
    for cuts in step_list:
        rows, pos, req, cu, slots, firsts, order = [], [], [], [0], [], [], []
        for r, c in enumerate(cuts):
            if c == 0:
                continue
            rows.append(proj[r][at[r]:at[r] + c])
            firsts.append(first[r][at[r]:at[r] + c])
            pos += list(range(at[r], at[r] + c))
            req += [len(order)] * c
            slots += slot_of[r][at[r]:at[r] + c]
            cu.append(cu[-1] + c)
            order.append((r, c))
            at[r] += c
        i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
        q, kept = ops.conv_qkv_store(torch.cat(rows).to(DEV), cq, ck, cv, conv=None if conv is None else conv.to(DEV), bias=bias.to(DEV),
                                     conv_t=None if conv is None or not transposed else conv.t().contiguous().to(DEV), single_tokens=max(cuts) == 1,
                                     tails=tails[:, :C * max(taps - 1, 0)] if taps > 1 else None, k_pool=k_pool, v_pool=v_pool, slots=i32(slots),
                                     req_of_token=i32(req), cu_q=i32(cu), state_slots=i32([top_slot - r for r, _ in order]), positions=i32(pos),
                                     n_requests=len(order), status=status, temp_coef=coef, temp_every=every,
                                     blend=torch.tensor([lam], device=DEV), first=torch.cat(firsts).to(DEV), keep_values=True)
        row = 0
        for r, c in order:
            got_q[r].append(q[row:row + c].float().cpu())
            row += c
    ops.check_status(status)
    assert at == lens
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    for r, n in enumerate(lens):
        wq, wk, wv = want[r]
        scale = max(1.0, float(wq.abs().max()))
        assert (torch.cat(got_q[r]) - wq).abs().max() <= tol * scale, "queries"
        k_rows = k_pool.view(-1, ck)[slot_of[r]].float().cpu()
        v_rows = v_pool.view(-1, cv)[slot_of[r]].float().cpu()
        assert (k_rows - wk).abs().max() <= tol * max(1.0, float(wk.abs().max())), "cached keys"
        assert (v_rows - wv).abs().max() <= tol * max(1.0, float(wv.abs().max())), "cached values"
        if taps > 1:
            tail = tails[top_slot - r, :C * (taps - 1)].view(C, taps - 1).cpu()
            last = (proj[r][:, :C].float() + bias)[-(taps - 1):].T
            assert torch.allclose(tail, last, atol=1e-6), "the tail holds the last projected values, oldest first"
    assert torch.all(tails[:, C * max(taps - 1, 0):] == 0), "nothing was written beyond a slot's tail"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_filter_kernel_writes_into_heads_wider_than_its_own(dtype):
    """Pools and queries whose heads are wider than the projection's (keys and values padded to one size): every head's entries land at
    the head's start and the padding is left alone."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(8)
    H, KV, DK, DV, P, n = 4, 2, 8, 16, 4, 6
    cq, ck, cv = H * DK, KV * DK, KV * DV
    proj = torch.randn(n, cq + ck + cv, generator=g).to(dtype)
    k_pool = torch.full((3, P, KV, 24), 7.0, dtype=dtype, device=DEV)
    v_pool = torch.full((3, P, KV, 24), 7.0, dtype=dtype, device=DEV)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    slots = [5, 6, 7, 8, 0, 1]
    q, _ = ops.conv_qkv_store(proj.to(DEV), cq, ck, cv, conv=None, bias=None, tails=None, k_pool=k_pool, v_pool=v_pool, slots=i32(slots),
                              req_of_token=i32([0] * 4 + [1] * 2), cu_q=i32([0, 4, 6]), state_slots=i32([0, 1]), positions=i32([0, 1, 2, 3, 0, 1]),
                              n_requests=2, status=ops.new_status(DEV), q_head_width=24)
    q = q.view(n, H, 24).cpu()
    assert torch.equal(q[:, :, :DK], proj[:, :cq].view(n, H, DK)) and torch.all(q[:, :, DK:] == 0)
    k_rows, v_rows = k_pool.view(-1, KV, 24)[slots].cpu(), v_pool.view(-1, KV, 24)[slots].cpu()
    assert torch.equal(k_rows[:, :, :DK], proj[:, cq:cq + ck].view(n, KV, DK)) and torch.all(k_rows[:, :, DK:] == 7)
    assert torch.equal(v_rows[:, :, :DV], proj[:, cq + ck:].view(n, KV, DV)) and torch.all(v_rows[:, :, DV:] == 7)
    assert (k_pool == 7).sum() == k_pool.numel() - n * ck


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,DK,DV", [(2, 16, 24), (1, 70, 40), (3, 256, 8), (4, 33, 65)])
def test_matrix_memory_kernel(dtype, H, DK, DV):
    """The recurrence kernel in two steps (the second continues from the state the first left; two requests of unequal length) against
    the recurrence written out in float64."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(DK)
    lens, cap = [13, 6], 7.0
    width = 2 * H * DK + H * DV
    size = H * DK * DV + H * DK + H
    state = torch.zeros(4, size + 3, device=DEV)
    outs = {0: [], 1: []}
    seqs = []
    for n in lens:
        proj = torch.randn(n, width + 4, generator=g).to(dtype)
        gates = torch.randn(n, 2 * H, generator=g) * 4
        seqs.append((proj, gates))
    bias = torch.randn(2 * H, generator=g)
    i32 = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)  # noqa: E731
    for lo, hi in ((0, 5), (5, 13)):
        rows, gate_rows, cu, order = [], [], [0], []
        for r, (proj, gates) in enumerate(seqs):
            a, b = min(lo, lens[r]), min(hi, lens[r])
            if b > a:
                rows.append(proj[a:b])
                gate_rows.append(gates[a:b])
                cu.append(cu[-1] + b - a)
                order.append((r, b - a))
        y = ops.mlstm_scan(torch.cat(rows).to(DEV), 4, 4 + H * DK, 4 + 2 * H * DK, torch.cat(gate_rows).to(DEV), bias.to(DEV), heads=H, key_dim=DK,
                           value_dim=DV, cap=cap, q_scale=DK ** -0.5, state=state[:, :size], cu_q=i32(cu), state_slots=i32([3 - r for r, _ in order]),
                           n_requests=len(order))
        row = 0
        for r, c in order:
            outs[r].append(y[row:row + c].cpu())
            row += c
    for r, (proj, gates) in enumerate(seqs):
        n = lens[r]
        p = proj.double()
        q = p[:, 4:4 + H * DK].view(n, H, DK) * DK ** -0.5
        k = p[:, 4 + H * DK:4 + 2 * H * DK].view(n, H, DK)
        v = p[:, 4 + 2 * H * DK:4 + 2 * H * DK + H * DV].view(n, H, DV)
        z = gates.double() + bias.double()
        a = cap * torch.tanh(z[:, :H] / cap)
        b = torch.nn.functional.logsigmoid(cap * torch.tanh(z[:, H:] / cap))
        S, nv, m = torch.zeros(H, DK, DV, dtype=torch.float64), torch.zeros(H, DK, dtype=torch.float64), torch.zeros(H, dtype=torch.float64)
        want = torch.zeros(n, H, DV, dtype=torch.float64)
        for t in range(n):
            m_new = torch.maximum(b[t] + m, a[t])
            keep, take = torch.exp(b[t] + m - m_new), torch.exp(a[t] - m_new)
            S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
            nv = keep[:, None] * nv + take[:, None] * k[t]
            m = m_new
            den = torch.maximum((nv * q[t]).sum(-1).abs(), torch.exp(-m)) + 1e-6
            want[t] = torch.einsum("hdv,hd->hv", S, q[t]) / den[:, None]
        got = torch.cat(outs[r]).view(n, H, DV).double()
        assert (got - want).abs().max() <= 2e-4 * max(1.0, float(want.abs().max())), f"request {r}"
        left = state[3 - r, :size].cpu().double()
        assert (left[:H * DK * DV].view(H, DK, DV) - S).abs().max() <= 1e-4 * max(1.0, float(S.abs().max()))
        assert (left[H * DK * DV:H * DK * DV + H * DK].view(H, DK) - nv).abs().max() <= 1e-4 * max(1.0, float(nv.abs().max()))
        assert (left[-H:] - m).abs().max() <= 1e-5
    assert torch.all(state[:, size:] == 0) and torch.all(state[:2] == 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm_with_gate(dtype):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(2)
    n, H, DV = 9, 3, 40
    y = torch.randn(n, H * DV, generator=g) * 5
    proj = torch.randn(n, 7 + H * DV, generator=g).to(dtype)
    w = 1 + 0.2 * torch.randn(H * DV, generator=g)
    got = ops.head_norm_gate(y.to(DEV), proj.to(DEV), 7, w.to(DEV), H, 1e-5).float().cpu()
    want = BP.rms_norm(y.double().view(n, H, DV), None, 1e-5).view(n, H * DV) * w.double() * torch.sigmoid(proj[:, 7:].double())
    assert (got - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2) * want.abs().max()


@pytest.mark.parametrize("E,top,groups,keep", [(15, 4, 5, 3), (6, 2, 3, 2), (8, 3, 1, 1), (5, 2, 5, 3), (64, 8, 8, 4), (9, 1, 3, 1), (4, 4, 2, 2), (256, 32, 32, 9),
                                               (320, 6, 64, 20), (66, 3, 33, 4)])
def test_router_kernel(E, top, groups, keep):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(E * 100 + top)
    n = 300
    z = torch.randn(n, E, generator=g) * 3
    gate, ids, wts = ops.route(z.to(DEV), top=top, groups=groups, keep=keep, scale=1.75)
    r = {"experts": E, "top": top, "scale": 1.75}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    chosen, weight = BP.route(z.double(), r)
    dense = torch.zeros(n, E, dtype=torch.float64).scatter_(1, chosen, weight)
    assert (gate.cpu().double() - dense).abs().max() < 1e-5
    assert torch.equal(ids.cpu().sort(1).values.long(), chosen.sort(1).values)
    assert (torch.zeros(n, E).scatter_(1, ids.cpu().long(), wts.cpu()) - gate.cpu()).abs().max() == 0
    assert ((gate > 0).sum(1) == top).all()


@pytest.mark.parametrize("ff", [12, 16])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_experts_activation(dtype, ff):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(3)
    n, E = 11, 5
    u = torch.randn(n, E * ff, generator=g).to(dtype)
    gate = torch.rand(n, E, generator=g) * (torch.rand(n, E, generator=g) > 0.5)
    got = ops.gated_relu2(u.to(DEV), gate.to(DEV), ff).float().cpu()
    want = gate.double().repeat_interleave(ff, 1) * torch.relu(u.double()) ** 2
    assert (got - want).abs().max() <= (1e-6 if dtype == torch.float32 else 1e-2) * max(1.0, float(want.abs().max()))
    assert torch.all(got[gate.repeat_interleave(ff, 1) == 0] == 0)


def test_bias_and_scale_in_place():
    from oxr_inference_b200 import ops

    x = torch.randn(7, 10)
    row = torch.randn(10)
    for dtype in (torch.float32, torch.bfloat16):
        got = ops.add_bias_(x.to(dtype).to(DEV), row.to(DEV)).float().cpu()
        assert (got - (x.to(dtype).float() + row)).abs().max() <= (1e-6 if dtype == torch.float32 else 3e-2)
    got = ops.scale_(x.to(DEV).clone(), 0.37).cpu()
    assert torch.equal(got, x * torch.tensor(0.37))


# ------------------------------------------------------------------------------------------------ keys that must, or must not, be seen
def _paged(keys, values, page_size, dtype, spare=3):
    """Scatter rows [ctx, KV, D] into pools with shuffled pages; returns pools, block table row."""
    ctx = keys.shape[0]
    n_pages = (ctx + page_size - 1) // page_size
    perm = torch.randperm(n_pages + spare, generator=torch.Generator().manual_seed(ctx))[:n_pages]
    k_pool = torch.zeros((n_pages + spare, page_size, *keys.shape[1:]), dtype=dtype)
    v_pool = torch.zeros((n_pages + spare, page_size, *values.shape[1:]), dtype=dtype)
    for j in range(ctx):
        k_pool[perm[j // page_size], j % page_size] = keys[j]
        v_pool[perm[j // page_size], j % page_size] = values[j]
    return k_pool.to(DEV), v_pool.to(DEV), perm.to(torch.int32).view(1, -1).to(DEV)


def _plain_attention(q, keys, values, positions, scale):
    n, H, _ = q.shape
    KV = keys.shape[1]
    out = torch.zeros(n, H, values.shape[2], dtype=torch.float64)
    for t, p in enumerate(positions):
        for h in range(H):
            g = h // (H // KV)
            s = (keys[:p + 1, g].double() @ q[t, h].double()) * scale
            out[t, h] = torch.softmax(s, 0) @ values[:p + 1, g].double()
    return out


@pytest.mark.parametrize("case,D", [("far_key", 64), ("page_borders", 64), ("first_tokens", 64), ("far_key", 128), ("page_borders", 32), ("first_tokens", 128)])
def test_marked_keys_through_the_kernels_of_plain_causal_attention(case, D):
    """One key is made to stand out (its score beats all others by far), so the output is that key's value when it is seen: a page read
    wrongly, a key lost far back or at a sequence's start changes the output by its whole size. Through the kernels that serve keys
    and values of one size in bfloat16 (with TMA maps where the sizes allow), as a portion, as single tokens, and mixed."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(11)
    H, KV, P, ctx = 4, 2, 16, 700
    marked = {"far_key": [3, 77], "page_borders": [15, 16, 17, 31, 32, 255, 256, 511, 512], "first_tokens": [0, 1]}[case]
    keys = torch.randn(ctx, KV, D, generator=g) * 0.3
    values = torch.randn(ctx, KV, D, generator=g)
    direction = torch.randn(D, generator=g)
    direction /= direction.norm()
    for j in marked:
        keys[j] += 6 * direction
    keys, values = keys.to(torch.bfloat16).float(), values.to(torch.bfloat16).float()
    k_pool, v_pool, table = _paged(keys, values, P, torch.bfloat16)
    k5, v5 = k_pool.unsqueeze(0).contiguous(), v_pool.unsqueeze(0).contiguous()
    maps = ops.make_kv_maps(k5, v5, P)
    assert (maps is not None) == (D % 64 == 0)
    k_pool, v_pool = k5[0], v5[0]
    status = ops.new_status(DEV)
    specs = ops.attention_tile_specs(H, KV, D, torch.bfloat16, P)

    def run(q_lens, ctx_lens):
        n = sum(q_lens)
        q = (torch.randn(n, H, D, generator=g) * 0.3 + 4 * direction).to(torch.bfloat16)
        cu = [0]
        for x in q_lens:
            cu.append(cu[-1] + x)
        tiles = {}
        for spec in specs:
            req, tok0 = [], []
            for r, x in enumerate(q_lens):
                if spec[1] <= x <= spec[2]:
                    for t0 in range(0, x, spec[0]):
                        req.append(r)
                        tok0.append(t0)
            tiles[spec] = (torch.tensor(req + [0], dtype=torch.int32, device=DEV), torch.tensor(tok0 + [0], dtype=torch.int32, device=DEV), len(req))
        out = ops.paged_attention(q.to(DEV), k_pool, v_pool, tiles=tiles, cu_q=torch.tensor(cu, dtype=torch.int32, device=DEV),
                                  ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=DEV), block_table=table.repeat(len(q_lens), 1).contiguous(),
                                  page_size=P, scale=0.5, window=0, kv_len_bound=max(ctx_lens), status=status, kv_maps=maps)
        ops.check_status(status)
        at = 0
        for x, c in zip(q_lens, ctx_lens):
            want = _plain_attention(q[at:at + x].float(), keys, values, list(range(c - x, c)), 0.5)
            err = (out[at:at + x].float().cpu() - want).abs().max()
            assert err <= 2e-2 * max(1.0, want.abs().max()), f"{case}: request of {x} new tokens ending at {c}: off by {err:.2e}"
            at += x

    run([300, 5, 70], [700, 18, 300])
    run([1] * 9, [1, 2, 16, 17, 33, 256, 257, 513, 700])
    run([1, 33, 2, 1], [700, 290, 2, 1])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_marked_keys_with_values_of_another_size(dtype):
    """The same through the kernel that takes keys and values of different sizes (the 32-bit path of every size)."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(5)
    H, KV, DK, DV, P, ctx = 4, 2, 16, 24, 8, 700
    marked, queries = [0, 3, 7, 8, 63, 64, 511, 512], [0, 1, 3, 7, 8, 9, 64, 65, 512, 513, 699]
    keys = torch.randn(ctx, KV, DK, generator=g) * 0.3
    values = torch.randn(ctx, KV, DV, generator=g)
    direction = torch.randn(DK, generator=g)
    direction /= direction.norm()
    for j in marked:
        keys[j] += 6 * direction
    q = torch.randn(len(queries), H, DK, generator=g) * 0.3 + 4 * direction
    q, keys, values = (t.to(dtype).float() for t in (q, keys, values))
    want = _plain_attention(q, keys, values, queries, 0.5)
    k_pool, v_pool, table = _paged(keys, values, P, dtype)
    status = ops.new_status(DEV)
    n = len(queries)
    pos = torch.tensor(queries, dtype=torch.int32, device=DEV)
    for name, req, tab in (("portion", torch.zeros(n, dtype=torch.int32, device=DEV), table),
                           ("single tokens", torch.arange(n, dtype=torch.int32, device=DEV), table.repeat(n, 1).contiguous())):
        out = ops.attention_rows(q.to(dtype).view(n, H * DK).to(DEV), H, k_pool, v_pool, value_dim=DV, positions=pos, req_of_token=req,
                                 block_table=tab, scale=0.5, status=status)
        err = (out.float().cpu().view(n, H, DV) - want).abs().max()
        assert err <= (2e-5 if dtype == torch.float32 else 2e-2) * max(1.0, want.abs().max()), f"{name}: off by {err:.2e}"
    ops.check_status(status)
    shifted = _plain_attention(q, keys, values, [max(0, p - 1) for p in queries], 0.5)
    assert (shifted - want).abs().max() > 0.1


# ------------------------------------------------------------------------------------------------ experts over the rows that chose them
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,top,groups,keep,n", [(6, 2, 3, 2, 37), (15, 4, 5, 3, 300), (5, 1, 1, 1, 64), (8, 3, 2, 1, 9)])
def test_experts_grouped_by_expert_equal_the_single_product_and_the_plain_sum(dtype, E, top, groups, keep, n):
    """The form for many tokens (pairs ordered by expert, each expert over its own rows, weighted sum) against the form for few (one
    product over all experts) and against the plain sum; some experts get no row at all."""
    from oxr_inference_b200 import ops
    from oxr_inference_b200.parts.base import Runtime
    from oxr_inference_b200.parts.experts import RoutedExperts

    g = torch.Generator().manual_seed(E * 10 + top)
    width, ff = 48, 16
    rt = Runtime(device=torch.device(DEV), dtype=dtype, max_positions=1, status=ops.new_status(DEV))
    part = RoutedExperts(rt, hidden_size=width, intermediate_size=ff, experts=E, top=top, groups=groups, keep=keep, scale=1.5, grouped_min_rows=1)
    w = {name: (torch.randn(info.shape, generator=g) * (0.8 if name == "router" else 0.2)).to(torch.bfloat16) for name, info in part.parameters().items()}
    w["router"][E - 1] -= 3.0          # the last expert is hardly ever chosen
    for name, t in w.items():
        part.assign(name, t)
    h = torch.randn(n, width, generator=g).to(dtype)
    grouped = part.forward(h.to(DEV)).float().cpu()
    part.grouped_min_rows = 0
    single = part.forward(h.to(DEV)).float().cpu()
    r = {"experts": E, "top": top, "scale": 1.5}
    if groups > 1:
        r["groups"] = {"count": groups, "keep": keep}
    plain_w = {"mlp." + k: v.double() for k, v in w.items()}
    want = BP.routed_experts(h.double(), plain_w, "mlp.", {"router": r})
    margin = BP.route_margin(h.double() @ plain_w["mlp.router"].T, r)
    clear = margin > (1e-4 if dtype == torch.float32 else 2e-2)
    assert clear.float().mean() > 0.5
    tol = (1e-4 if dtype == torch.float32 else 3e-2) * float(want.abs().max())
    assert (grouped - want)[clear].abs().max() <= tol
    assert (single - want)[clear].abs().max() <= tol


def test_expert_sort_gather_and_combine():
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(4)
    n, top, E, width = 150, 3, 7, 24
    ids = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(n)]).to(torch.int32)
    counts, order, place, _ = ops.expert_sort(ids.to(DEV), E)
    counts, order, place = counts.cpu(), order.cpu().long(), place.cpu().long()
    assert torch.equal(counts.long(), torch.bincount(ids.view(-1).long(), minlength=E))
    assert torch.equal(order[place], torch.arange(n * top))
    sorted_experts = ids.view(-1)[order]
    assert torch.all(sorted_experts[1:] >= sorted_experts[:-1])
    x = torch.randn(n, width, generator=g).to(torch.bfloat16)
    rows = ops.gather_rows(x.to(DEV), order.to(torch.int32).to(DEV), top).cpu()
    assert torch.equal(rows, x[order // top])
    y = torch.randn(n * top, width, generator=g)
    wts = torch.rand(n, top, generator=g)
    got = ops.combine_rows(y.to(DEV), place.to(torch.int32).to(DEV), wts.to(DEV)).cpu()
    want = (y[place].view(n, top, width).double() * wts.double()[:, :, None]).sum(1)
    assert (got - want).abs().max() < 1e-5
    # padded: every expert's stretch starts at a multiple of 16 places, the places in between hold -1 and gather zeros
    counts2, order2, place2, tile_group = ops.expert_sort(ids.to(DEV), E, pad=16)
    order2, place2, tile_group = order2.cpu().long(), place2.cpu().long(), tile_group.cpu().long()
    assert torch.equal(counts2.cpu(), counts.to(torch.int32)) and order2.numel() % 16 == 0 and order2.numel() >= n * top + E * 15
    assert torch.equal(order2[place2], torch.arange(n * top))
    starts = torch.cat([torch.zeros(1, dtype=torch.long), ((counts + 15) // 16 * 16).cumsum(0)])
    for e in range(E):
        stretch = order2[starts[e]:starts[e + 1]]
        assert torch.all(ids.view(-1)[stretch[:counts[e]]] == e) and torch.all(stretch[counts[e]:] == -1)
        assert torch.all(tile_group[starts[e] // 16:starts[e + 1] // 16] == e)
    assert torch.all(order2[starts[-1]:] == -1)
    rows2 = ops.gather_rows(x.to(DEV), order2.to(torch.int32).to(DEV), top).cpu()
    assert torch.equal(rows2[order2 >= 0], x[order2[order2 >= 0] // top]) and torch.all(rows2[order2 < 0] == 0)


@pytest.mark.parametrize("n_in,n_out,groups", [(64, 48, 3), (256, 200, 5), (72, 16, 1)])
def test_grouped_product(n_in, n_out, groups):
    """Rows ordered by the matrix they multiply, each group padded to whole tiles: one launch against the products group by group."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(n_in)
    tiles = [2, 0, 1, 3, 1][:groups]
    group_of_tile = [e for e, c in enumerate(tiles) for _ in range(c)] + [-1]         # a last tile nobody uses: not computed
    rows = len(group_of_tile) * ops.GROUP_TILE_ROWS
    x = torch.randn(rows, n_in, generator=g).to(torch.bfloat16)
    w = (torch.randn(groups * n_out, n_in, generator=g) * 0.2).to(torch.bfloat16)
    got = ops.grouped_linear(x.to(DEV), w.to(DEV), torch.tensor(group_of_tile, dtype=torch.int32, device=DEV), n_out).float().cpu()
    squared = ops.grouped_linear(x.to(DEV), w.to(DEV), torch.tensor(group_of_tile, dtype=torch.int32, device=DEV), n_out, relu2=True).float().cpu()
    for t, e in enumerate(group_of_tile):
        lo = t * ops.GROUP_TILE_ROWS
        if e < 0:
            continue          # not computed, not to be read
        want = x[lo:lo + ops.GROUP_TILE_ROWS].double() @ w[e * n_out:(e + 1) * n_out].double().T
        assert (got[lo:lo + ops.GROUP_TILE_ROWS] - want).abs().max() <= 2e-2 * want.abs().max(), f"tile {t} of group {e}"
        assert (squared[lo:lo + ops.GROUP_TILE_ROWS] - torch.relu(want) ** 2).abs().max() <= 2e-2 * (want.abs().max() ** 2), f"tile {t}: relu squared"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_whole_model_with_experts_grouped_from_few_rows_on(dtype, tmp_path, monkeypatch):
    """A whole model whose feed-forwards take the grouped form from 8 tokens on: whole prompt, portions on both sides of that limit, and
    two requests in one step."""
    from oxr_inference_b200.parts.experts import RoutedExperts

    monkeypatch.setattr(RoutedExperts, "GROUPED_MIN_ROWS", 8)
    cfg = BU.MODEL_P
    folder = BU.make_folder(tmp_path, cfg, "P", seed=13)
    ids = BU.tokens(cfg, 90, seed=6)
    want, mg = BU.plain_logits(folder, ids), BU.router_margins(folder, ids)
    r = runner_for(folder, dtype)
    close(run_cut(r, ids, [90]), want, dtype, "whole prompt", mg)
    close(run_cut(r, ids, [7, 8, 9, 30, 1, 1, 34]), want, dtype, "portions", mg)
    other = BU.tokens(cfg, 20, seed=7)
    a, b = r.cache.open("a"), r.cache.open("b")
    got = r.step([feed(r, a, ids, 0, 50), feed(r, b, other, 0, 20)])
    close(got[:50], want[:50], dtype, "two requests in one step: the first", mg[:50])
    close(got[50:], BU.plain_logits(folder, other), dtype, "two requests in one step: the second", BU.router_margins(folder, other))
    r.cache.close(a)
    r.cache.close(b)
