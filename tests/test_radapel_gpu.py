"""Radapel on the GPU against the plain statement in ``tests/plain/radapel_plain.py``: each mechanism alone, whole prompts against
token-by-token decoding, portions down to two tokens, batches of unequal requests, pages and state slots that are used again,
keys at page borders and at the edges of chunks, the sink, long decoding, and greedy generation through the engine."""

import math

import pytest
import torch

import radapel_util as RU
from plain import radapel_plain as RP
from util import Replay

pytestmark = pytest.mark.gpu

DEV = "cuda"


def close(got, want, dtype, what):
    got, want = got.float().cpu(), want.float().cpu()
    assert got.shape == want.shape, f"{what}: {tuple(got.shape)} vs {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    d = (got - want) - (got - want).mean(-1, keepdim=True)
    err = d.pow(2).mean(-1).sqrt() / want.std(-1).clamp_min(1e-6)
    limit = 2e-4 if dtype == "float32" else 8e-2
    assert err.max() <= limit, f"{what}: row {int(err.argmax())} is off by {err.max():.2e} of the row's spread (limit {limit:.0e})"


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
SINGLE = {
    "chunked_biased": RU.model_config([RU.attention_layer(mlp=None)]),
    "chunk_smaller_than_page": RU.model_config([RU.attention_layer(heads=6, kv_heads=3, dim=8, vdim=40, chunk=5, bias_rows=4, bias_max=3.5, mlp=None)]),
    "causal_no_bias": RU.model_config([RU.attention_layer(chunk=0, bias_max=0, mlp=None)]),
    "tiled_chunked_biased": RU.model_config([RU.attention_layer(dim=32, vdim=32, mlp=None)]),
    "tiled_causal_biased_many_heads": RU.model_config([RU.attention_layer(heads=20, kv_heads=1, dim=16, vdim=16, chunk=0, scale=0.2, mlp=None)]),
    "tiled_chunk_of_three": RU.model_config([RU.attention_layer(heads=2, kv_heads=2, dim=48, vdim=48, chunk=3, bias_max=0, mlp=None)]),
    "latent_sink": RU.model_config([RU.latent_layer(mlp=None)]),
    "latent_not_tiled": RU.model_config([RU.latent_layer(kv_rank=20, mlp=None)]),
    "latent_nothing_rotated": RU.model_config([{"type": "latent_attention", "mlp": None, "mixer": {
        "heads": 3, "dim": 16, "rot_dim": 0, "vdim": 8, "kv_rank": 24, "scale": 0.3}}]),
    "latent_wide_row": RU.model_config([RU.latent_layer(heads=2, dim=16, rot_dim=8, rot_dims=8, vdim=16, kv_rank=600, mlp=None)]),
    "latent_part_rotated": RU.model_config([RU.latent_layer(heads=5, dim=24, rot_dim=12, rot_dims=6, vdim=20, kv_rank=36, mlp=None)], width=56),
    "mamba2": RU.model_config([RU.mamba_layer()]),
    "mamba2_one_group_wide_state": RU.model_config([RU.mamba_layer(heads=3, vdim=5, state=130, groups=1, conv=5, norm_groups=1)]),
    "mamba2_one_tap": RU.model_config([RU.mamba_layer(conv=1, groups=4, norm_groups=4)]),
    "feed_forward": RU.model_config([RU.mamba_layer(heads=2, vdim=4, state=8, groups=1, norm_groups=1, mlp=(44, 0.3))]),
    "reentry": RU.model_config([RU.mamba_layer(heads=2, vdim=4, state=8, groups=1, norm_groups=1)], loop=(0, 1, 4)),
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(SINGLE))
def test_one_mechanism(name, dtype, tmp_path):
    cfg = SINGLE[name]
    folder = RU.make_folder(tmp_path, cfg, name, seed=5)
    ids = RU.tokens(cfg, 61, seed=1)
    want = RU.plain_logits(folder, ids)
    r = runner_for(folder, dtype)
    close(run_cut(r, ids, [61]), want, dtype, f"{name}, whole prompt")
    close(run_cut(r, ids, [29] + [1] * 32), want, dtype, f"{name}, 29 tokens then one by one")
    close(run_cut(r, ids, [2, 3, 2, 11, 2, 17, 1, 2, 21]), want, dtype, f"{name}, portions")


# ------------------------------------------------------------------------------------------------ whole models, every cutting
MODELS = {"X": RU.MODEL_X, "Y": RU.MODEL_Y, "Z": RU.MODEL_Z}


@pytest.fixture(scope="module", params=[(m, d) for m in sorted(MODELS) for d in ("float32", "bfloat16")], ids=lambda p: f"{p[0]}-{p[1]}")
def model(request, tmp_path_factory):
    name, dtype = request.param
    folder = RU.make_folder(tmp_path_factory.mktemp(f"radapel_{name}_{dtype}"), MODELS[name], name, seed=11)
    return name, dtype, folder, runner_for(folder, dtype, page_size=8, num_pages=40)


def test_whole_prompt_equals_token_by_token(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    for n in (1, 2, 9, 75):
        ids = RU.tokens(cfg, n, seed=2)
        want = RU.plain_logits(folder, ids)
        close(run_cut(r, ids, [n]), want, dtype, f"{name}: whole prompt of {n}")
        close(run_cut(r, ids, [1] * n), want, dtype, f"{name}: {n} tokens one by one")


def test_portions_of_several_sizes(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = RU.tokens(cfg, 120, seed=3)
    want = RU.plain_logits(folder, ids)
    for cuts in ([2] * 60, [7, 2, 13, 3, 2, 31, 1, 16, 2, 17, 8, 18], [33, 33, 33, 21], [119, 1]):
        close(run_cut(r, ids, cuts), want, dtype, f"{name}: portions {cuts[:4]}...")


def test_long_decoding(model):
    name, dtype, folder, r = model
    cfg = MODELS[name]
    ids = RU.tokens(cfg, 260, seed=4)
    close(run_cut(r, ids, [4] + [1] * 256), RU.plain_logits(folder, ids), dtype, f"{name}: 256 decoded tokens")


def test_unequal_requests_in_one_batch_with_pages_and_slots_used_again(model):
    """Four live requests at most, 40 pages of 8 tokens: the lengths below need far more over time, so pages and state slots come
    back and are handed out again; every request's logits equal those it gets alone."""
    name, dtype, folder, r = model
    cfg = MODELS[name]
    lengths = [97, 3, 64, 30, 1, 121, 45, 18, 70]
    todo = [(f"q{i}", RU.tokens(cfg, n, seed=20 + i)) for i, n in enumerate(lengths)]
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
        close(torch.cat(got[f"q{i}"]), RU.plain_logits(folder, RU.tokens(cfg, n, seed=20 + i)), dtype, f"{name}: request {i} of {n} tokens in the mix")


def test_replay_program_runs_the_design(tmp_path):
    cfg = RU.MODEL_Z
    folder = RU.make_folder(tmp_path, cfg, "Z", seed=11)
    ids_a, ids_b = RU.tokens(cfg, 50, seed=7), RU.tokens(cfg, 9, seed=8)
    r = Replay(folder, "float32", tmp_path / "out", max_tokens=128, page_size=16)
    got = r.step([{"id": "a", "tokens": ids_a[:31], "want": [0, 30]}, {"id": "b", "tokens": ids_b[:2], "want": []}])
    close(got, RU.plain_logits(folder, ids_a)[[0, 30]], "float32", "replay: first step")
    assert r.step([{"id": "b", "tokens": ids_b[2:8], "want": []}]) is None
    got = r.step([{"id": "a", "tokens": ids_a[31:], "want": [18]}, {"id": "b", "tokens": ids_b[8:], "want": [0]}], end=["a", "b"])
    close(got, torch.stack([RU.plain_logits(folder, ids_a)[49], RU.plain_logits(folder, ids_b)[8]]), "float32", "replay: last step")
    assert r.close() == 0


# ------------------------------------------------------------------------------------------------ greedy generation through the engine
@pytest.mark.parametrize("graphs", [False, True])
def test_greedy_generation_through_the_engine(graphs, tmp_path):
    from oxr_inference_b200.config import EngineSettings
    from oxr_inference_b200.engine.api import Engine, SamplingParams

    cfg = RU.MODEL_X
    folder = RU.make_folder(tmp_path, cfg, "X", seed=11)
    plain_cfg, w = RP.read_model(folder, torch.float64)
    prompts = [RU.tokens(cfg, n, seed=30 + n) for n in (5, 23, 1, 40, 12, 9)]
    engine = Engine(folder, EngineSettings(dtype="float32", num_pages=48, page_size=8, max_running=3, max_step_tokens=32, prefill_chunk=16,
                                           cuda_graphs=graphs))
    done = engine.generate(prompts, SamplingParams(max_tokens=14, ignore_eos=True))
    compared = 0
    for prompt, c in zip(prompts, done):
        want, gaps = RP.greedy(plain_cfg, w, prompt, 14)
        for a, b, gap in zip(c.token_ids, want, gaps):
            if gap < 1e-3:
                break          # a near-tie: from here on the two may differ for no fault
            assert a == b, f"prompt of {len(prompt)}: generated {c.token_ids}, the plain implementation {want}"
            compared += 1
    assert compared >= 60
    if graphs:
        assert engine.counters["graph_steps"] > 0


# ------------------------------------------------------------------------------------------------ keys that must, or must not, be seen
def _paged(keys, values, page_size, dtype, spare=3):
    """Scatter rows [ctx, KV, D] into pools with shuffled pages; returns pools, block table row."""
    ctx = keys.shape[0]
    n_pages = (ctx + page_size - 1) // page_size
    perm = torch.randperm(n_pages + spare, generator=torch.Generator().manual_seed(ctx))[:n_pages]
    k_pool = torch.zeros((n_pages + spare, page_size, *keys.shape[1:]), dtype=dtype)
    v_pool = torch.zeros((n_pages + spare, page_size, *values.shape[1:]), dtype=dtype) if values is not None else None
    for j in range(ctx):
        k_pool[perm[j // page_size], j % page_size] = keys[j]
        if values is not None:
            v_pool[perm[j // page_size], j % page_size] = values[j]
    return k_pool.to(DEV), (v_pool.to(DEV) if values is not None else None), perm.to(torch.int32).view(1, -1).to(DEV)


def _plain_attention(q, keys, values, positions, scale, chunk, window, bias, sink):
    """q [n, H, DK] at the given positions over keys/values [ctx, KV, *] of the same request, in float64."""
    n, H, _ = q.shape
    KV = keys.shape[1]
    out = torch.zeros(n, H, values.shape[2], dtype=torch.float64)
    for t, p in enumerate(positions):
        for h in range(H):
            g = h // (H // KV)
            seen = [j for j in range(p + 1) if (not chunk or j // chunk == p // chunk) and (not window or j > p - window)]
            s = torch.stack([q[t, h].double() @ keys[j, g].double() * scale + (bias[min(p - j, bias.shape[0] - 1), h].double() if bias is not None else 0)
                             for j in seen])
            top = max(s.max(), sink[h].double()) if sink is not None else s.max()
            e = torch.exp(s - top)
            denom = e.sum() + (torch.exp(sink[h].double() - top) if sink is not None else 0)
            out[t, h] = (e / denom) @ torch.stack([values[j, g].double() for j in seen])
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("case", ["far_key", "page_borders", "chunk_edges", "window_edges", "first_tokens", "sink", "values_in_key_rows"])
def test_keys_seen_and_not_seen(case, dtype):
    """One key is made to stand out (its score beats all others by far), so the output is that key's value when it is seen and
    something else when it is not: a mask that is one position off, or a page read wrongly, changes the output by its whole size."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(hash(case) % 1000)
    H, KV, DK, DV, P = 4, 2, 16, 24, 8
    chunk = window = 0
    sink = bias = None
    ctx = 75
    if case == "far_key":
        ctx, marked, queries = 700, [3], [699, 650, 3]
    elif case == "page_borders":
        marked, queries = [7, 8, 9, 15, 16, 63, 64], [64, 70, 74, 9, 8]
    elif case == "chunk_edges":
        chunk, marked, queries = 20, [19, 20, 39, 40, 59, 60], [20, 21, 39, 40, 41, 59, 60, 61, 74]
        bias = torch.randn(9, H, generator=g)
    elif case == "window_edges":
        window, marked, queries = 12, [30, 31, 50], [41, 42, 43, 61, 62, 50]
    elif case == "first_tokens":
        marked, queries = [0, 1], [0, 1, 2, 74]
    elif case == "sink":
        marked, queries = [40], [39, 40, 74]
        sink = torch.tensor([9.0, -4.0, 2.0, 30.0])
    else:
        marked, queries = [10, 33], [33, 34, 74]
    keys = torch.randn(ctx, KV, DK, generator=g) * 0.3
    values = torch.randn(ctx, KV, DV, generator=g)
    direction = torch.randn(DK, generator=g)
    direction /= direction.norm()
    for j in marked:
        keys[j] += 6 * direction          # every query leans on `direction`: marked keys win when seen
    q = torch.randn(len(queries), H, DK, generator=g) * 0.3 + 4 * direction
    if case == "values_in_key_rows":
        DV = 10
        values = keys[:, :, :DV].clone()
    q, keys, values = (t.to(dtype).float() for t in (q, keys, values))   # what the kernel will read, exactly
    want = _plain_attention(q, keys, values, queries, 0.5, chunk, window, bias, sink)
    k_pool, v_pool, table = _paged(keys, None if case == "values_in_key_rows" else values, P, dtype)
    status = ops.new_status(DEV)
    # the queries as a prompt's portion (all rows of one request) ...
    n = len(queries)
    pos = torch.tensor(queries, dtype=torch.int32, device=DEV)
    common = dict(value_dim=DV, block_table=table, scale=0.5, chunk=chunk, window=window,
                  dist_bias=None if bias is None else bias.to(DEV), sink=None if sink is None else sink.to(DEV), status=status)
    got = ops.attention_rows(q.to(dtype).view(n, H * DK).to(DEV), H, k_pool, v_pool, positions=pos, req_of_token=torch.zeros(n, dtype=torch.int32, device=DEV), **common)
    # ... and each as a single decoded token of a request of its own (row r of the table is request r's)
    common["block_table"] = table.repeat(n, 1).contiguous()
    alone = ops.attention_rows(q.to(dtype).view(n, H * DK).to(DEV), H, k_pool, v_pool, positions=pos,
                               req_of_token=torch.arange(n, dtype=torch.int32, device=DEV), **common)
    ops.check_status(status)
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for name, out in (("portion", got), ("single tokens", alone)):
        err = (out.float().cpu().view(n, H, DV) - want).abs().max()
        assert err <= tol * max(1.0, want.abs().max()), f"{case}, {name}: off by {err:.2e}"
    # the marked keys decide the output: hiding the mask's edge by one would have changed it
    shifted = _plain_attention(q, keys, values, [max(0, p - 1) for p in queries], 0.5, chunk, window, bias, sink)
    assert (shifted - want).abs().max() > 0.1


@pytest.mark.parametrize("case,D", [("chunk_bias", 32), ("sink", 32), ("window_chunk", 32), ("chunk_bias", 96), ("sink", 144), ("chunk_bias", 192),
                                    ("window_chunk", 224), ("sink", 256)])
def test_keys_seen_and_not_seen_by_the_tiled_kernels(case, D):
    """The same marked keys through the tensor-core kernels (bfloat16, keys and values of one size): a prompt's portion that crosses
    chunk edges (long tiles), a short portion, and single tokens of several requests with split keys."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(7)
    H, KV, P, ctx = 4, 2, 8, 300
    chunk, window, bias, sink = 0, 0, None, None
    if case == "chunk_bias":
        chunk, bias = 20, torch.randn(9, H, generator=g)
    elif case == "sink":
        sink = torch.tensor([9.0, -4.0, 2.0, 30.0])
    else:
        chunk, window = 64, 12
    keys = torch.randn(ctx, KV, D, generator=g) * 0.3
    values = torch.randn(ctx, KV, D, generator=g)
    direction = torch.randn(D, generator=g)
    direction /= direction.norm()
    for j in (0, 19, 20, 39, 40, 59, 60, 63, 64, 127, 128, 200, 255, 256, 288):
        keys[j] += 6 * direction
    keys, values = keys.to(torch.bfloat16).float(), values.to(torch.bfloat16).float()
    k_pool, v_pool, table = _paged(keys, values, P, torch.bfloat16)
    status = ops.new_status(DEV)
    specs = ops.attention_tile_specs(H, KV, D, torch.bfloat16)

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
                                  page_size=P, scale=0.5, window=window, kv_len_bound=max(ctx_lens), status=status, chunk=chunk,
                                  dist_bias=None if bias is None else bias.to(DEV), sink=None if sink is None else sink.to(DEV))
        ops.check_status(status)
        at = 0
        for x, c in zip(q_lens, ctx_lens):
            positions = list(range(c - x, c))
            want = _plain_attention(q[at:at + x].float(), keys, values, positions, 0.5, chunk, window, bias, sink)
            err = (out[at:at + x].float().cpu() - want).abs().max()
            assert err <= 2e-2 * max(1.0, want.abs().max()), f"{case}: request of {x} new tokens ending at {c}: off by {err:.2e}"
            at += x

    run([90, 5, 70], [130, 63, 300])                 # portions: long tiles, a short one
    run([1] * 9, [20, 21, 40, 41, 64, 65, 129, 257, 300])   # single tokens at and around the edges
    run([1, 33, 2, 1], [289, 290, 61, 1])            # mixed


# ------------------------------------------------------------------------------------------------ small kernels against their formulas
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_stream_kernels(dtype):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(1)
    n, hidden = 19, 88
    stream = torch.randn(n, hidden, generator=g) * 3
    y = (torch.randn(n, hidden, generator=g) * 0.2).to(dtype)
    w1, w2 = 1 + 0.1 * torch.randn(hidden, generator=g), 1 + 0.1 * torch.randn(hidden, generator=g)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    s = stream.clone().to(DEV)
    h = ops.norm_add_norm(s, y.to(DEV), w1.to(DEV), 1e-5, w2.to(DEV), 1e-3)
    want_s = stream.double() + RP.rms_norm(y.double(), w1.double(), 1e-5)
    assert (s.cpu() - want_s).abs().max() < 1e-5
    assert (h.float().cpu() - RP.rms_norm(want_s, w2.double(), 1e-3)).abs().max() < tol * 4
    rows = torch.tensor([5, 0, 18], dtype=torch.int32, device=DEV)
    picked = ops.stream_rms_norm(s, w2.to(DEV), 1e-3, dtype, rows=rows)
    assert (picked.float().cpu() - RP.rms_norm(want_s[[5, 0, 18]], w2.double(), 1e-3)).abs().max() < tol * 4
    gu = (torch.randn(n, 2 * 36, generator=g) * 2).to(dtype)
    got = ops.clamped_glu(gu.to(DEV), alpha=1.702, limit=0.9)
    gate, up = gu[:, :36].double().clamp(max=0.9), gu[:, 36:].double().clamp(-0.9, 0.9)
    assert (got.float().cpu() - gate * torch.sigmoid(1.702 * gate) * (up + 1)).abs().max() < tol * 2
    both = ops.concat2_cast(s, stream.to(DEV), dtype)
    assert torch.equal(both.float().cpu(), torch.cat([s.cpu(), stream], 1).to(dtype).float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n", [5, 16, 17, 150])
def test_per_head_linear(dtype, n):
    """Few rows run the CUDA-core kernel, more rows (bfloat16) the tensor-core one; both against the plain product, with entries
    of the output outside the written stretch left alone."""
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(n)
    heads, n_in, n_out = 3, 48, 80
    x = torch.randn(n, heads, n_in + 8, generator=g).to(dtype)
    w = (torch.randn(heads, n_in, n_out, generator=g) * 0.2).to(dtype)
    out = torch.full((n, heads, n_out + 5), 7.0, dtype=dtype)
    got = ops.head_linear(out.to(DEV), 3, x.to(DEV), 8, w.to(DEV)).float().cpu()
    want = torch.einsum("thi,hio->tho", x[:, :, 8:].double(), w.double())
    assert (got[:, :, 3:3 + n_out] - want).abs().max() <= (1e-4 if dtype == torch.float32 else 3e-2) * want.abs().max()
    assert torch.all(got[:, :, :3] == 7.0) and torch.all(got[:, :, 3 + n_out:] == 7.0)


@pytest.mark.parametrize("hidden", [88, 4096 + 64, 20000])
def test_wide_rows_through_the_vector_kernels(hidden):
    from oxr_inference_b200 import ops

    g = torch.Generator().manual_seed(hidden)
    n = 7
    stream = torch.randn(n, hidden, generator=g)
    y = torch.randn(n, hidden, generator=g).to(torch.bfloat16)
    w1, w2 = 1 + 0.1 * torch.randn(hidden, generator=g), 1 + 0.1 * torch.randn(hidden, generator=g)
    s = stream.clone().to(DEV)
    h = ops.norm_add_norm(s, y.to(DEV), w1.to(DEV), 1e-5, w2.to(DEV), 1e-6)
    want_s = stream.double() + RP.rms_norm(y.double(), w1.double(), 1e-5)
    assert (s.cpu() - want_s).abs().max() < 2e-5
    assert (h.float().cpu() - RP.rms_norm(want_s, w2.double(), 1e-6)).abs().max() < 4e-2
    s2 = stream.clone().to(DEV)
    assert ops.norm_add_norm(s2, y.to(DEV), w1.to(DEV), 1e-5) is None and torch.equal(s2, s)
    gu = (torch.randn(n, 2 * hidden, generator=g) * 2).to(torch.bfloat16)
    got = ops.clamped_glu(gu.to(DEV), alpha=1.702, limit=1.1)
    gate, up = gu[:, :hidden].double().clamp(max=1.1), gu[:, hidden:].double().clamp(-1.1, 1.1)
    assert (got.float().cpu() - gate * torch.sigmoid(1.702 * gate) * (up + 1)).abs().max() < 2e-2


def test_rotary_angles_are_exact_far_out():
    from oxr_inference_b200 import ops

    pos = torch.tensor([0, 1, 1000, 123457, 1 << 20], dtype=torch.int32, device=DEV)
    freq = torch.tensor([1e6 ** (-2 * i / 16) for i in range(8)], dtype=torch.float64)
    cos, sin = ops.rotary_angles(pos, freq.to(DEV))
    ang = pos.cpu().double()[:, None] * freq[None]
    assert (cos.cpu() - ang.cos()).abs().max() < 1e-7 and (sin.cpu() - ang.sin()).abs().max() < 1e-7


def test_scaled_embedding_is_rounded_once():
    from oxr_inference_b200 import ops

    table = torch.randn(10, 24).to(torch.bfloat16)
    ids = torch.tensor([3, 9, 0], dtype=torch.int32, device=DEV)
    out = ops.embedding(ids, table.to(DEV), torch.float32, ops.new_status(DEV), 0.7)
    assert torch.equal(out.cpu(), table[[3, 9, 0]].float() * torch.tensor(0.7, dtype=torch.float32))
