"""Todupel on the GPU against the plain implementation (tests/plain_todupel.py): every mechanism alone with inputs
made so that a fault shows, then whole models through the step function in every cut (whole, a long tail decoded
token by token, portions down to two tokens, mixed batches over a pool so small that pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's entry point and scheduler."""

import os
import subprocess

import numpy as np
import pytest
import torch

import plain_todupel as plain
from replay_util import (ROOT, compare, plan_chunks, plan_many_rows, plan_mixed, plan_tail, plan_whole, random_requests,
                         run_plan_in_process, run_plan_trace_run)
from todupel_configs import TODUPEL

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": (2e-5, 2e-5), "bfloat16": (5e-2, 0.0)}
LENGTHS = {"ta": [5, 70, 150, 33, 260, 129], "tb": [1, 7, 64, 100, 129, 40], "tc": [3, 48, 95, 200, 16, 131],
           "td": [2, 65, 130, 31, 17], "te": [4, 150, 33, 71, 129]}
SIZES = [16, 7, 2, 5, 3, 2, 11, 32, 2, 9, 64, 2]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """dtype -> name -> model folder whose file holds that dtype."""
    from dynalm_b200.weights import write_model_folder
    out = {"float32": {}, "bfloat16": {}}
    for name, (cfg, seed) in TODUPEL.items():
        for dtype, t in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            d = tmp_path_factory.mktemp(f"todupel_{name}_{dtype}")
            write_model_folder(str(d), cfg, seed, dtype=t)
            out[dtype][name] = str(d)
    return out


@pytest.fixture(scope="module")
def plain_logits(folders):
    made = {}

    class Lookup:
        def __getitem__(self, key):
            name, dtype = key
            if key not in made:
                reqs = random_requests(TODUPEL[name][0]["vocab"], LENGTHS[name], seed=31 + len(made))
                model = plain.PlainTodupel(folders[dtype][name])
                made[key] = (reqs, {r: model.logits(t) for r, t in reqs.items()})
            return made[key]
    return Lookup()


def _built(folder, dtype, kv_tokens, max_batch, max_requests=8):
    from dynalm_b200.engine import build
    return build(folder, dtype=dtype, kv_tokens=kv_tokens, max_batch_tokens=max_batch, max_requests=max_requests,
                 context=max(kv_tokens, 256))


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------

def _paged(n_tokens, page, record, dtype, seed, slots=3, slot=1):
    """An empty cache [pages, page, record] with a shuffled block table whose row `slot` covers n_tokens."""
    blocks = -(-n_tokens // page)
    rng = np.random.RandomState(seed)
    pages = rng.permutation(blocks + 5)[:blocks].astype(np.int32)
    table = np.full((slots, blocks + 2), -1, dtype=np.int32)
    table[slot, :blocks] = pages
    cache = torch.zeros(blocks + 5, page, record, dtype=dtype, device=DEV)
    return cache, torch.from_numpy(table).to(DEV), pages


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,dim,vdim,every", [(4, 2, 16, 32, 7), (3, 1, 20, 36, 5), (2, 2, 64, 64, 0), (8, 2, 128, 128, 16)])
def test_unit_norm_temperature_and_cache_write(dtype, heads, groups, dim, vdim, every):
    """Per-unit norm of q and k, the temperature on both sides of every step of its floor, and where keys and
    values land in the paged records."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(3)
    page, eps, coef = 16, 1e-5, 0.6
    # rows of one request at positions around the steps of floor((p + 1) / every), the first tokens and a page border
    positions = sorted(set([0, 1, 15, 16, 17] + ([every * k + o for k in (1, 2, 3) for o in (-2, -1, 0)] if every else [30, 31])))
    n = len(positions)
    qw, kw, vw = heads * 2 * dim, groups * 2 * dim, groups * vdim
    x = torch.from_numpy(rng.randn(n, qw + kw + vw) * 3.0).to(DEV, dtype)
    wq = torch.from_numpy(1.0 + 0.3 * rng.randn(dim)).to(DEV, torch.float32)
    wk = torch.from_numpy(1.0 + 0.3 * rng.randn(dim)).to(DEV, torch.float32)
    cache, table, pages = _paged(max(positions) + 1, page, kw + vw, dtype, seed=4)
    pos_t = torch.tensor(positions, dtype=torch.int32, device=DEV)
    slot_t = torch.full((n,), 1, dtype=torch.int32, device=DEV)
    ref_in = x.double().cpu().numpy()
    ops.qk_norm_cache_write(x, pos_t, slot_t, table, cache, 0, kw, wq, wk, eps, coef, every, 2 * heads, 2 * groups, dim, vw, page)
    q_ref = plain.rms_norm(ref_in[:, :qw].reshape(n, 2 * heads, dim), eps, wq.double().cpu().numpy())
    if every:
        q_ref = q_ref * plain.query_temperature(np.asarray(positions), coef, every)[:, None, None]
    k_ref = plain.rms_norm(ref_in[:, qw:qw + kw].reshape(n, 2 * groups, dim), eps, wk.double().cpu().numpy())
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    got_q = x[:, :qw].double().cpu().numpy().reshape(n, 2 * heads, dim)
    assert np.abs(got_q - q_ref).max() <= tol * max(1.0, np.abs(q_ref).max())
    host = cache.double().cpu().numpy()
    for r, p in enumerate(positions):
        rec = host[pages[p // page], p % page]
        assert np.abs(rec[:kw].reshape(2 * groups, dim) - k_ref[r]).max() <= tol * max(1.0, np.abs(k_ref).max()), f"keys of position {p}"
        assert np.array_equal(rec[kw:], ref_in[r, qw + kw:]), f"values of position {p}"
    # a layer that reads another's records touches only its queries
    before = cache.clone()
    y = torch.from_numpy(rng.randn(n, qw)).to(DEV, dtype)
    ops.qk_norm_cache_write(y, pos_t, slot_t, None, None, 0, 0, wq, None, eps, coef, every, 2 * heads, 0, dim, 0, page,
                            write_cache=False)
    assert torch.equal(before, cache)


def _attention_case(heads, groups, dim, vdim, n_keys, page, dtype, seed, scale, cap, standout=True):
    """Records of n_keys positions with random keys and values, queries for the positions in `at`, and, when
    `standout`, per query one far key per map made to carry the score (a different key for each map)."""
    rng = np.random.RandomState(seed)
    kw, vw = groups * 2 * dim, groups * vdim
    keys = rng.randn(n_keys, groups, 2, dim)
    values = rng.randn(n_keys, groups, vdim) * 2.0
    return rng, kw, vw, keys, values


ATTENTION_SHAPES = [(4, 2, 16, 32), (6, 2, 48, 16), (2, 2, 64, 64), (5, 1, 20, 36), (8, 2, 128, 128), (4, 1, 32, 128),
                    (20, 1, 16, 16)]       # the last: more heads on a KV head than one tile of the single-token kernel holds


def _run_attention(kind, q, cache, kw, table, pos_t, slot_t, heads, groups, dim, vdim, page, scale, cap, lam, out_scale, eps):
    from dynalm_b200.kernels import ops
    out = torch.zeros(q.shape[0], heads * vdim, dtype=q.dtype, device=DEV)
    if kind == "plain":
        ops.diff_attention(q, cache, 0, kw, table, pos_t, slot_t, out, heads, groups, dim, vdim, page, scale, cap, lam,
                           out_scale, eps)
    else:
        from dynalm_b200.kernels import diff_attention as fast
        fast.run_for_test(kind, q, cache, kw, table, pos_t, slot_t, out, heads, groups, dim, vdim, page, scale, cap, lam,
                          out_scale, eps)
    return out


def _attention_kinds(dtype, dim, vdim):
    kinds = ["plain"]
    if dtype == torch.bfloat16 and dim % 16 == 0 and vdim % 16 == 0 and dim <= 128 and vdim <= 128:
        kinds += ["flash", "split"]
    return kinds


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,groups,dim,vdim", ATTENTION_SHAPES)
def test_differential_attention_where_one_key_carries_the_score(dtype, heads, groups, dim, vdim):
    """Each query's two maps are each pointed at one key of their own: far back, at a page's first or last place, at
    the query's own position, at position 0. A kernel that loses a key, reads the other map's keys or a neighbour's
    page gives another value row. Queries sit at the first tokens, at page borders and at the borders of the
    kernels' key tiles (64) and chunks (512)."""
    page, eps, init = 16, 1e-5, 0.4
    n_keys = 1040
    scale, cap = 0.3, 40.0
    rng, kw, vw, keys, values = _attention_case(heads, groups, dim, vdim, n_keys, page, dtype, 9, scale, cap)
    at = [0, 1, 2, 15, 16, 17, 63, 64, 65, 127, 128, 511, 512, 513, 1023, 1024, 1039]
    targets = {}       # (query row, head, map) -> key position
    q = rng.randn(len(at), heads, 2, dim) * 0.1
    choices = lambda p: [0, p, max(0, p - 1), (p // page) * page, max(0, (p // page) * page - 1), p // 2, min(p, 3)]
    for r, p in enumerate(at):
        for h in range(heads):
            g = h // (heads // groups)
            for m in range(2):
                t = choices(p)[(r + 2 * h + m) % 7]
                targets[r, h, m] = t
                q[r, h, m] = keys[t, g, m] / np.linalg.norm(keys[t, g, m]) * (9.0 + m)      # q . k_t stands out
    lam = torch.tensor([0.37], dtype=torch.float32, device=DEV)
    cache, table, pages = _paged(n_keys, page, kw + vw, dtype, seed=10)
    rec = np.concatenate([keys.reshape(n_keys, kw), values.reshape(n_keys, vw)], axis=1)
    host = np.zeros(tuple(cache.shape))
    for t in range(n_keys):
        host[pages[t // page], t % page] = rec[t]
    cache.copy_(torch.from_numpy(host).to(dtype))
    q_t = torch.from_numpy(q.reshape(len(at), -1)).to(DEV, dtype)
    # the plain implementation sees what the kernels see: operands rounded to the storage type
    k_r = cache.double().cpu().numpy()
    rec_r = np.stack([k_r[pages[t // page], t % page] for t in range(n_keys)])
    keys_r, values_r = rec_r[:, :kw].reshape(n_keys, groups, 2, dim), rec_r[:, kw:].reshape(n_keys, groups, vdim)
    q_r = q_t.double().cpu().numpy().reshape(len(at), heads, 2, dim)
    want = np.zeros((len(at), heads, vdim))
    k_pos = np.arange(n_keys)
    for h in range(heads):
        g = h // (heads // groups)
        a = [plain.map_attention(q_r[:, h, m], keys_r[:, g, m], values_r[:, g], np.asarray(at), k_pos, scale, cap) for m in range(2)]
        want[:, h] = plain.diff_combine(a[0], a[1], 0.37, init, eps)
    pos_t = torch.tensor(at, dtype=torch.int32, device=DEV)
    slot_t = torch.full((len(at),), 1, dtype=torch.int32, device=DEV)
    tol = 2e-5 if dtype == torch.float32 else 3e-2
    for kind in _attention_kinds(dtype, dim, vdim):
        got = _run_attention(kind, q_t, cache, kw, table, pos_t, slot_t, heads, groups, dim, vdim, page, scale, cap, lam,
                             1.0 - init, eps).double().cpu().numpy().reshape(len(at), heads, vdim)
        err = np.abs(got - want).max(axis=-1)
        r, h = np.unravel_index(np.argmax(err), err.shape)
        assert err.max() <= tol, (f"{kind}: query at position {at[r]}, head {h} (its maps point at keys "
                                  f"{targets[r, h, 0]} and {targets[r, h, 1]}): max |diff| {err.max():.3g}")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pair_norm_adds_both_pending_outputs_and_shares_one_statistic(dtype):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(5)
    for width, rows in ((96, 5), (100, 3), (90, 4), (2048, 2), (5000, 2)):
        x = torch.from_numpy(rng.randn(rows, width)).to(DEV, torch.float32)
        da = torch.from_numpy(rng.randn(rows, width)).to(DEV, dtype)
        db = torch.from_numpy(rng.randn(3, rows, width)).to(DEV, torch.float32)       # partial sums of a split product
        w1 = torch.from_numpy(1 + 0.2 * rng.randn(width)).to(DEV, torch.float32)
        w2 = torch.from_numpy(1 + 0.2 * rng.randn(width)).to(DEV, torch.float32)
        v = x.double().cpu().numpy() + da.double().cpu().numpy() + db.double().cpu().numpy().sum(0)
        o1 = torch.zeros(rows, width, dtype=dtype, device=DEV)
        o2 = torch.zeros(rows, width, dtype=dtype, device=DEV)
        ops.rmsnorm_pair(x, w1, o1, w2, o2, 2e-5, delta_a=da, delta_b=db)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        assert np.abs(x.double().cpu().numpy() - v).max() <= 1e-5
        assert np.abs(o1.double().cpu().numpy() - plain.rms_norm(v, 2e-5, w1.double().cpu().numpy())).max() <= tol
        assert np.abs(o2.double().cpu().numpy() - plain.rms_norm(v, 2e-5, w2.double().cpu().numpy())).max() <= tol
        # gathered rows, one output, nothing written back
        keep = x.clone()
        pick = torch.tensor([rows - 1, 0], dtype=torch.int32, device=DEV)
        o3 = torch.zeros(2, width, dtype=dtype, device=DEV)
        ops.rmsnorm_pair(x, w1, o3, None, None, 2e-5, delta_a=da, delta_b=None, rows=pick)
        v2 = (keep.double().cpu().numpy() + da.double().cpu().numpy())[[rows - 1, 0]]
        assert torch.equal(keep, x)
        assert np.abs(o3.double().cpu().numpy() - plain.rms_norm(v2, 2e-5, w1.double().cpu().numpy())).max() <= tol


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 5, 40, 300])
def test_squared_relu_feed_forward(dtype, rows):
    from dynalm_b200.config.plan import FeedForwardSpec
    from dynalm_b200.engine.runtime import Runtime
    from dynalm_b200.parts.base import build_part
    rng = np.random.RandomState(6)
    for width, inner in ((96, 160), (100, 172)):
        rt = Runtime(DEV, dtype, max_tokens=512)
        up = torch.from_numpy(rng.randn(inner, width) * 0.2).to(DEV, dtype)
        down = torch.from_numpy(rng.randn(width, inner) * 0.2).to(DEV, dtype)
        part = build_part(FeedForwardSpec("mlp", width, {"up": "u", "down": "d"}, inner=inner, activation="relu2"),
                          {"u": up, "d": down}, rt)
        x = torch.from_numpy(rng.randn(rows, width)).to(DEV, dtype)
        got = part.forward(x, None)
        got = got.double().sum(0) if got.dim() == 3 else got.double()
        want = plain.relu2_mlp(x.double().cpu().numpy(), up.double().cpu().numpy(), down.double().cpu().numpy())
        tol = 1e-4 if dtype == torch.float32 else 6e-2
        assert np.abs(got.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("rows,inner,width", [(4, 272, 256), (12, 272, 256), (40, 272, 256), (1024, 2048, 256), (300, 4096, 512)])
def test_squared_relu_in_the_epilogue_of_every_product_kernel(rows, inner, width):
    """max(x W^T, 0)^2 by whichever kernel the dispatcher picks for the shape (few rows: the weight-streaming ones; many
    tiles: the tcgen05 one; in between the library followed by the activation kernel) against the plain product."""
    from dynalm_b200.engine.runtime import Runtime
    from dynalm_b200.kernels.gemm import linear_relu2
    rng = np.random.RandomState(rows)
    rt = Runtime(DEV, torch.bfloat16, max_tokens=1024)
    x = torch.from_numpy(rng.randn(rows, width)).to(DEV, torch.bfloat16)
    w = torch.from_numpy(rng.randn(inner, width) * 0.1).to(DEV, torch.bfloat16)
    got = linear_relu2(x, w, rt, inner).double().cpu().numpy()
    z = np.maximum(x.double().cpu().numpy() @ w.double().cpu().numpy().T, 0.0)
    want = z * z
    assert np.abs(got - want).max() <= 1e-2 * max(1.0, np.abs(want).max())
    assert (got >= 0).all() and (got[want == 0] == 0).all()


# ---------------------------------------------------------------------------------------------
# whole models through the step function
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(TODUPEL))
def test_replay_all_cuts(name, dtype, folders, plain_logits):
    reqs, logits = plain_logits[name, dtype]
    tol = TOL[dtype]
    plans = {
        "whole": plan_whole(reqs),
        "tail48": plan_tail(reqs, 48),
        "chunks": plan_chunks(reqs, SIZES),
        "mixed": plan_mixed(reqs, seed=5),
        "mixed2": plan_mixed(reqs, seed=6, max_live=3, decode_tail=20),
    }
    for what, plan in plans.items():
        need = plan.max_live_tokens(64)          # just what the plan needs: pages of finished requests are used again
        built = _built(folders[dtype][name], dtype, need, max(need, 64), max_requests=4)
        got = run_plan_in_process(built.step_fn, plan)
        compare(plan, got, logits, tol[0], tol[1], f"{name}/{dtype}/{what}")
        assert built.cache.free_pages == built.cache.num_pages, "pages were lost"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_single_token_rows_beside_a_portion(dtype, folders):
    """A couple of dozen live requests decoding beside portions of long prompts: unequal requests in one batch
    against each alone."""
    name = "ta"
    vocab = TODUPEL[name][0]["vocab"]
    short = {f"s{k}": v for k, v in random_requests(vocab, [12 + (5 * i) % 29 for i in range(20)], seed=8).items()}
    long = {f"l{k}": v for k, v in random_requests(vocab, [150, 90], seed=9).items()}
    model = plain.PlainTodupel(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in {**short, **long}.items()}
    plan = plan_many_rows(short, long, seed=3, tail_lo=4, tail_hi=10)
    need = plan.max_live_tokens(64)
    built = _built(folders[dtype][name], dtype, need, 256, max_requests=24)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], f"{name}/{dtype}/many rows")


def test_long_decoding_keeps_its_place(folders):
    """300 tokens decoded one by one after a 3-token prompt: every step of the temperature's floor, every page and
    every key tile is entered by a decoded token."""
    name, dtype = "ta", "bfloat16"
    reqs = random_requests(TODUPEL[name][0]["vocab"], [303], seed=12)
    model = plain.PlainTodupel(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_tail(reqs, 300)
    built = _built(folders[dtype][name], dtype, 320, 64, max_requests=2)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], "long decoding")


def test_trace_run_replays_a_plan(folders, tmp_path):
    name = "tb"
    reqs = random_requests(TODUPEL[name][0]["vocab"], [40, 7, 90], seed=13)
    model = plain.PlainTodupel(folders["float32"][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_mixed(reqs, seed=2)
    got = run_plan_trace_run(folders["float32"][name], "float32", plan, str(tmp_path), plan.max_live_tokens(64),
                             TODUPEL[name][0]["vocab"])
    compare(plan, got, logits, *TOL["float32"], "trace_run")


# ---------------------------------------------------------------------------------------------
# generation through the entry point
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["ta", "tb", "tc"])
def test_greedy_generation_through_the_engine(name, folders):
    from dynalm_b200 import Engine
    folder = folders["float32"][name]
    model = plain.PlainTodupel(folder)
    reqs = random_requests(TODUPEL[name][0]["vocab"], [5, 17, 33, 70], seed=14)
    eng = Engine(folder, dtype="float32", ctx=512, batch=64, max_running=4)
    outs = eng.generate(list(reqs.values()), max_tokens=12)
    for prompt, g in zip(reqs.values(), outs):
        assert g.status == "finished" and len(g.tokens) == 12
        seq = list(prompt) + list(g.tokens)
        rows = model.logits(seq[:-1])
        for i, tok in enumerate(g.tokens):
            row = rows[len(prompt) - 1 + i]
            assert row[tok] >= row.max() - 2e-5, f"token {i}: chose {tok} at {row[tok]:.6f}, best {row.max():.6f}"
    alone = [eng.generate(p, max_tokens=12).tokens for p in reqs.values()]
    assert alone == [g.tokens for g in outs]


def test_few_pages_give_the_same_tokens(folders):
    """An engine whose pool is too small for its requests preempts and recomputes, and gives the tokens of a roomy one."""
    from dynalm_b200 import Engine, SchedulerConfig
    name = "ta"
    reqs = list(random_requests(TODUPEL[name][0]["vocab"], [40, 90, 17, 100, 64, 33], seed=15).values())

    def run(ctx):
        eng = Engine(folders["float32"][name], dtype="float32", ctx=ctx, batch=128, max_running=8,
                     scheduler=SchedulerConfig(max_running=6, decode_token_budget=8, prefill_token_budget=64,
                                               max_prefill_chunk=32, max_batch_tokens=128))
        out = eng.generate(reqs, max_tokens=40)
        assert eng.built.cache.free_pages == eng.built.cache.num_pages
        return [g.tokens for g in out], eng.scheduler.stats.preemptions

    roomy, p0 = run(4096)
    tight, p1 = run(320)
    assert p0 == 0 and p1 > 0
    assert tight == roomy


def test_command_line_generates(folders):
    proc = subprocess.run([os.path.join(ROOT, "bin", "dynalm"), "run", folders["bfloat16"]["ta"], "--tokens", "5,9,200,31",
                           "-n", "8", "--ctx", "256", "--batch", "64", "--no-stream"], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(t) for t in proc.stdout.split()]
    assert len(ids) == 8 and all(0 <= t < TODUPEL["ta"][0]["vocab"] for t in ids)
    from dynalm_b200 import Engine
    assert Engine(folders["bfloat16"]["ta"], ctx=256, batch=64).generate([5, 9, 200, 31], max_tokens=8).tokens == ids
