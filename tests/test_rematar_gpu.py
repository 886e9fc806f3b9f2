"""Rematar on the GPU against the plain implementation (tests/plain_rematar.py): every mechanism alone with inputs
made so that a fault shows, then whole models through the step function in every cut (whole, a long tail decoded
token by token, portions down to two tokens, mixed batches over a pool so small that pages and slots are used
again), in 32-bit and in bfloat16, and greedy generation through the engine's entry point and scheduler."""

import os
import subprocess

import numpy as np
import pytest
import torch

import plain_rematar as plain
from replay_util import (ROOT, compare, plan_chunks, plan_many_rows, plan_mixed, plan_tail, plan_whole, random_requests,
                         run_plan_in_process, run_plan_trace_run)
from rematar_configs import REMATAR

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
TOL = {"float32": (2e-5, 2e-5), "bfloat16": (5e-2, 0.0)}
LENGTHS = {"ra": [5, 70, 150, 33, 260, 129], "rb": [1, 7, 64, 100, 129, 40], "rc": [3, 48, 95, 200, 16, 131],
           "rd": [2, 65, 130, 31, 17, 140]}
SIZES = [16, 7, 2, 5, 3, 2, 11, 32, 2, 9, 64, 2]


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """dtype -> name -> model folder whose file holds that dtype."""
    from dynalm_b200.weights import write_model_folder
    out = {"float32": {}, "bfloat16": {}}
    for name, (cfg, seed) in REMATAR.items():
        for dtype, t in (("float32", torch.float32), ("bfloat16", torch.bfloat16)):
            d = tmp_path_factory.mktemp(f"rematar_{name}_{dtype}")
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
                reqs = random_requests(REMATAR[name][0]["vocab"], LENGTHS[name], seed=51 + len(made))
                model = plain.PlainRematar(folders[dtype][name])
                made[key] = (reqs, {r: model.logits(t) for r, t in reqs.items()})
            return made[key]
    return Lookup()


def _built(folder, dtype, kv_tokens, max_batch, max_requests=8):
    from dynalm_b200.engine import build
    return build(folder, dtype=dtype, kv_tokens=kv_tokens, max_batch_tokens=max_batch, max_requests=max_requests,
                 context=max(kv_tokens, 256))


def _t(a, dtype=torch.float32):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV, dtype)


def _np(t):
    return t.double().cpu().numpy()


def _ints(v):
    return torch.tensor(list(v), dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_after_the_sum(dtype):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(5)
    for width, rows, alpha, scaled in ((96, 5, 2.0, True), (100, 3, 1.0, False), (90, 4, 0.5, True), (2048, 2, 3.0, True),
                                       (5000, 2, 3.0, True), (9001, 1, 1.5, False)):
        x = _t(rng.randn(rows, width))
        w = _t(1 + 0.2 * rng.randn(width))
        ls = _t(1 + 0.5 * rng.randn(width)) if scaled else None
        for delta in (_t(rng.randn(rows, width), dtype), _t(rng.randn(3, rows, width))):      # whole, and split-K partial sums
            d = _np(delta) if delta.dim() == 2 else _np(delta).sum(0)
            want = plain.sum_then_norm(_np(x), d, alpha, 2e-5, _np(w), _np(ls) if scaled else None)
            got_x = x.clone()
            out = torch.zeros(rows, width, dtype=dtype, device=DEV)
            ops.norm_after_sum(got_x, delta, w, 2e-5, alpha, ls, out)
            tol = 1e-5 if dtype == torch.float32 else 2e-2
            assert np.abs(_np(got_x) - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
            assert np.abs(_np(out) - want).max() <= tol * max(1.0, np.abs(want).max())
            if dtype == torch.bfloat16:
                assert torch.equal(out, got_x.to(torch.bfloat16))        # the copy is the stream, rounded once


@pytest.mark.parametrize("rows,inner,width", [(4, 272, 256), (12, 272, 256), (40, 272, 256), (1024, 2048, 256), (300, 4096, 512)])
def test_gelu_in_the_epilogue_of_every_product_kernel(rows, inner, width):
    """gelu_tanh(x W^T) by whichever kernel the dispatcher picks for the shape (few rows: the weight-streaming ones; many
    tiles: the tcgen05 one; in between the library followed by the activation kernel) against the plain product."""
    from dynalm_b200.engine.runtime import Runtime
    from dynalm_b200.kernels.gemm import linear_act
    rng = np.random.RandomState(rows)
    rt = Runtime(DEV, torch.bfloat16, max_tokens=1024)
    x = _t(rng.randn(rows, width), torch.bfloat16)
    w = _t(rng.randn(inner, width) * 0.1, torch.bfloat16)
    got = _np(linear_act(x, w, rt, inner, "gelu_tanh"))
    want = plain.gelu_tanh(_np(x) @ _np(w).T)
    assert np.abs(got - want).max() <= 1e-2 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 5, 40, 300])
def test_gelu_feed_forward(dtype, rows):
    from dynalm_b200.config.plan import FeedForwardSpec
    from dynalm_b200.engine.runtime import Runtime
    from dynalm_b200.parts.base import build_part
    rng = np.random.RandomState(6)
    for width, inner in ((96, 160), (100, 172)):
        rt = Runtime(DEV, dtype, max_tokens=512)
        up = _t(rng.randn(inner, width) * 0.3, dtype)
        down = _t(rng.randn(width, inner) * 0.2, dtype)
        part = build_part(FeedForwardSpec("mlp", width, {"up": "u", "down": "d"}, inner=inner, activation="gelu_tanh"),
                          {"u": up, "d": down}, rt)
        x = _t(rng.randn(rows, width), dtype)
        got = part.forward(x, None)
        got = got.double().sum(0) if got.dim() == 3 else got.double()
        want = plain.dense_mlp(_np(x), _np(up), _np(down))
        tol = 1e-4 if dtype == torch.float32 else 6e-2
        assert np.abs(got.cpu().numpy() - want).max() <= tol * max(1.0, np.abs(want).max())


def _step_arrays(portions, slots):
    """The step's index arrays for requests that bring (first position, tokens) each, in state slots `slots`."""
    positions, row_request, row_slot, q_start, pos_start = [], [], [], [0], []
    for r, ((first, n), slot) in enumerate(zip(portions, slots)):
        positions += list(range(first, first + n))
        row_request += [r] * n
        row_slot += [slot] * n
        q_start.append(q_start[-1] + n)
        pos_start.append(first)
    return _ints(positions), _ints(row_request), _ints(row_slot), _ints(q_start), _ints(pos_start), _ints(slots)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps,channels,col0", [(4, 40, 3), (2, 7, 3), (1, 16, 3), (5, 300, 3), (4, 48, 8), (3, 64, 16)])
def test_convolution_in_portions_carries_its_last_inputs(dtype, taps, channels, col0):
    """Two requests in slots 2 and 0, cut differently (portions shorter than, equal to and longer than the taps),
    side by side in one batch; then slot 2 is used again by a new request and must not see the old inputs."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(taps * 100 + channels)
    extra = 2 if col0 % 8 else 8                                               # (pitches in multiples of 8 take 16-byte loads)
    w, b = _t(rng.randn(channels, taps)), _t(rng.randn(channels))
    keep_off = 11
    state = torch.zeros(4, keep_off + (taps - 1) * channels + 5, device=DEV)
    state[:, :keep_off] = 7.0                                                  # what lies in front is not touched
    seqs = {2: rng.randn(23, channels), 0: rng.randn(17, channels)}
    cuts = {2: [1, 1, 2, 3, 4, 5, 1, 6], 0: [5, 1, 1, 1, 2, 7]}
    want = {s: plain.silu(plain.causal_conv(_np(_t(u, dtype)), _np(w), _np(b))) for s, u in seqs.items()}
    at = {2: 0, 0: 0}
    for k in range(8):
        batch = [(s, at[s], cuts[s][k]) for s in (2, 0) if k < len(cuts[s])]
        rows = sum(n for _, _, n in batch)
        proj = torch.zeros(rows, col0 + channels + extra, dtype=dtype, device=DEV)
        r0 = 0
        for s, first, n in batch:
            proj[r0:r0 + n, col0:col0 + channels] = _t(seqs[s][first:first + n], dtype)
            r0 += n
        pos, rreq, rslot, q_start, pos_start, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        out = torch.zeros(rows, channels, dtype=dtype, device=DEV)
        ops.ssm_conv(proj, col0, channels, w.t().contiguous(), b, state, keep_off, pos, rreq, rslot, pos_start, out)
        ops.ssm_conv_keep(proj, col0, channels, taps, state, keep_off, q_start, slots, len(batch))
        r0 = 0
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        for s, first, n in batch:
            ref = want[s][first:first + n]
            assert np.abs(_np(out[r0:r0 + n]) - ref).max() <= tol * max(1.0, np.abs(ref).max()), f"slot {s} at {first}"
            r0 += n
            at[s] += n
    assert (state[:, :keep_off] == 7.0).all() and (state[1][keep_off:] == 0).all() and (state[3][keep_off:] == 0).all()
    if taps > 1:
        last = _np(_t(seqs[2][-(taps - 1):], dtype)).reshape(-1)
        assert np.array_equal(_np(state[2, keep_off:keep_off + (taps - 1) * channels]), last)      # oldest first
    # slot 2 handed out again: zeroed by the manager, here by hand
    state[2, keep_off:] = 0
    fresh = rng.randn(3, channels)
    proj = torch.zeros(3, col0 + channels + extra, dtype=dtype, device=DEV)
    proj[:, col0:col0 + channels] = _t(fresh, dtype)
    pos, rreq, rslot, q_start, pos_start, slots = _step_arrays([(0, 3)], [2])
    out = torch.zeros(3, channels, dtype=dtype, device=DEV)
    ops.ssm_conv(proj, col0, channels, w.t().contiguous(), b, state, keep_off, pos, rreq, rslot, pos_start, out)
    ref = plain.silu(plain.causal_conv(_np(_t(fresh, dtype)), _np(w), _np(b)))
    assert np.abs(_np(out) - ref).max() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, np.abs(ref).max())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G", [(4, 32, 64, 2), (5, 20, 12, 1), (4, 8, 16, 4), (2, 64, 128, 1), (3, 48, 40, 3), (1, 3, 5, 1),
                                     (2, 128, 256, 2)])
def test_recurrence_in_portions_keeps_its_state(dtype, H, P, N, G):
    """Two requests cut differently in one batch, against the plain scan of each whole sequence. The first head
    forgets almost nothing (a_log far below zero), and the first token of each sequence is made large: a state that
    is lost or started anew at a portion's first token shows at every later token."""
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H * 1000 + P + N)
    inner, dt_col, width = H * P, 2, 2 + H + 3
    lengths = {1: 41, 3: 19}
    cuts = {1: [1, 2, 9, 8, 1, 1, 16, 3], 3: [7, 1, 1, 2, 8]}
    a_log = rng.randn(H) * 0.3
    a_log[0] = -6.0
    dt_bias, d_skip = rng.randn(H) * 0.3, 1 + 0.2 * rng.randn(H)
    seqs, want = {}, {}
    for s, n in lengths.items():
        u = rng.randn(n, inner + 2 * G * N) * 0.7
        u[0, :inner] *= 6.0
        dt_raw = rng.randn(n, H)
        u_t, dt_t = _np(_t(u, dtype)), _np(_t(dt_raw, dtype))
        seqs[s] = (u, dt_raw)
        per = H // G
        B = np.repeat(u_t[:, inner:inner + G * N].reshape(n, G, N), per, axis=1)
        C = np.repeat(u_t[:, inner + G * N:].reshape(n, G, N), per, axis=1)
        want[s], _ = plain.ssm_scan(u_t[:, :inner].reshape(n, H, P), plain.softplus(dt_t + dt_bias), B, C, a_log, d_skip)
    tail = 9
    state = torch.zeros(5, inner * N + tail, device=DEV)
    state[:, inner * N:] = 3.0                                                 # what lies behind the matrices is not touched
    at = {1: 0, 3: 0}
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for k in range(8):
        batch = [(s, at[s], cuts[s][k]) for s in (3, 1) if k < len(cuts[s])]
        rows = sum(n for _, _, n in batch)
        u = torch.cat([_t(seqs[s][0][f:f + n], dtype) for s, f, n in batch])
        proj = torch.zeros(rows, width, dtype=dtype, device=DEV)
        proj[:, dt_col:dt_col + H] = torch.cat([_t(seqs[s][1][f:f + n], dtype) for s, f, n in batch])
        _, _, _, q_start, _, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        y = torch.zeros(rows, inner, device=DEV)
        ops.ssm_scan(u, proj, dt_col, _t(dt_bias), _t(a_log), _t(d_skip), state, q_start, slots, y, len(batch), H, P, N, G)
        r0 = 0
        for s, first, n in batch:
            ref = want[s][first:first + n].reshape(n, inner)
            err = np.abs(_np(y[r0:r0 + n]) - ref).max()
            assert err <= tol * max(1.0, np.abs(ref).max()), f"slot {s}, tokens {first}..{first + n - 1}: {err:.3g}"
            r0 += n
            at[s] += n
    assert (state[:, inner * N:] == 3.0).all() and (state[0][:inner * N] == 0).all() and (state[2][:inner * N] == 0).all()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,P,N,G", [(4, 32, 64, 2), (5, 20, 12, 1), (2, 64, 128, 1)])
def test_long_portions_run_as_segments_side_by_side(dtype, H, P, N, G):
    """Portions longer than a segment are cut by the step plan and run in three launches; shorter ones beside them run
    as one piece; a second step goes on from the states the first left (one of its requests long again)."""
    from types import SimpleNamespace
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(H + P + N)
    seg = ops.SSM_SEGMENT
    inner, dt_col, width = H * P, 1, 1 + H
    a_log = rng.randn(H) * 0.3
    a_log[0] = -7.0                                                            # a head that forgets almost nothing
    dt_bias, d_skip = rng.randn(H) * 0.3, 1 + 0.2 * rng.randn(H)
    steps = [{0: 2 * seg + 37, 2: 5, 3: seg, 1: seg + 1}, {0: seg + 3, 2: 1, 3: 2}]     # slot -> tokens brought
    total = {s: sum(st.get(s, 0) for st in steps) for s in range(4)}
    seqs, want = {}, {}
    for s, n in total.items():
        u = rng.randn(n, inner + 2 * G * N) * 0.7
        u[0, :inner] *= 6.0
        dt_raw = rng.randn(n, H)
        u_t, dt_t = _np(_t(u, dtype)), _np(_t(dt_raw, dtype))
        seqs[s] = (u, dt_raw)
        per = H // G
        B = np.repeat(u_t[:, inner:inner + G * N].reshape(n, G, N), per, axis=1)
        C = np.repeat(u_t[:, inner + G * N:].reshape(n, G, N), per, axis=1)
        want[s], _ = plain.ssm_scan(u_t[:, :inner].reshape(n, H, P), plain.softplus(dt_t + dt_bias), B, C, a_log, d_skip)
    state = torch.zeros(4, inner * N + 3, device=DEV)
    plan = ops.SSM_SEGMENTS
    max_tokens = 512
    at = {s: 0 for s in total}
    tol = 2e-5 if dtype == torch.float32 else 2e-2
    for st in steps:
        batch = [(s, at[s], n) for s, n in st.items()]
        rows = sum(n for _, _, n in batch)
        u = torch.cat([_t(seqs[s][0][f:f + n], dtype) for s, f, n in batch])
        proj = torch.zeros(rows, width, dtype=dtype, device=DEV)
        proj[:, dt_col:dt_col + H] = torch.cat([_t(seqs[s][1][f:f + n], dtype) for s, f, n in batch])
        _, _, _, q_start, _, slots = _step_arrays([(f, n) for _, f, n in batch], [s for s, _, _ in batch])
        host = np.zeros(plan.ints(max_tokens, 4), dtype=np.int32)
        meta = plan.fill(host, SimpleNamespace(q_len=[n for _, _, n in batch], q_start=[int(v) for v in q_start.cpu()[:-1]],
                                               slots=[s for s, _, _ in batch]))
        assert meta[0] == sum(-(-n // seg) for _, _, n in batch if n > seg) and meta[1] == sum(n > seg for _, _, n in batch)
        most = plan.most_segments(max_tokens)
        scratch = torch.full((most * inner * N,), float("nan"), device=DEV)     # whatever it held before must not matter
        decay = torch.full((most * H,), float("nan"), device=DEV)
        y = torch.zeros(rows, inner, device=DEV)
        ops.ssm_scan(u, proj, dt_col, _t(dt_bias), _t(a_log), _t(d_skip), state, q_start, slots, y, len(batch), H, P, N, G,
                     (torch.from_numpy(host).to(DEV), meta), scratch, decay)
        r0 = 0
        for s, first, n in batch:
            ref = want[s][first:first + n].reshape(n, inner)
            err = np.abs(_np(y[r0:r0 + n]) - ref).max(axis=1)
            bad = int(err.argmax())
            assert err[bad] <= tol * max(1.0, np.abs(ref).max()), f"slot {s}, token {first + bad}: {err[bad]:.3g}"
            r0 += n
            at[s] += n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gate_comes_before_the_norm_of_every_part(dtype):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(8)
    for inner, parts, rows in ((128, 2, 5), (100, 1, 3), (96, 3, 4), (2048, 4, 2), (30, 5, 7), (4096, 8, 3), (16384, 1, 2)):
        y = _t(rng.randn(rows, inner) * 3)
        z = _t(rng.randn(rows, inner + (9 if parts == 5 or inner == 128 else 8)) * 2, dtype)   # the gate's columns first, others behind
        w = _t(1 + 0.3 * rng.randn(inner))
        out = torch.zeros(rows, inner, dtype=dtype, device=DEV)
        ops.gated_group_norm(y, z, w, 1e-5, parts, out)
        want = plain.gated_group_norm(_np(y), _np(z)[:, :inner], parts, 1e-5, _np(w))
        assert np.abs(_np(out) - want).max() <= (1e-5 if dtype == torch.float32 else 2e-2) * max(1.0, np.abs(want).max())


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
@pytest.mark.parametrize("q_rank,R,r,rot,base", [(80, 64, 16, 16, 1e6), (36, 44, 12, 8, 500.0), (16, 24, 4, 0, 1.0), (72, 320, 32, 32, 1e4)])
def test_latents_are_normed_keys_turned_and_records_land_in_their_pages(dtype, q_rank, R, r, rot, base):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(q_rank)
    page, eps = 16, 1e-5
    positions = [0, 1, 15, 16, 17, 31, 32, 100, 4095, 100000]                    # first tokens, page borders, far out
    n = len(positions)
    proj = _t(rng.randn(n, q_rank + R + r + 5) * 2, dtype)
    wq, wkv = _t(1 + 0.3 * rng.randn(q_rank)), _t(1 + 0.3 * rng.randn(R))
    freq = torch.from_numpy(base ** (-2.0 * np.arange(rot // 2) / max(rot, 1))).to(DEV) if rot else None
    cache, table, pages = _paged(max(positions) + 1, page, R + r, dtype, seed=4)
    cq = torch.zeros(n, q_rank, dtype=dtype, device=DEV)
    ops.latent_prep(proj, q_rank, R, r, rot, wq, wkv, eps, freq, _ints(positions), _ints([1] * n), table, cache, page, cq)
    src = _np(proj)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    want_q = plain.rms_norm(src[:, :q_rank], eps, _np(wq))
    assert np.abs(_np(cq) - want_q).max() <= tol * max(1.0, np.abs(want_q).max())
    want_c = plain.rms_norm(src[:, q_rank:q_rank + R], eps, _np(wkv))
    want_k = src[:, q_rank + R:q_rank + R + r]
    if rot:
        want_k = plain.rotate_pairs(want_k, np.asarray(positions), rot, base)
    host = _np(cache)
    for i, p in enumerate(positions):
        rec = host[pages[p // page], p % page]
        assert np.abs(rec[:R] - want_c[i]).max() <= tol * max(1.0, np.abs(want_c).max()), f"latent of position {p}"
        assert np.abs(rec[R:] - want_k[i]).max() <= tol * max(1.0, np.abs(want_k).max()), f"key part of position {p}"
    assert np.count_nonzero(host.reshape(-1, R + r).any(axis=1)) == n              # nothing else was written
    # the queries' rotated pieces into the tails of wide queries, head by head
    H, d = 3, 10
    q = _t(rng.randn(n, H * (d + r) + 2), dtype)
    wide = torch.zeros(n, H * (R + r), dtype=dtype, device=DEV)
    if r:
        ops.rotate_pairs(q, d + r, d, wide, R + r, R, r, rot, freq, _ints(positions), H)
        got = _np(wide).reshape(n, H, R + r)
        piece = _np(q)[:, :H * (d + r)].reshape(n, H, d + r)[:, :, d:]
        want = plain.rotate_pairs(piece, np.asarray(positions), rot, base) if rot else piece
        assert np.abs(got[:, :, R:] - want).max() <= tol * max(1.0, np.abs(want).max())
        assert not got[:, :, :R].any()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows", [1, 8, 9, 70])
def test_per_head_products(dtype, rows):
    from dynalm_b200.kernels import ops
    rng = np.random.RandomState(rows)
    # (sizes in multiples of 8 take the tensor-core kernel in bfloat16, the others the plain one)
    for H, n_in, n_out, head_in, head_out in ((4, 16, 48, 24, 56), (3, 44, 28, 44, 28), (2, 320, 64, 320, 64), (5, 7, 150, 9, 150),
                                              (3, 40, 72, 48, 80), (2, 136, 200, 136, 200)):
        x = _t(rng.randn(rows, (H - 1) * head_in + n_in + 3), dtype)
        w = _t(rng.randn(H, n_in, n_out) * 0.3, dtype)
        gate = _t(rng.randn(rows, H * n_out + 4) * 2, dtype)
        xs = np.stack([_np(x)[:, h * head_in:h * head_in + n_in] for h in range(H)], axis=1)
        want = np.einsum("rhi,hio->rho", xs, _np(w))
        tol = 1e-5 if dtype == torch.float32 else 3e-2
        out = torch.zeros(rows, (H - 1) * head_out + n_out + 1, dtype=dtype, device=DEV)
        ops.head_linear(x, head_in, n_in, w, out, head_out)
        got = np.stack([_np(out)[:, h * head_out:h * head_out + n_out] for h in range(H)], axis=1)
        assert np.abs(got - want).max() <= tol * max(1.0, np.abs(want).max())
        assert not _np(out)[:, (H - 1) * head_out + n_out:].any()
        out.zero_()
        ops.head_linear(x, head_in, n_in, w, out, head_out, gate, n_out)
        got = np.stack([_np(out)[:, h * head_out:h * head_out + n_out] for h in range(H)], axis=1)
        gated = want * plain.sigmoid(_np(gate)[:, :H * n_out].reshape(rows, H, n_out))
        assert np.abs(got - gated).max() <= tol * max(1.0, np.abs(want).max())


def _attention_case(H, R, r, n_keys, page, dtype, seed):
    """Records of n_keys positions in shuffled pages; random wide queries are made by the caller."""
    rng = np.random.RandomState(seed)
    cache, table, pages = _paged(n_keys, page, R + r, dtype, seed=seed + 1)
    rec = rng.randn(n_keys, R + r)
    host = np.zeros((cache.shape[0], page, R + r))
    for p in range(n_keys):
        host[pages[p // page], p % page] = rec[p]
    cache.copy_(_t(host, dtype))
    return rng, cache, table, _np(_t(rec, dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,R,r,window", [(6, 64, 16, 24), (3, 44, 12, 7), (2, 32, 16, 0), (5, 24, 4, 33), (2, 320, 32, 64),
                                          (4, 48, 8, 600)])
def test_attention_over_records_with_a_key_made_to_stand_out(dtype, H, R, r, window):
    """Every query gets one key, at a distance of its own, whose record is made to carry the score: the newest key,
    the first token, the last key inside the window and the first outside it, keys on both sides of a page border and
    of a chunk's edge. A key outside must leave no trace; the sink is checked with sinks large enough to matter."""
    from dynalm_b200.kernels import ops
    page, n_keys, scale = 16, 1100, 0.3
    rng, cache, table, rec = _attention_case(H, R, r, n_keys, page, dtype, seed=H * 100 + R)
    w = window if window > 0 else 10 ** 9
    cases = []                                                                    # (query position, distance of its target)
    for pos in (0, 1, 5, 15, 16, 17, w - 1 if w < n_keys else 40, w if w < n_keys else 41, 511, 512, 513, 700, 1023, 1024, 1099):
        if pos >= n_keys:
            continue
        for dist in (0, 1, w - 1, w, w + 1, pos, pos % page, pos % page + 1, pos - 512):
            if 0 <= dist <= pos:
                cases.append((pos, dist))
    cases = sorted(set(cases))
    n = len(cases)
    q = rng.randn(n, H, R + r) * 0.5
    for i, (pos, dist) in enumerate(cases):
        for h in range(H):
            target = rec[pos - dist]
            q[i, h] += (4.0 + h) * target / (scale * np.dot(target, target))      # its score rises by 4 + h
    q_t = _t(q.reshape(n, -1), dtype)
    sink = rng.randn(H) + 2.0
    out = torch.zeros(n, H * R, dtype=dtype, device=DEV)
    positions = [p for p, _ in cases]
    for sk in (sink, None):
        ops.latent_attention(q_t, cache, table, _ints(positions), _ints([1] * n), _t(sk) if sk is not None else None, out, H,
                             R, r, page, scale, window)
        got = _np(out).reshape(n, H, R)
        qf = _np(q_t).reshape(n, H, R + r)
        k_pos = np.arange(n_keys)
        tol = 2e-5 if dtype == torch.float32 else 3e-2
        for h in range(H):
            s = (qf[:, h] @ rec.T) * scale
            wts = plain.window_sink_softmax(s, np.asarray(positions), k_pos, window, None if sk is None else float(sk[h]))
            want = wts @ rec[:, :R]
            err = np.abs(got[:, h] - want).max(axis=1)
            bad = int(err.argmax())
            assert err[bad] <= tol * max(1.0, np.abs(want).max()), \
                f"head {h}, query at {cases[bad][0]} whose key stands {cases[bad][1]} back: {err[bad]:.3g}"


@pytest.mark.parametrize("H,R,r,window", [(6, 64, 16, 24), (2, 32, 16, 0), (5, 24, 8, 33), (16, 320, 32, 64), (40, 48, 8, 600),
                                          (3, 512, 64, 100), (33, 16, 0, 5)])
def test_tensor_core_attention_over_tiles_of_a_step(H, R, r, window):
    """The bfloat16 kernel whose blocks take 32 (row, head) units: portions of two requests cut into tiles by the step
    plan, beside single decoded tokens; every query has a key made to stand out at the window's edge, just outside it,
    at a key tile's border or at the first token."""
    from dynalm_b200.kernels import latent_attention as fast
    from dynalm_b200.kernels import ops
    from types import SimpleNamespace
    dtype, page, n_keys, scale = torch.bfloat16, 16, 700, 0.3
    rng, cache, table, rec = _attention_case(H, R, r, n_keys, page, dtype, seed=H * 10 + R)
    # the same records serve three requests (their table rows name the same pages): a portion from the first token, a
    # portion in the middle that crosses key tiles and a chunk border, two single tokens
    table[0] = table[1]
    table[2] = table[1]
    portions = [(1, 0, 75), (0, 600, 1), (2, 430, 97), (1, 699, 1)]              # (slot, first position, rows)
    w = window if window > 0 else 10 ** 9
    positions, slots = [], []
    for slot, first, n in portions:
        positions += list(range(first, first + n))
        slots += [slot] * n
    n = len(positions)
    q = rng.randn(n, H, R + r) * 0.5
    for i, pos in enumerate(positions):
        for h in range(H):
            dist = [0, w - 1, w, pos % 64, pos % 64 + 1, pos][(i + h) % 6]
            if 0 <= dist <= pos:
                target = rec[pos - dist]
                q[i, h] += (4.0 + h % 5) * target / (scale * np.dot(target, target))
    q_t = _t(q.reshape(n, -1), dtype)
    sink = _t(rng.randn(H) + 2.0)
    spec = SimpleNamespace(num_heads=H, kv_rank=R, rot_dim=r)
    plan = fast.tile_plan(spec)
    host = np.zeros(plan.ints(n, len(portions)), dtype=np.int32)
    q_start = np.cumsum([0] + [p[2] for p in portions])
    n_tiles = plan.fill(host, SimpleNamespace(q_len=[p[2] for p in portions], q_start=list(q_start[:-1]),
                                               pos_start=[p[1] for p in portions], slots=[p[0] for p in portions]))
    assert n_tiles == sum(-(-p[2] // plan.rows) for p in portions) and plan.rows * fast.heads_per_block(H) <= 32
    tiles = torch.from_numpy(host).to(DEV)
    out = torch.zeros(n, H * R, dtype=dtype, device=DEV)
    ops.latent_attention_flash(q_t, cache, table, tiles, n_tiles, sink, out, H, R, r, page, scale, window, fast.heads_per_block(H))
    qf = _np(q_t).reshape(n, H, R + r)
    want = [plain.window_sink_softmax((qf[:, h] @ rec.T) * scale, np.asarray(positions), np.arange(n_keys), window,
                                      float(sink[h])) @ rec[:, :R] for h in range(H)]

    def check(what):
        got = _np(out).reshape(n, H, R)
        for h in range(H):
            err = np.abs(got[:, h] - want[h]).max(axis=1)
            bad = int(err.argmax())
            assert err[bad] <= 3e-2 * max(1.0, np.abs(want[h]).max()), f"{what}: head {h}, query at {positions[bad]}: {err[bad]:.3g}"

    check("one block per tile")
    # the keys of every tile dealt over several blocks (more parts than some tiles have key tiles), merged afterwards
    for parts in (2, 5, 16):
        out.fill_(7.0)
        scratch = torch.full((n * H * parts * (R + 2),), float("nan"), device=DEV)
        ops.latent_attention_flash(q_t, cache, table, tiles, n_tiles, sink, out, H, R, r, page, scale, window,
                                   fast.heads_per_block(H), parts, scratch)
        check(f"{parts} parts")


# ---------------------------------------------------------------------------------------------
# whole models through the step function
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(REMATAR))
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


def test_a_model_without_scales_sinks_and_gate(tmp_path):
    """The tensors a model takes by presence, left out: the file decides, and both implementations follow it."""
    from dynalm_b200.registry import find_architecture
    from dynalm_b200.weights.loader import expected_tensors
    from dynalm_b200.weights.random_init import random_tensors
    from dynalm_b200.weights.safetensors import write_safetensors
    import json
    cfg, seed = REMATAR["ra"]
    arch = find_architecture(cfg)
    full = set(expected_tensors(arch.plan(arch.read_config(cfg))))
    lean = {n for n in full if not n.endswith((".ls1", ".ls2", ".mix.sink", ".mix.g"))}
    assert len(lean) < len(full)
    tensors = random_tensors(arch.plan(arch.read_config(cfg), present=lean), seed, torch.float32)
    assert set(tensors) == lean
    (tmp_path / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(tmp_path / "model.safetensors"), tensors)
    reqs = random_requests(cfg["vocab"], [50, 9], seed=3)
    model = plain.PlainRematar(str(tmp_path))
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_chunks(reqs, [5, 2, 30])
    built = _built(str(tmp_path), "float32", 256, 64, max_requests=2)
    compare(plan, run_plan_in_process(built.step_fn, plan), logits, *TOL["float32"], "lean")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_many_single_token_rows_beside_a_portion(dtype, folders):
    """A couple of dozen live requests decoding beside portions of long prompts: unequal requests in one batch
    against each alone."""
    name = "ra"
    vocab = REMATAR[name][0]["vocab"]
    short = {f"s{k}": v for k, v in random_requests(vocab, [12 + (5 * i) % 29 for i in range(20)], seed=8).items()}
    long = {f"l{k}": v for k, v in random_requests(vocab, [150, 90], seed=9).items()}
    model = plain.PlainRematar(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in {**short, **long}.items()}
    plan = plan_many_rows(short, long, seed=3, tail_lo=4, tail_hi=10)
    need = plan.max_live_tokens(64)
    built = _built(folders[dtype][name], dtype, need, 256, max_requests=24)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], f"{name}/{dtype}/many rows")


@pytest.mark.parametrize("name", ["ra", "rd"])
def test_long_decoding_keeps_its_place(name, folders):
    """300 tokens decoded one by one after a 3-token prompt: the window passes over decoded tokens many times, pages
    behind it are given back while the request lives, and the recurrent state is carried through every step (also
    through the steps that are replayed from a captured graph)."""
    dtype = "float32"
    reqs = random_requests(REMATAR[name][0]["vocab"], [303], seed=12)
    model = plain.PlainRematar(folders[dtype][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_tail(reqs, 300)
    built = _built(folders[dtype][name], dtype, 320, 64, max_requests=2)
    got = run_plan_in_process(built.step_fn, plan)
    compare(plan, got, logits, *TOL[dtype], "long decoding")
    assert built.cache.free_pages == built.cache.num_pages


def test_trace_run_replays_a_plan(folders, tmp_path):
    name = "rb"
    reqs = random_requests(REMATAR[name][0]["vocab"], [40, 7, 90], seed=13)
    model = plain.PlainRematar(folders["float32"][name])
    logits = {r: model.logits(t) for r, t in reqs.items()}
    plan = plan_mixed(reqs, seed=2)
    got = run_plan_trace_run(folders["float32"][name], "float32", plan, str(tmp_path), plan.max_live_tokens(64),
                             REMATAR[name][0]["vocab"])
    compare(plan, got, logits, *TOL["float32"], "trace_run")


# ---------------------------------------------------------------------------------------------
# generation through the entry point
# ---------------------------------------------------------------------------------------------

@pytest.mark.parametrize("name", ["ra", "rb", "rc"])
def test_greedy_generation_through_the_engine(name, folders):
    from dynalm_b200 import Engine
    folder = folders["float32"][name]
    model = plain.PlainRematar(folder)
    reqs = random_requests(REMATAR[name][0]["vocab"], [5, 17, 33, 70], seed=14)
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
    """An engine whose pool is too small for its requests preempts and recomputes (a state cannot be rewound, so a
    preempted request starts again from its first token), and gives the tokens of a roomy one."""
    from dynalm_b200 import Engine, SchedulerConfig
    name = "rc"                                      # one of its layers has no window: its pages are never given back
    reqs = list(random_requests(REMATAR[name][0]["vocab"], [40, 90, 17, 100, 64, 33], seed=15).values())

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
    proc = subprocess.run([os.path.join(ROOT, "bin", "dynalm"), "run", folders["bfloat16"]["ra"], "--tokens", "5,9,200,31",
                           "-n", "8", "--ctx", "256", "--batch", "64", "--no-stream"], capture_output=True, text=True,
                          timeout=600)
    assert proc.returncode == 0, proc.stderr[-3000:]
    ids = [int(t) for t in proc.stdout.split()]
    assert len(ids) == 8 and all(0 <= t < REMATAR["ra"][0]["vocab"] for t in ids)
    from dynalm_b200 import Engine
    assert Engine(folders["bfloat16"]["ra"], ctx=256, batch=64).generate([5, 9, 200, 31], max_tokens=8).tokens == ids
