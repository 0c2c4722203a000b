"""Latinex on the GPU: each new kernel against the plain statement of its mechanism, each mixer alone through a
one-layer model, and whole models through the engine (step function, cache and state manager, scheduler) under every
way of cutting the work, in 32-bit and in bfloat16."""
import copy
import json
import math
import os

import pytest
import torch

import plain_latinex as plain
import traces
from latinex_models import CASES, write

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

# Relative to the largest |logit| of a request.
TOL = {"float32": 5e-5, "bfloat16": 4e-2}
# A differing expert choice must be a near-tie of the router's scores.
MARGIN = 2e-2
LENGTHS = {"A": [1, 9, 40, 83, 150, 2], "B": [150, 5, 67, 200, 31], "C": [3, 70, 140, 45, 210, 64, 65],
           "D": [1, 2, 30, 5], "E": [140, 66, 3, 129, 230]}


def requests_for(name):
    vocab = CASES[name][0]["vocab"]
    return {f"r{i}": traces.random_tokens(vocab, n, seed=41 * i + n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write(name, str(tmp_path_factory.mktemp(f"latinex_{name}"))) for name in CASES}


@pytest.fixture(scope="module")
def expected(folders):
    out = {}
    for name, folder in folders.items():
        cfg, w = plain.load_folder(folder)
        out[name] = {rid: plain.forward(cfg, w, toks) for rid, toks in requests_for(name).items()}
    return out


def engine_for(folder, dtype, max_tokens, max_batch=4, page_size=None, graphs=True):
    from sharpinference_b200 import Engine, EngineOptions
    opts = EngineOptions()
    if page_size:
        opts.page_size = page_size
    opts.max_cache_tokens = max(max_tokens, opts.page_size)
    opts.max_batch = max_batch
    opts.cuda_graphs = graphs
    return Engine(folder, dtype=dtype, device=DEV, options=opts)


def reference_for(folder, reqs, routing, fallback, dtype):
    """float32 runs are held to the plain logits as they are; bfloat16 runs to the plain logits under the engine's
    own expert choices, each differing choice having to be a near-tie of the plain router's scores."""
    if dtype == "float32":
        return fallback
    cfg, w = plain.load_folder(folder)
    ref = {}
    for rid, toks in reqs.items():
        choices = []
        for per_layer in routing[rid]:
            t = torch.tensor(per_layer, dtype=torch.long)
            choices.append(t.view(len(toks), -1))
        logits, _, seen = plain.forward(cfg, w, toks, want_layers=True, choices=choices)
        for (scores, chosen), forced in zip(seen, choices):
            top = forced.shape[1]
            kth = scores.topk(top, dim=-1).values[:, -1:]                       # the smallest score a free choice takes
            picked = scores.gather(1, forced)
            assert float((kth - picked).max()) < MARGIN, f"request {rid}: an expert choice differs beyond a near-tie"
        ref[rid] = logits
    return ref


def run_and_compare(folder, name, dtype, steps, expected, page_size=None, max_batch=4, reqs=None):
    reqs = reqs or requests_for(name)
    eng = engine_for(folder, dtype, traces.max_tokens(steps, page_size or 64), max_batch=max_batch, page_size=page_size)
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(eng, steps, routing)
    eng.runner.flush_status()
    eng.cache.check_invariants()
    assert not eng.cache.requests and all(g.pages.held_count == 0 for g in eng.cache.groups)
    wanted = sum(len(e["want"]) for st in steps for e in st["entries"])
    assert len({rid for rid, _ in got}) == len(reqs) and len(got) == wanted
    ref = reference_for(folder, reqs, routing, expected[name] if expected else None, dtype)
    err, where = traces.worst_error(got, ref)
    assert err < TOL[dtype], f"{name} {dtype}: error {err} at {where}"
    return eng


def _step_meta(lengths, slots):
    """row_request, row_offsets, state_slots of a step whose requests bring ``lengths`` rows."""
    rr, off = [], [0]
    for b, n in enumerate(lengths):
        rr += [b] * n
        off.append(off[-1] + n)
    i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)
    return i32(rr), i32(off), i32(slots)


f32 = lambda t: t.float().to(DEV).contiguous()


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H", [16, 52, 257, 1024])
def test_tanh_norm_with_the_residual_add(H):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(H)
    T = 11
    x, delta = 3 * torch.randn(T, H, generator=g, dtype=F64), torch.randn(T, H, generator=g, dtype=F64)
    w, b = torch.randn(H, generator=g, dtype=F64), torch.randn(H, generator=g, dtype=F64)
    alpha = torch.tensor([0.37], dtype=torch.float32, device=DEV)
    xd = f32(x)
    out, out32 = ops.add_dyt(xd, f32(delta), f32(w), f32(b), alpha, torch.bfloat16, want_fp32=True)
    want = plain.dyt((x + delta).float().double(), 0.37, w, b)
    assert torch.allclose(xd.double().cpu(), x + delta, atol=1e-5)                       # the stream is moved on
    assert torch.allclose(out32.double().cpu(), want, atol=1e-5)
    assert torch.equal(out, out32.to(torch.bfloat16))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32, device=DEV)
    before = xd.clone()
    out, _ = ops.add_dyt(xd, f32(delta), f32(w), f32(b), alpha, torch.float32, rows=rows)
    assert torch.equal(xd, before)                                                       # gathered rows: x stays
    assert torch.allclose(out.double().cpu(), plain.dyt(xd.double().cpu() + delta.float().double(), 0.37, w, b)[[7, 0, 3]],
                          atol=1e-5)
    out, _ = ops.add_dyt(xd, None, f32(w), None, alpha, torch.float32)
    assert torch.allclose(out.double().cpu(), plain.dyt(xd.double().cpu(), 0.37, w, torch.zeros(H, dtype=F64)), atol=1e-5)


def _plain_ssd(x, B, C, dt_raw, dt_bias, a_log, dskip, heads, groups):
    """x [T, heads, P], B and C [T, groups, N], dt_raw [T, heads]: the recurrence token by token."""
    T, _, P = x.shape
    N = B.shape[-1]
    dt = plain.softplus(dt_raw + dt_bias)
    S = torch.zeros(heads, N, P, dtype=F64)
    y = torch.zeros(T, heads, P, dtype=F64)
    for t in range(T):
        for h in range(heads):
            gi = h // (heads // groups)
            S[h] = torch.exp(-torch.exp(a_log[h]) * dt[t, h]) * S[h] + dt[t, h] * torch.outer(B[t, gi], x[t, h])
            y[t, h] = S[h].T @ C[t, gi] + dskip[h] * x[t, h]
    return y.reshape(T, heads * P)


@pytest.mark.parametrize("heads,groups,N,P", [(4, 2, 16, 8), (2, 1, 5, 13), (1, 1, 1, 2), (3, 3, 200, 16), (4, 1, 64, 32),
                                              (2, 2, 48, 48), (6, 2, 128, 64), (1, 1, 9, 70)])
def test_state_space_duality_scan(heads, groups, N, P):
    """Three requests in portions (one sits steps out; the state is carried in its slot) against the plain walk."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(heads * 1000 + N + P)
    lens = (37, 9, 21)
    inner, bc = heads * P, groups * N
    ld = inner + 2 * bc + 3                                   # x | B | C and three columns that are not read
    seqs = [0.7 * torch.randn(n, ld, generator=g, dtype=F64) for n in lens]
    dts = [torch.randn(n, heads + 2, generator=g, dtype=F64) for n in lens]            # raw step sizes at column 2
    dt_bias = -2.0 + 2.0 * torch.rand(heads, generator=g, dtype=F64)
    a_log = -3.0 + 3.0 * torch.rand(heads, generator=g, dtype=F64)
    dskip = torch.randn(heads, generator=g, dtype=F64)
    want = [_plain_ssd(s[:, :inner].reshape(-1, heads, P), s[:, inner:inner + bc].reshape(-1, groups, N),
                       s[:, inner + bc:inner + 2 * bc].reshape(-1, groups, N), d[:, 2:], dt_bias, a_log, dskip, heads, groups)
            for s, d in zip(seqs, dts)]
    state = torch.zeros(5, heads * N * P, device=DEV)
    state[4] = 7.0                                            # a slot that no request of the step holds stays as it is
    slots = [3, 0, 2]
    got, at = [[] for _ in seqs], [0, 0, 0]
    for cut in ([17, 2, 1], [1, 0, 2], [2, 3, 16], [16, 0, 1], [1, 4, 1]):
        live = [b for b in range(3) if cut[b]]
        _, off, sl = _step_meta([cut[b] for b in live], [slots[b] for b in live])
        xbc = torch.cat([seqs[b][at[b]:at[b] + cut[b]] for b in live])
        dt = torch.cat([dts[b][at[b]:at[b] + cut[b]] for b in live])
        y = ops.ssd_scan(f32(xbc), f32(dt), col_x=0, col_b=inner, col_c=inner + bc, col_dt=2, dt_bias=f32(dt_bias),
                         a_log=f32(a_log), dskip=f32(dskip), row_offsets=off, state_slots=sl, state=state, heads=heads,
                         groups=groups, states=N, vdim=P)
        r = 0
        for b in live:
            got[b].append(y[r:r + cut[b]].double().cpu())
            r += cut[b]
            at[b] += cut[b]
    for b in range(3):
        scale = float(want[b].abs().max())
        assert float((torch.cat(got[b]) - want[b]).abs().max()) < 2e-5 * max(scale, 1.0)
    assert float(state[4].min()) == 7.0 and float(state[1].abs().max()) == 0.0


@pytest.mark.parametrize("N,P", [(48, 24), (64, 32), (128, 64)])
def test_scan_rows_do_not_depend_on_the_cut(N, P):
    """The walk adds a row's parts in one fixed order: a prompt in one step and the same prompt in portions of 1, 2
    and 16 rows give the same bits, row by row and in the state left behind (sizes that leave padding in the walk's
    buffers and sizes that leave none; single rows and longer portions are launched differently)."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(3)
    heads, groups, T = 3, 1, 67
    inner, bc = heads * P, groups * N
    xbc, dt = f32(torch.randn(T, inner + 2 * bc, generator=g)), f32(torch.randn(T, heads, generator=g))
    vec = lambda: f32(torch.randn(heads, generator=g) - 1.0)
    dt_bias, a_log, dskip = vec(), vec(), vec()
    run = lambda rows, state, off: ops.ssd_scan(rows[0], rows[1], col_x=0, col_b=inner, col_c=inner + bc, col_dt=0,
                                                dt_bias=dt_bias, a_log=a_log, dskip=dskip, row_offsets=off[1],
                                                state_slots=off[2], state=state, heads=heads, groups=groups, states=N, vdim=P)
    s_a, s_b = torch.zeros(1, heads * N * P, device=DEV), torch.zeros(1, heads * N * P, device=DEV)
    whole = run((xbc, dt), s_a, _step_meta([T], [0]))
    parts, at = [], 0
    for n in (1, 2, 16, 1, 31, 2, 14):
        parts.append(run((xbc[at:at + n].contiguous(), dt[at:at + n].contiguous()), s_b, _step_meta([n], [0])))
        at += n
    assert at == T and torch.equal(torch.cat(parts), whole) and torch.equal(s_a, s_b)


@pytest.mark.parametrize("width,parts", [(32, 1), (32, 2), (48, 3), (26, 1), (26, 13), (768, 4)])
def test_gate_then_norm_in_parts(width, parts):
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(width + parts)
    T, col = 7, 5
    y = 2 * torch.randn(T, width, generator=g, dtype=F64)
    proj = torch.randn(T, col + width + 2, generator=g, dtype=F64)
    w = torch.randn(width, generator=g, dtype=F64)
    u = y.float().double() * plain.silu(proj[:, col:col + width].float().double())
    want = plain.rms(u.view(T, parts, width // parts), 1e-3).reshape(T, width) * w
    got = ops.gated_group_norm(f32(y), f32(proj), col, f32(w), 1e-3, parts, torch.float32)
    assert torch.allclose(got.double().cpu(), want, atol=2e-5)
    # the gate comes before the norm: norming first and gating after is something else
    other = plain.rms(y.view(T, parts, width // parts), 1e-3).reshape(T, width) * w * plain.silu(proj[:, col:col + width])
    assert not torch.allclose(want, other, atol=1e-2)


def _paged_keys(keys, page_size, seed):
    """Keys [T, nkv, d] written into shuffled pages of a pool that also holds garbage: (kv_layer, block_table)."""
    T, nkv, d = keys.shape
    blocks = (T + page_size - 1) // page_size
    pool = blocks + 5
    perm = torch.randperm(pool, generator=torch.Generator().manual_seed(seed))[:blocks]
    kv = 50.0 * torch.ones(pool, 1, nkv, page_size, d)                        # what a page held before
    for t in range(T):
        kv[perm[t // page_size], 0, :, t % page_size] = keys[t]
    return kv, perm.to(torch.int32).view(1, blocks)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,keep,page", [(75, 21, 64), (33, 5, 16), (64, 3, 64), (130, 64, 64), (5, 0, 16), (1, 2, 16),
                                              (0, 0, 64)])
def test_keys_as_values_attention_with_one_key_that_stands_out(window, keep, page, dtype):
    """For a query at the end of 300 positions, one key at a time is made to stand out (a score of 36 against at
    most 6): a far one, the first and last kept, the one behind them, the two at the window's edge, those at page
    borders, the query's own.  The output is then that key if the rule lets the query see it and a mixture of the
    others if not, so a rule that is one position off shows as an error of the key's size.  A whole prompt in one
    step and single rows (decoding) run the same check; the distance bias is on."""
    from sharpinference_b200.kernels import ops
    T, nq, nkv, d, rows_rel, far = 300, 4, 2, 16, 8, 40
    g = torch.Generator().manual_seed(window * 7 + keep)
    rel = torch.randn(rows_rel, nq, generator=g)
    table = torch.stack([rel[plain.distance_bucket(n, rows_rel, far)] for n in range(far + 1)])
    i = T - 1
    targets = sorted({0, 1, keep - 1, keep, keep + 1, i - window, i - window + 1, i - window + 2, 63, 64, 127, 128, i - 1, i,
                      150} & set(range(T)))
    unit = torch.nn.functional.normalize(torch.randn(d, generator=g), dim=0)
    for j in targets:
        keys = torch.randn(T, nkv, d, generator=g)
        keys = keys - (keys @ unit)[..., None] * unit                          # the others have no part along `unit`
        keys[j] = keys[j] + 6.0 * unit
        q = 0.3 * torch.randn(T, nq, d, generator=g)
        q[i] = q[i] + 6.0 * unit
        kq, qq = keys.to(dtype).double(), q.to(dtype).double()
        vis = plain.window_with_first(T, window, keep) if window else plain.causal(T)
        want = torch.empty(T, nq, d, dtype=F64)
        dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0, max=far)
        for h in range(nq):
            kh = kq[:, h // (nq // nkv)]
            p = plain.softmax_rows(qq[:, h] @ kh.T * 1.0 + table.double()[dist, h], vis)
            want[:, h] = p @ kh
        seen = bool(vis[i, j])
        assert (float((want[i, 0] @ unit.double())) > 5.0) == seen, (j, seen)
        kv, bt = _paged_keys(keys, page, seed=j)
        kv, bt = kv.to(dtype).to(DEV), bt.to(DEV)
        tol = 2e-4 if dtype == torch.float32 else 6e-2
        kw = dict(nq=nq, nkv=nkv, d=d, page_size=page, mask_kind=ops.MASK_WINDOW if window else ops.MASK_FULL,
                  mask_span=max(window, 1), scale=1.0, keep_first=keep if window else 0, dist_bias=table.to(DEV))
        rr, pos = torch.zeros(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV)
        out = ops.paged_attention_generic(q.to(dtype).to(DEV).view(T, nq * d), kv, bt, rr, pos, **kw)
        assert float((out.double().cpu().view(T, nq, d) - want).abs().max()) < tol, (j, "prompt")
        for row in (i, max(j, 0), min(j + window, i) if window else i):
            one = ops.paged_attention_generic(q[row:row + 1].to(dtype).to(DEV).view(1, nq * d), kv, bt, rr[:1],
                                              pos[row:row + 1].contiguous(), **kw)
            assert float((one.double().cpu().view(nq, d) - want[row]).abs().max()) < tol, (j, row, "single row")
        if dtype == torch.bfloat16:
            # the tensor-core kernels for keys-only pages: tiles of 64 rows, and single rows split over their keys
            kw.pop("d")
            qd = q.to(dtype).to(DEV).view(T, nq * d)
            tiles = torch.tensor([[t0, min(64, T - t0), t0, 0] for t0 in range(0, T, 64)], dtype=torch.int32, device=DEV)
            out = torch.zeros(T, nq * d, dtype=dtype, device=DEV)
            ops.attention_keys_prefill(qd, kv, bt, tiles, out, d=d, dv=d, **kw)
            assert float((out.double().cpu().view(T, nq, d) - want).abs().max()) < tol, (j, "prompt, tensor cores")
            some = torch.tensor(sorted({i, j, min(j + window, i), max(min(j + window, i) - 1, 0), 17, 255, 256}),
                                dtype=torch.int32, device=DEV)
            out = torch.zeros(T, nq * d, dtype=dtype, device=DEV)
            ops.attention_keys_decode(qd, kv, bt, rr, pos, out, rows=some, num_rows=some.numel(), max_context=T, d=d, dv=d, **kw)
            got = out.double().cpu().view(T, nq, d)[some.cpu().long()]
            assert float((got - want[some.cpu().long()]).abs().max()) < tol, (j, "single rows, tensor cores")


@pytest.mark.parametrize("nq,nkv,d,dv,page", [(16, 1, 320, 256, 64), (4, 1, 48, 48, 16), (8, 1, 96, 64, 64), (2, 2, 512, 512, 64),
                                              (20, 1, 128, 128, 64), (3, 3, 16, 16, 16), (6, 2, 208, 144, 32)])
def test_tensor_core_attention_over_keys_only_pages(nq, nkv, d, dv, page):
    """Rows of many sizes whose leading ``dv`` elements are the value: two requests on shuffled pages, portions as
    tiles and single rows in one step, against the plain softmax."""
    from sharpinference_b200.kernels import ops
    g = torch.Generator().manual_seed(nq * d + dv)
    lens, scale = (333, 70), 2.0 / math.sqrt(d)
    keys = [torch.randn(n, nkv, d, generator=g).to(torch.bfloat16) for n in lens]
    qs = [torch.randn(n, nq, d, generator=g).to(torch.bfloat16) for n in lens]
    want = []
    for k, q in zip(keys, qs):
        w = torch.empty(k.shape[0], nq, dv, dtype=F64)
        for h in range(nq):
            kh = k[:, h // (nq // nkv)].double()
            w[:, h] = plain.softmax_rows(q[:, h].double() @ kh.T * scale, plain.causal(k.shape[0])) @ kh[:, :dv]
        want.append(w)
    blocks = [(n + page - 1) // page for n in lens]
    pool = sum(blocks) + 3
    perm = torch.randperm(pool, generator=g)
    kv = torch.full((pool, 1, nkv, page, d), 30.0).to(torch.bfloat16)
    bt = torch.full((2, max(blocks)), -1, dtype=torch.int32)
    at = 0
    for b, k in enumerate(keys):
        for blk in range(blocks[b]):
            pg = int(perm[at])
            at += 1
            bt[b, blk] = pg
            rows = k[blk * page:(blk + 1) * page]
            kv[pg, 0, :, :rows.shape[0]] = rows.transpose(0, 1)
    kv, bt = kv.to(DEV), bt.to(DEV)
    # one step: request 0 brings its rows 100 .. 332 (a portion: tiles), request 1 its last three rows (single rows)
    step_rows = [(0, r) for r in range(100, 333)] + [(1, r) for r in range(67, 70)]
    q = torch.stack([qs[b][r] for b, r in step_rows]).to(DEV).view(len(step_rows), nq * d)
    rr = torch.tensor([b for b, _ in step_rows], dtype=torch.int32, device=DEV)
    pos = torch.tensor([r for _, r in step_rows], dtype=torch.int32, device=DEV)
    tiles = torch.tensor([[t0, min(64, 233 - t0), 100 + t0, 0] for t0 in range(0, 233, 64)], dtype=torch.int32, device=DEV)
    single = torch.tensor([233, 234, 235], dtype=torch.int32, device=DEV)
    out = torch.zeros(len(step_rows), nq * dv, dtype=torch.bfloat16, device=DEV)
    kw = dict(nq=nq, nkv=nkv, d=d, dv=dv, page_size=page, mask_kind=ops.MASK_FULL, mask_span=1, scale=scale)
    ops.attention_keys_prefill(q, kv, bt, tiles, out, **kw)
    ops.attention_keys_decode(q, kv, bt, rr, pos, out, rows=single, num_rows=3, max_context=333, **kw)
    got = out.double().cpu().view(len(step_rows), nq, dv)
    ref = torch.stack([want[b][r] for b, r in step_rows])
    assert float((got - ref).abs().max()) < 3e-2
    # a row alone gives the bits it gave in the batch, and a row of a tile the bits of the same row in a tile cut elsewhere
    alone = torch.zeros_like(out)
    ops.attention_keys_decode(q, kv, bt, rr, pos, alone, rows=single[1:2].contiguous(), num_rows=1, max_context=70, **kw)
    assert torch.equal(alone[234], out[234])
    other = torch.zeros_like(out)
    tiles2 = torch.tensor([[0, 7, 100, 0], [7, 64, 107, 0], [71, 64, 171, 0], [135, 64, 235, 0], [199, 34, 299, 0]],
                          dtype=torch.int32, device=DEV)
    ops.attention_keys_prefill(q, kv, bt, tiles2, other, **kw)
    assert torch.equal(other[:233], out[:233])


@pytest.mark.parametrize("d,dv,window,keep", [(80, 80, 100, 3), (320, 256, 300, 70), (128, 128, 256, 0), (16, 16, 7, 257)])
def test_single_rows_with_whole_splits_behind_the_window(d, dv, window, keep):
    """Single rows deep in a sequence of 1200 positions: between the kept first positions and the window lie whole
    splits of 256 keys that the row does not see, and the window's lower edge falls inside a split and at its border.
    Row sizes on both sides of the size at which a CTA holds all keys of a split (a block a warp) or a ring of two
    blocks; one far kept key is made to carry a head's row."""
    from sharpinference_b200.kernels import ops
    T, nq, nkv, page, far, rows_rel = 1200, 6, 2, 64, 500, 12
    g = torch.Generator().manual_seed(d + window)
    rel = torch.randn(rows_rel, nq, generator=g)
    table = torch.stack([rel[plain.distance_bucket(n, rows_rel, far)] for n in range(far + 1)])
    keys = torch.randn(T, nkv, d, generator=g).to(torch.bfloat16)
    q = torch.randn(T, nq, d, generator=g)
    if keep:
        q[:, 0] = 12.0 * keys[keep - 1, 0].float() / math.sqrt(d)         # head 0 asks for the last kept key
    q = q.to(torch.bfloat16)
    scale = 1.0 / math.sqrt(d)
    vis = plain.window_with_first(T, window, keep)
    dist = (torch.arange(T)[:, None] - torch.arange(T)[None, :]).clamp(min=0, max=far)
    rows = sorted({T - 1, 1023, 1024, 1024 + window - 1, 1024 + window, 767 + window, 768 + window, 700, 255, 256, keep + window,
                   max(keep + window - 1, 0)} & set(range(T)))
    want = torch.empty(len(rows), nq, dv, dtype=F64)
    for h in range(nq):
        kh = keys[:, h // (nq // nkv)].double()
        p = plain.softmax_rows(q[:, h].double() @ kh.T * scale + table.double()[dist, h], vis)
        want[:, h] = (p @ kh[:, :dv])[rows]
    if keep:
        p0 = plain.softmax_rows(q[:, 0].double() @ keys[:, 0].double().T * scale + table.double()[dist, 0], vis)
        assert float(p0[T - 1, keep - 1]) > 0.5 and not bool(vis[T - 1, keep])
    kv, bt = _paged_keys(keys.float(), page, seed=d)
    kv, bt = kv.to(torch.bfloat16).to(DEV), bt.to(DEV)
    rr = torch.zeros(T, dtype=torch.int32, device=DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    some = torch.tensor(rows, dtype=torch.int32, device=DEV)
    out = torch.zeros(T, nq * dv, dtype=torch.bfloat16, device=DEV)
    kw = dict(nq=nq, nkv=nkv, d=d, dv=dv, page_size=page, mask_kind=ops.MASK_WINDOW, mask_span=window, scale=scale,
              keep_first=keep, dist_bias=table.to(DEV))
    ops.attention_keys_decode(q.to(DEV).view(T, nq * d), kv, bt, rr, pos, out, rows=some, num_rows=len(rows), max_context=T, **kw)
    got = out.double().cpu().view(T, nq, dv)[rows]
    assert float((got - want).abs().max()) < 4e-2
    # the same rows as the tails of tiles give the same values
    tiles = torch.tensor([[r - 10, 11, r - 10, 0] for r in rows if r >= 10], dtype=torch.int32, device=DEV)
    tiled = torch.zeros_like(out)
    ops.attention_keys_prefill(q.to(DEV).view(T, nq * d), kv, bt, tiles, tiled, **kw)
    keep_rows = [k for k, r in enumerate(rows) if r >= 10]
    got_t = tiled.double().cpu().view(T, nq, dv)[[rows[k] for k in keep_rows]]
    assert float((got_t - want[keep_rows]).abs().max()) < 4e-2


def test_distance_bias_is_not_scaled_and_reads_the_head_of_the_query():
    """Two keys with equal dot products: the bias alone decides, per head, and the score factor leaves it alone."""
    from sharpinference_b200.kernels import ops
    nq, d, page = 3, 8, 16
    keys = torch.zeros(2, 1, d)
    keys[0, 0, 0], keys[1, 0, 1] = 1.0, 1.0
    q = torch.ones(1, nq, d)
    table = torch.tensor([[0.0, 2.0, -3.0], [1.0, 0.0, 0.5]])                   # distance 0 and 1, three heads
    kv, bt = _paged_keys(keys, page, seed=1)
    out = ops.paged_attention_generic(f32(q.view(1, nq * d)), kv.to(DEV), bt.to(DEV), torch.zeros(1, dtype=torch.int32, device=DEV),
                                      torch.ones(1, dtype=torch.int32, device=DEV), nq=nq, nkv=1, d=d, page_size=page,
                                      mask_kind=ops.MASK_FULL, mask_span=1, scale=0.125, dist_bias=table.to(DEV))
    out = out.cpu().view(nq, d)
    for h in range(nq):
        w_far = 1.0 / (1.0 + math.exp(float(table[0, h] - table[1, h])))       # weight of the key at distance 1
        assert out[h, 0].item() == pytest.approx(w_far, abs=1e-5) and out[h, 1].item() == pytest.approx(1 - w_far, abs=1e-5)


# ------------------------------------------------------------------------------------------
# one mixer (and its feed-forward) at a time, through the engine
# ------------------------------------------------------------------------------------------
_PLAIN_MIXER = {"latent_attention": lambda h, m, w, eps: plain.latent_attention(h, m, w, "l0.mix.", eps),
                "attention": lambda h, m, w, eps: plain.window_attention(h, m, w, "l0.mix."),
                "mamba2": lambda h, m, w, eps: plain.mamba2(h, m, w, "l0.mix.", eps)}


@pytest.mark.parametrize("name,index", [(n, i) for n in sorted(CASES) for i in range(len(CASES[n][0]["layers"]))])
def test_each_layer_alone(tmp_path, name, index):
    """A model of one layer: the residual stream behind it is the embedding plus the plain mixer's output (without a
    feed-forward), and plus the plain mixture's output (with the layer's own); a prompt of 150 tokens in one step, then
    the same prompt with its last 40 tokens one by one."""
    from latinex_models import one_layer, write_config
    from sharpinference_b200 import StepEntry
    _, std, seed = CASES[name]
    for variant, mlp in (("bare", None), ("own", "same")):
        cfg = one_layer(name, index, mlp)
        if variant == "own" and cfg["layers"][0]["mlp"] is None:
            continue
        folder = write_config(cfg, std, seed + index, str(tmp_path / variant))
        cfg, w = plain.load_folder(folder)
        toks = traces.random_tokens(cfg["vocab"], 150, seed=index)
        x0 = w["embed"][torch.tensor(toks)] * cfg["embedding"]["scale"]
        h = plain.dyt(x0, w["l0.norm1.alpha"], w["l0.norm1"], w["l0.norm1.b"])
        layer = cfg["layers"][0]
        want = x0 + _PLAIN_MIXER[layer["type"]](h, layer["mixer"], w, cfg["norm"]["eps"])
        if layer["mlp"] is not None:
            h2 = plain.dyt(want, w["l0.norm2.alpha"], w["l0.norm2"], w["l0.norm2.b"])
            want = want + plain.mixture(h2, layer["mlp"], w, "l0.mlp.")[0]
        eng = engine_for(folder, "float32", 256)
        eng.runner.trace_streams = True
        scale = float(want.abs().max())
        eng.open_request("a")
        eng.forward_step([StepEntry("a", toks, [])])
        got = eng.runner.last_layer_streams[0].double().cpu()
        assert float((got - want).abs().max()) < 3e-5 * scale, (variant, "prompt")
        eng.close_request("a")
        eng.open_request("b")
        eng.forward_step([StepEntry("b", toks[:110], [])])
        for t in range(110, 150):
            eng.forward_step([StepEntry("b", [toks[t]], [])])
            got = eng.runner.last_layer_streams[0].double().cpu()
            assert float((got[0] - want[t]).abs().max()) < 3e-5 * scale, (variant, "decoded", t)
        eng.close_request("b")


# ------------------------------------------------------------------------------------------
# whole models through the engine
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name", sorted(CASES))
def test_layers_one_after_the_other(folders, name):
    """The residual stream behind every layer of a whole model against the plain model's."""
    from sharpinference_b200 import StepEntry
    cfg, w = plain.load_folder(folders[name])
    toks = traces.random_tokens(cfg["vocab"], 140, seed=8)
    _, after, _ = plain.forward(cfg, w, toks, want_layers=True)
    eng = engine_for(folders[name], "float32", 256)
    eng.runner.trace_streams = True
    eng.open_request("a")
    eng.forward_step([StepEntry("a", toks, [])])
    for i, (got, want) in enumerate(zip(eng.runner.last_layer_streams, after)):
        assert float((got.double().cpu() - want).abs().max()) < 5e-5 * float(want.abs().max()), (i, cfg["layers"][i]["type"])
    eng.close_request("a")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_whole_prompts(folders, expected, name, dtype):
    run_and_compare(folders[name], name, dtype, traces.whole(requests_for(name)), expected)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_prompt_then_token_by_token(folders, expected, name, dtype):
    """The last 110 tokens one by one: windows of 1 to 100 positions pass wholly over decoded tokens, kept positions
    stay visible from decoded rows, and every recurrent state is carried through 110 single-row steps."""
    run_and_compare(folders[name], name, dtype, traces.tail_decode(requests_for(name), tail=110), expected)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_portions_down_to_two_tokens(folders, expected, name, dtype):
    run_and_compare(folders[name], name, dtype, traces.portions(requests_for(name)), expected)
    run_and_compare(folders[name], name, dtype, traces.portions(requests_for(name), sizes=(2, 2, 3, 64, 1, 63, 2, 33)),
                    expected, page_size=16)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CASES))
def test_mixed_batches_reuse_pages_and_slots(folders, expected, name, dtype):
    """Up to three live requests for three state slots and a pool sized for the schedule's peak: every later
    request runs in a slot and on pages that an earlier one left behind."""
    steps = traces.mixed(requests_for(name), max_live=3)
    eng = run_and_compare(folders[name], name, dtype, steps, expected, max_batch=3)
    assert eng.cache.state_slots.free_count == 3
    run_and_compare(folders[name], name, dtype, traces.drawn(requests_for(name), seed=5, max_live=4), expected)
    run_and_compare(folders[name], name, dtype, traces.drawn(requests_for(name), seed=6, max_live=4), expected, page_size=16)


@pytest.mark.parametrize("name", sorted(CASES))
def test_one_slot_used_again_starts_from_zero(folders, expected, name):
    """One state slot and one request's worth of pages for all requests in turn: the convolution's inputs, the
    recurrent state and the cached rows of the request before must be gone."""
    reqs = requests_for(name)
    eng = engine_for(folders[name], "float32", 256, max_batch=1)
    for rid, toks in reqs.items():
        got = traces.replay(eng, traces.whole({rid: toks}))
        err, where = traces.worst_error(got, expected[name])
        assert err < TOL["float32"], (rid, err, where)


@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_a_window_or_kept_count_one_position_off_would_show(folders, name):
    """The comparison is sharp enough: the plain model with every window one position longer or shorter, or with
    one kept position fewer, differs from the engine by far more than the tolerance, in prompts and in decoded
    tokens, once a sequence is longer than the window, and not at all before."""
    cfg, w = plain.load_folder(folders[name])
    windows = [c["mixer"]["mask"]["size"] for c in cfg["layers"] if c["type"] == "attention" and c["mixer"].get("mask")]
    reqs = {"r": traces.random_tokens(cfg["vocab"], 230, seed=77)}
    eng = engine_for(folders[name], "float32", 256)
    got = traces.replay(eng, traces.tail_decode(reqs, tail=80))
    right = {"r": plain.forward(cfg, w, reqs["r"])}
    assert traces.worst_error(got, right)[0] < TOL["float32"]
    scale = float(right["r"].abs().max())
    for kw in ({"window_delta": -1}, {"window_delta": 1}, {"keep_delta": -1}):
        wrong = plain.forward(cfg, w, reqs["r"], **kw)
        early = min(windows) + min(kw.get("window_delta", 0), 0)
        assert float((wrong[:early] - right["r"][:early]).abs().max()) / scale < 1e-9
        late_prompt = float((wrong[early:150] - right["r"][early:150]).abs().max()) / scale
        late_decode = float((wrong[150:] - right["r"][150:]).abs().max()) / scale
        assert late_prompt > 40 * TOL["float32"] and late_decode > 40 * TOL["float32"], (kw, late_prompt, late_decode)


def test_a_lost_state_or_far_key_would_show(folders, expected):
    """A far token matters: the plain model fed a request without its first 30 tokens differs at the request's end,
    200 tokens later, by far more than the tolerance (the recurrent memories, the kept positions and the latent
    attention reach that far back)."""
    for name, rid in (("E", "r4"), ("C", "r4"), ("B", "r3")):
        cfg, w = plain.load_folder(folders[name])
        toks = requests_for(name)[rid]
        full, cut = expected[name][rid], plain.forward(cfg, w, toks[30:])
        assert float((full[-1] - cut[-1]).abs().max()) / float(full.abs().max()) > 100 * TOL["float32"], name


def _aim(w, cfg, kind, marked, asking):
    """Edit one-layer weights so that the query of token ``asking`` meets the key of token ``marked`` with a score far
    above every other: a rank-one term in the key projection along what sets the marked token's normed embedding
    apart from the average one, and one in the query's for the asking token.  In latent attention the term goes into
    the rotated key part's last element, which the configuration leaves unrotated and which passes no norm."""
    m = cfg["layers"][0]["mixer"]
    h = plain.dyt(w["embed"] * cfg["embedding"]["scale"], w["l0.norm1.alpha"], w["l0.norm1"], w["l0.norm1.b"])
    vk, vq = h[marked] - h.mean(0), h[asking] - h.mean(0)
    if kind == "attention":
        d = m["dim"]
        w["l0.mix.k"][1] += 6.0 * vk / (vk @ vk)                               # element 1 of the one key head
        for hd in range(m["heads"]):
            w["l0.mix.q"][hd * d + 1] += 6.0 * vq / (vq @ vq)
    else:
        r, qr, d, dr = m["kv_rank"], m["q_rank"], m["dim"], m["rot_dim"]
        assert m["rot"]["dims"] < dr
        w["l0.mix.dkv"][r + dr - 1] += 6.0 * vk / (vk @ vk)
        w["l0.mix.dq"][0] += 40.0 * vq / (vq @ vq)                             # the asking token's query latent: along 0
        w["l0.mix.dq.norm"][0] = 1.0
        for hd in range(m["heads"]):
            w["l0.mix.uq"][hd * (d + dr) + d + dr - 1, 0] = 1.5               # times sqrt(q_rank) = 4 behind the norm
    return w


@pytest.mark.parametrize("kind", ["latent_attention", "attention"])
def test_a_far_key_among_hundreds_carries_the_output(tmp_path, kind):
    """One-layer models whose weights are edited so that the last token's query meets the key of one early token with
    a score far above all others: 400 positions back and across six pages, in a prompt's last row and in a decoded
    token.  Exchanging that early token then changes the layer's output at the end by a large part of its size.  For
    windowed attention the early token is a kept one; the same token one place later (not kept, outside the window)
    leaves no trace."""
    from latinex_models import _att, _lat, _top, write_config
    from safetensors.torch import save_file
    from sharpinference_b200 import StepEntry
    if kind == "latent_attention":
        layer = _lat(2, 8, 6, 8, 16, 16, 1.0, (4, 1000.0), None)
    else:
        layer = _att(2, 1, 16, 1.0, 8, 50, 40, 3, None)
    folder = write_config(_top(40, 32, 1e-5, 1.0, 1.0, [layer]), 0.3, 5, str(tmp_path / "base"))
    cfg, w = plain.load_folder(folder)
    w = _aim(w, cfg, kind, marked=37, asking=39)
    variant = str(tmp_path / "aimed")
    os.makedirs(variant)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(variant, "model.safetensors"))
    with open(os.path.join(variant, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    cfg, w = plain.load_folder(variant)
    n = 403
    eng = engine_for(variant, "float32", 512)
    for place, reaches in ((2, True), (3, kind == "latent_attention")):
        toks = [t % 30 for t in traces.random_tokens(30, n, seed=3)]
        toks[place], toks[-2], toks[-1] = 37, 39, 39                 # the asking token as a prompt's last row and decoded
        want, after, _ = plain.forward(cfg, w, toks, want_layers=True)
        other = plain.forward(cfg, w, toks[:place] + [5] + toks[place + 1:], want_layers=True)[1]
        for row in (n - 2, n - 1):
            moved = float((after[0][row] - other[0][row]).abs().max()) / float(after[0].abs().max())
            assert (moved > 0.05) == reaches, (place, row, moved)
            if not reaches:
                assert moved < 1e-12
        eng.open_request("a")
        lg = eng.forward_step([StepEntry("a", toks[:-1], [n - 2])]).double().cpu()
        assert float((lg[0] - want[n - 2]).abs().max()) < TOL["float32"] * float(want.abs().max()), place
        lg = eng.forward_step([StepEntry("a", toks[-1:], [0])]).double().cpu()
        assert float((lg[0] - want[n - 1]).abs().max()) < TOL["float32"] * float(want.abs().max()), place
        eng.close_request("a")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_long_decoding_through_graphs(folders, name, dtype):
    """Three requests decode 260 tokens each side by side, past every window's edge and over several pages;
    decode-only steps are replayed as CUDA graphs."""
    cfg, w = plain.load_folder(folders[name])
    reqs = {f"d{i}": traces.random_tokens(cfg["vocab"], 263 + i, seed=200 + i) for i in range(3)}
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": toks[:3 + i], "want": [2 + i]}
                                     for i, (rid, toks) in enumerate(reqs.items())], "end": []}]
    for t in range(260):
        steps.append({"step": t + 1, "entries": [{"id": rid, "tokens": [toks[3 + i + t]], "want": [0]}
                                                 for i, (rid, toks) in enumerate(reqs.items())],
                      "end": list(reqs) if t == 259 else []})
    eng = engine_for(folders[name], dtype, traces.max_tokens(steps))
    routing = {} if dtype == "bfloat16" else None
    got = traces.replay(eng, steps, routing)
    if routing is None:
        assert eng.runner.graph_replays > 200
        ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    else:
        ref = reference_for(folders[name], reqs, routing, None, dtype)
    err, where = traces.worst_error(got, ref)
    assert err < TOL[dtype], (err, where)


@pytest.mark.parametrize("name", sorted(CASES))
def test_greedy_generation_through_the_scheduler(folders, name):
    """``Engine.generate``: admission, portions under a small token budget, decoding in one batch, sampling
    (greedy) and the release of pages and slots, against the plain model generating token by token."""
    from sharpinference_b200 import Engine, EngineOptions, SamplingParams
    cfg, w = plain.load_folder(folders[name])
    prompts = [traces.random_tokens(cfg["vocab"], n, seed=300 + n) for n in (5, 41, 90, 17, 2)]
    opts = EngineOptions()
    opts.max_cache_tokens, opts.max_batch, opts.max_tokens_per_step = 1024, 3, 48
    eng = Engine(folders[name], dtype="float32", device=DEV, options=opts)
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_new_tokens=12))
    for prompt, out in zip(prompts, outs):
        assert out == plain.generate_greedy(cfg, w, prompt, 12)
    m = eng.metrics()
    assert m["state_slots_free"] == 3 and all(g["held"] == 0 for g in m["cache_groups"].values())


def test_command_line_and_trace_program(folders, capsys, tmp_path):
    """``sharpi-cli`` generates greedily on a Latinex folder, and ``bin/trace_run`` as a child process replays a mixed
    schedule from standard input and writes the logits the plain model gives."""
    import subprocess
    import sys

    import numpy as np

    from sharpinference_b200 import cli
    cfg, w = plain.load_folder(folders["C"])
    prompt = traces.random_tokens(cfg["vocab"], 21, seed=9)
    rc = cli.main(["-m", folders["C"], "--tokens", ",".join(map(str, prompt)), "-n", "6", "--temp", "0", "--dtype", "float32",
                   "--repeat-penalty", "1.0", "--json", "--max-cache-tokens", "256"])
    out = capsys.readouterr()
    assert rc == 0
    assert json.loads(out.out.strip().splitlines()[-1])["outputs"][0]["tokens"] == plain.generate_greedy(cfg, w, prompt, 6)

    reqs = {f"t{i}": traces.random_tokens(cfg["vocab"], n, seed=50 + i) for i, n in enumerate((40, 3, 77, 18, 166))}
    steps = traces.mixed(reqs, max_live=4)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    res = subprocess.run([sys.executable, os.path.join(root, "bin", "trace_run"), "--model", folders["C"], "--dtype", "float32",
                          "--out", str(tmp_path), "--max-tokens", str(traces.max_tokens(steps))],
                         input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True, text=True, timeout=900)
    assert res.returncode == 0, res.stderr[-2000:]
    assert [ln for ln in res.stdout.splitlines() if ln.startswith("done ")] == [f"done {s['step']}" for s in steps]
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    at = {rid: 0 for rid in reqs}
    for st in steps:
        rows = np.fromfile(os.path.join(str(tmp_path), f"{st['step']}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        r = 0
        for e in st["entries"]:
            for wpos in e["want"]:
                want = ref[e["id"]][at[e["id"]] + wpos]
                assert float((torch.from_numpy(rows[r]).double() - want).abs().max()) < TOL["float32"] * float(ref[e["id"]].abs().max())
                r += 1
            at[e["id"]] += len(e["tokens"])


def test_parts_are_registered_with_their_constants():
    from sharpinference_b200.parts import part_kinds
    assert {"latent_attention", "state_space_duality"} <= set(part_kinds("mixer"))
    assert "dynamic_tanh" in part_kinds("norm") and "moe_sigmoid_topk_gated" in part_kinds("feed_forward")
