"""Gisilix on the GPU: each new kernel against the plain statement of its mechanism, each mixer alone through a
one-layer model, and whole models through the engine (step function, cache manager, scheduler) under every way of
cutting the work, in 32-bit and in bfloat16."""
import copy
import json
import math
import os

import pytest
import torch

import plain_gisilix as plain
import traces
from gisilix_models import CASES, write

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
F64 = torch.float64

# Relative to the largest |logit| of a request.
TOL = {"float32": 5e-5, "bfloat16": 4e-2}
# A differing expert choice must be a near-tie of the router's logits.
MARGIN = 6e-2
LENGTHS = {"A": [1, 9, 40, 83, 150, 2], "B": [150, 5, 67, 200, 31], "C": [3, 70, 140, 45, 210, 64, 65],
           "D": [1, 2, 30, 5], "E": [140, 66, 3, 129, 230]}


def requests_for(name):
    vocab = CASES[name][0]["vocab"]
    return {f"r{i}": traces.random_tokens(vocab, n, seed=43 * i + n) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    return {name: write(name, str(tmp_path_factory.mktemp(f"gisilix_{name}"))) for name in CASES}


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


def reference_for(folder, reqs, routing, fallback, dtype, slack=None):
    """float32 runs are held to the plain logits as they are; bfloat16 runs to the plain logits under the engine's
    own expert choices, each differing choice having to be a near-tie of the plain router's logits.  ``slack`` (a
    dict) receives, per request, what rounding alone does to every position's logits in the plain model (the operands
    of its matrix products rounded to bfloat16), relative to the request's largest logit: large score factors make
    single positions sensitive, and a bfloat16 run is held to three times that where it exceeds the tolerance."""
    if dtype == "float32":
        return fallback
    cfg, w = plain.load_folder(folder)
    ref = {}
    for rid, toks in reqs.items():
        choices = [torch.tensor(per_layer, dtype=torch.long).view(len(toks), -1) for per_layer in routing[rid]]
        seen = []
        logits = plain.forward(cfg, w, toks, choices=choices, choices_out=seen)
        for (z, _), forced in zip(seen, choices):
            kth = z.topk(forced.shape[1], dim=-1).values[:, -1:]               # the smallest logit a free choice takes
            assert float((kth - z.gather(1, forced)).max()) < MARGIN * max(1.0, float(z.abs().max())), \
                f"request {rid}: an expert choice differs beyond a near-tie"
        ref[rid] = logits
        if slack is not None:
            rounded = plain.forward(cfg, w, toks, choices=choices, round_to=torch.bfloat16)
            slack[rid] = (rounded - logits).abs().max(dim=-1).values / float(logits.abs().max())
    return ref


def worst_excess(got, ref, tol, slack):
    """The largest error over the wanted rows as a multiple of what the row is allowed: ``tol``, or three times what
    rounding alone does at that position where that is more."""
    worst, where = 0.0, None
    for (rid, pos), row in got.items():
        err = float((row.double() - ref[rid][pos]).abs().max()) / float(ref[rid].abs().max())
        allowed = max(tol, 3.0 * float(slack[rid][pos])) if slack else tol
        if not err / allowed <= worst:
            worst, where = err / allowed, (rid, pos, err)
    return worst, where


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
    slack = {} if dtype == "bfloat16" else None
    ref = reference_for(folder, reqs, routing, expected[name] if expected else None, dtype, slack)
    excess, where = worst_excess(got, ref, TOL[dtype], slack)
    assert excess < 1.0, f"{name} {dtype}: {excess} times the allowed error at {where}"
    return eng


f32 = lambda t: t.float().to(DEV).contiguous()
i32 = lambda v: torch.tensor(v, dtype=torch.int32, device=DEV)


def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# ------------------------------------------------------------------------------------------
# kernels alone
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("H", [1, 16, 52, 257, 1024, 13000])
def test_layer_norm_with_the_residual_add(H):
    from sharpinference_b200.kernels import ops
    T = 11
    x, delta = 3 * _rand(T, H, seed=H) + 2.0, _rand(T, H, seed=H + 1)
    w, b = _rand(H, seed=H + 2), _rand(H, seed=H + 3)
    xd = f32(x)
    out, out32 = ops.add_layernorm(xd, f32(delta), f32(w), f32(b), 1e-5, torch.bfloat16, want_fp32=True)
    want = plain.layer_norm(x.float().double() + delta.float().double(), w.float().double(), b.float().double(), 1e-5)
    assert float((out32.double().cpu() - want).abs().max()) < 2e-5 * max(1.0, float(want.abs().max()))
    assert torch.equal(out, out32.to(torch.bfloat16))
    assert float((xd.double().cpu() - (x.float().double() + delta.float().double())).abs().max()) < 1e-6      # written back
    rows = i32([7, 0, 7, 3])
    keep = xd.clone()
    got, _ = ops.add_layernorm(xd, f32(delta), f32(w), None, 1e-5, torch.float32, rows=rows)
    again = plain.layer_norm(keep.double().cpu()[[7, 0, 7, 3]] + delta.float().double()[[7, 0, 7, 3]], w.float().double(), 0.0, 1e-5)
    assert float((got.double().cpu() - again).abs().max()) < 2e-5 * max(1.0, float(again.abs().max()))
    assert torch.equal(xd, keep)                                                   # gathered rows leave x alone


def _pages(keys, values, page, seed):
    """Keys [T, G, d] and values [T, G, d] of one request scattered over shuffled pages: (kv [P, 2, G, page, d], table)."""
    T, G, d = keys.shape
    n = (T + page - 1) // page
    order = torch.randperm(n + 3, generator=torch.Generator().manual_seed(seed))[:n]
    kv = torch.zeros(n + 3, 2, G, page, d)
    for t in range(T):
        kv[order[t // page], 0, :, t % page] = keys[t]
        kv[order[t // page], 1, :, t % page] = values[t]
    return kv, order.to(torch.int32).view(1, n)


@pytest.mark.parametrize("nq,nkv,d,page,cap", [(4, 2, 64, 64, 3.0), (2, 2, 128, 128, 0.0), (6, 1, 32, 16, 1.5), (3, 3, 48, 64, 5.0)])
def test_attention_kernels_with_cap_and_sinks(nq, nkv, d, page, cap):
    """The generic kernel (float32 and bfloat16), the tile kernels and the split kernel, with a cap that bends the
    largest scores and sinks of both signs, against the plain softmax with a sink; rows before, at and after block
    and split borders."""
    from sharpinference_b200.kernels import ops
    T, scale = 600, 2.0 / math.sqrt(d)
    q = _rand(T, nq, d, seed=d).to(torch.bfloat16)
    keys, values = _rand(T, nkv, d, seed=d + 1).to(torch.bfloat16), _rand(T, nkv, d, seed=d + 2).to(torch.bfloat16)
    sinks = torch.tensor([(-1) ** h * (0.5 + h) for h in range(nq)], dtype=torch.float32)
    s = torch.einsum("ihd,jhd->hij", q.double(), keys.double().repeat_interleave(nq // nkv, dim=1)) * scale
    assert float(s.abs().max()) > 1.5 * cap                     # the cap matters where there is one
    if cap:
        s = cap * torch.tanh(s / cap)
    p = plain.softmax_rows(s, plain.causal(T), sinks.double())
    want = torch.einsum("hij,jhd->ihd", p, values.double().repeat_interleave(nq // nkv, dim=1))
    assert float(1 - p.sum(-1).min()) > 0.02                    # and so do the sinks
    kv, bt = _pages(keys.float(), values.float(), page, seed=d)
    rr, pos = torch.zeros(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV)
    kw = dict(nq=nq, nkv=nkv, d=d, page_size=page, mask_kind=ops.MASK_FULL, mask_span=1, scale=scale, softcap=cap,
              sinks=sinks.to(DEV))
    got = ops.paged_attention_generic(f32(q.view(T, nq * d)), kv.to(DEV), bt.to(DEV), rr, pos, **kw)
    assert float((got.double().cpu().view(T, nq, d) - want).abs().max()) < 2e-5
    qb, kvb = q.to(DEV).view(T, nq * d).contiguous(), kv.to(torch.bfloat16).to(DEV)
    got = ops.paged_attention_generic(qb, kvb, bt.to(DEV), rr, pos, **kw)
    assert float((got.double().cpu().view(T, nq, d) - want).abs().max()) < 2e-2
    tiles = i32([[t0, min(64, T - t0), t0, 0] for t0 in range(0, T, 64)])
    out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_prefill(qb.view(T, nq, d), kvb, bt.to(DEV), tiles, out, **kw)
    assert float((out.double().cpu().view(T, nq, d) - want).abs().max()) < 2e-2
    if ops.tc_prefill_supported(torch.bfloat16, d, page):
        tiles = i32([[t0, min(128, T - t0), t0, 0] for t0 in range(0, T, 128)])
        out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device=DEV)
        ops.attention_prefill_tc(qb.view(T, nq, d), kvb, bt.to(DEV), tiles, out, **kw)
        ops.check_status(DEV)
        assert float((out.double().cpu().view(T, nq, d) - want).abs().max()) < 2e-2
    rows = [0, 1, 63, 64, 255, 256, 257, 511, 512, 599]
    out = torch.zeros(T, nq * d, dtype=torch.bfloat16, device=DEV)
    ops.attention_decode(qb.view(T, nq, d), kvb, bt.to(DEV), rr, pos, out, rows=i32(rows), num_rows=len(rows),
                         max_context=T, **kw)
    ops.check_status(DEV)
    assert float((out.double().cpu().view(T, nq, d)[rows] - want[rows]).abs().max()) < 2e-2


def test_a_sink_far_above_every_score_empties_the_row():
    """A sink of 60 beside scores around zero: the row's weights sum to about e^-60 and the output is zero, with no
    overflow on the way; a sink of -60 changes nothing."""
    from sharpinference_b200.kernels import ops
    T, nq, d, page = 70, 2, 64, 64
    q, keys, values = _rand(T, nq, d, seed=1, scale=0.1), _rand(T, 1, d, seed=2, scale=0.1), _rand(T, 1, d, seed=3)
    kv, bt = _pages(keys.float(), values.float(), page, seed=4)
    rr, pos = torch.zeros(T, dtype=torch.int32, device=DEV), torch.arange(T, dtype=torch.int32, device=DEV)
    sinks = torch.tensor([60.0, -60.0], device=DEV)
    kw = dict(nq=nq, nkv=1, d=d, page_size=page, mask_kind=ops.MASK_FULL, mask_span=1, scale=1.0, sinks=sinks)
    free = dict(kw, sinks=None)
    a = ops.paged_attention_generic(f32(q.view(T, nq * d)), kv.to(DEV), bt.to(DEV), rr, pos, **kw).view(T, nq, d)
    b = ops.paged_attention_generic(f32(q.view(T, nq * d)), kv.to(DEV), bt.to(DEV), rr, pos, **free).view(T, nq, d)
    assert float(a[:, 0].abs().max()) < 1e-20 and bool(torch.isfinite(a).all()) and torch.allclose(a[:, 1], b[:, 1], atol=1e-6)
    qb, kvb = q.to(torch.bfloat16).to(DEV).contiguous(), kv.to(torch.bfloat16).to(DEV)
    for run in ("tiles", "tc", "rows"):
        out = torch.ones(T, nq * d, dtype=torch.bfloat16, device=DEV)
        if run == "tiles":
            ops.attention_prefill(qb, kvb, bt.to(DEV), i32([[0, 64, 0, 0], [64, 6, 64, 0]]), out, **kw)
        elif run == "tc":
            ops.attention_prefill_tc(qb, kvb, bt.to(DEV), i32([[0, 70, 0, 0]]), out, **kw)
        else:
            ops.attention_decode(qb, kvb, bt.to(DEV), rr, pos, out, rows=None, num_rows=T, max_context=T, **kw)
        o = out.float().view(T, nq, d)
        assert float(o[:, 0].abs().max()) < 1e-20 and bool(torch.isfinite(o).all()), run
        assert float((o[:, 1] - b[:, 1]).abs().max()) < 2e-2, run


@pytest.mark.parametrize("nq,nkv,d,count_d,page,borrow,pad", [
    (4, 2, 16, 16, 16, False, 5), (4, 2, 16, 16, 16, False, 8), (3, 3, 10, 10, 4, False, 5), (2, 1, 32, 24, 8, False, 4),
    (4, 1, 64, 64, 64, True, 5), (4, 1, 64, 64, 64, True, 12), (16, 4, 128, 128, 64, False, 8), (32, 8, 128, 128, 16, False, 0),
    (72, 8, 128, 128, 64, False, 4)])
def test_norm_over_the_whole_projection_and_cache_write(nq, nkv, d, count_d, page, borrow, pad):
    """q and k as wholes are divided by their root mean square (the mean over ``count_d`` elements a head where heads
    are padded), weighted, q is multiplied by the position's factor, and k and v land in the rows' pages.  Rows that
    are 16-byte aligned take the form of the kernel that holds the row in registers (2, 4 or 8 pieces a thread), the
    others and rows beyond 8192 floats the one that reads the row twice."""
    from sharpinference_b200.kernels import ops
    T, eps, coef, every = 40, 1e-5, 0.4, 7.0
    width = nq * d + (0 if borrow else 2 * nkv * d)
    core = _rand(T, width, seed=d, scale=2.0).float()
    if count_d < d:                                                             # padded heads hold zeros
        core.view(T, -1, d)[:, :, count_d:] = 0
    qkv = torch.cat([core, _rand(T, pad, seed=9).float()], dim=1)               # a column range of a wider product
    wq, wk = _rand(nq * d, seed=1).float(), _rand(nkv * d, seed=2).float()
    pos = torch.tensor([(3 * t) % 37 for t in range(T)], dtype=torch.int32)
    reqs = torch.tensor([t % 2 for t in range(T)], dtype=torch.int32)
    table = torch.tensor([[5, 1, 7, 0, 9, 2, 11, 3, 12, 13], [4, 6, 8, 10, 14, 15, 16, 17, 18, 19]], dtype=torch.int32)
    kv = torch.full((20, 2, nkv, page, d), 7.0, device=DEV)
    q_out = torch.empty(T, nq, d, device=DEV)
    src = qkv.to(DEV)
    ops.qkv_post_wide(src[:, :width], pos.to(DEV), reqs.to(DEV), table.to(DEV), q_out, kv, nq=nq, nkv=nkv, d=d, page_size=page,
                      q_weight=wq.to(DEV), k_weight=None if borrow else wk.to(DEV), eps=eps, q_count=nq * count_d,
                      k_count=nkv * count_d, temp_coef=coef, temp_every=every, write_kv=not borrow, has_kv=not borrow)
    x = qkv.double()
    q = x[:, : nq * d]
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) / (nq * count_d) + eps) * wq.double()
    q = q * (1 + coef * torch.log(torch.floor((pos.double() + 1) / every) + 1)).view(T, 1)
    assert float((q_out.double().cpu().view(T, -1) - q).abs().max()) < 1e-5
    if borrow:
        assert float((kv - 7.0).abs().max()) == 0.0
        return
    k = x[:, nq * d: (nq + nkv) * d]
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) / (nkv * count_d) + eps) * wk.double()
    v = x[:, (nq + nkv) * d: width]
    want = torch.full((20, 2, nkv, page, d), 7.0, dtype=F64)
    for t in range(T):                                                          # no place is written twice
        pg, at = int(table[reqs[t], int(pos[t]) // page]), int(pos[t]) % page
        want[pg, 0, :, at] = k[t].view(nkv, d)
        want[pg, 1, :, at] = v[t].view(nkv, d)
    assert float((kv.double().cpu() - want).abs().max()) < 1e-5


@pytest.mark.parametrize("T,H,E,k", [(1, 64, 4, 2), (37, 52, 3, 3), (600, 128, 12, 3), (5, 16, 1, 1), (9, 96, 40, 5)])
def test_router_with_a_bias_and_the_softmax_over_the_chosen(T, H, E, k):
    from sharpinference_b200.kernels import ops
    h, wr, b = _rand(T, H, seed=T).float(), _rand(E, H, seed=E, scale=0.3).float(), _rand(E, seed=k, scale=2.0).float()
    expert, weight, z = ops.router_topk(h.to(DEV), wr.to(DEV), k, bias=b.to(DEV), scoring="softmax_chosen", want_scores=True)
    want_z = h.double() @ wr.double().T + b.double()
    assert float((z.double().cpu() - want_z).abs().max()) < 1e-4
    val, idx = want_z.topk(k, dim=-1)
    got_idx = expert.cpu().long()
    differ = (got_idx != idx).any(-1)
    for t in differ.nonzero().flatten().tolist():                               # only a tie within rounding may differ
        assert float((val[t] - want_z[t].gather(0, got_idx[t])).abs().max()) < 1e-4
    same = ~differ
    assert float((weight.double().cpu()[same] - torch.softmax(val, -1)[same]).abs().max()) < 1e-5
    assert float((weight.sum(-1) - 1).abs().max()) < 1e-5
    # without the bias the choice follows the plain logits, and the sigmoid scoring is unchanged by the new arguments
    e2, w2, _ = ops.router_topk(h.to(DEV), wr.to(DEV), k)
    s = torch.sigmoid(h.double() @ wr.double().T)
    sv, si = s.topk(k, dim=-1)
    ok = (e2.cpu().long() == si).all(-1)
    assert float(ok.float().mean()) > 0.95 and float((w2.double().cpu()[ok] - sv[ok]).abs().max()) < 1e-5


def test_latent_helpers_take_column_ranges_an_amplitude_and_a_head_gate():
    from sharpinference_b200.kernels import ops
    T, H, dim, rot, rank, D = 9, 3, 4, 6, 5, 16
    wide = _rand(T, H * (dim + rot) + 7, seed=1).float().to(DEV)
    q = wide[:, : H * (dim + rot)]
    qa = _rand(H * T, rank, seed=2).float().to(DEV)
    pos = torch.arange(3, 3 + T, dtype=torch.int32, device=DEV)
    inv = torch.tensor([0.7, 0.05], device=DEV)
    got = ops.latent_q_join(qa, q, pos, inv, heads=H, dim=dim, rank=rank, rot=rot, rot_dims=4, D=D, out_dtype=torch.float32,
                            rot_amplitude=1.3).double().cpu()
    qr = q.double().cpu().view(T, H, dim + rot)[..., dim:]
    a = pos.double().cpu().view(T, 1, 1) * inv.double().cpu()
    want = qr.clone()
    want[..., 0:4:2] = 1.3 * (qr[..., 0:4:2] * torch.cos(a) - qr[..., 1:4:2] * torch.sin(a))
    want[..., 1:4:2] = 1.3 * (qr[..., 1:4:2] * torch.cos(a) + qr[..., 0:4:2] * torch.sin(a))
    assert float((got[..., rank: rank + rot] - want).abs().max()) < 1e-5          # the last two elements pass unscaled
    assert torch.equal(got[..., :rank], qa.double().cpu().view(H, T, rank).transpose(0, 1))
    assert float(got[..., rank + rot:].abs().max()) == 0.0
    plainq = ops.head_major(q, heads=H, stride=dim + rot, col0=0, n=dim, out_dtype=torch.float32).cpu()
    assert torch.equal(plainq.view(H, T, dim), q.cpu().view(T, H, dim + rot)[..., :dim].transpose(0, 1))
    v = _rand(H * T, 4, seed=3).float().to(DEV)
    gate = wide[:, H * (dim + rot): H * (dim + rot) + H]
    out = ops.head_minor(v, heads=H, out_dtype=torch.float32, gate=gate).double().cpu().view(T, H, 4)
    want = v.double().cpu().view(H, T, 4).transpose(0, 1) * torch.sigmoid(gate.double().cpu()).view(T, H, 1)
    assert float((out - want).abs().max()) < 1e-6


# ------------------------------------------------------------------------------------------
# one mixer (and its feed-forward) at a time, through the engine
# ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("name,index", [(n, i) for n in sorted(CASES) for i in range(len(CASES[n][0]["layers"]))])
def test_each_layer_alone(tmp_path, name, index):
    """A model of one layer (a borrowing layer behind the layer it borrows from): the residual stream behind it against
    the plain mixer's and feed-forward's outputs; a prompt of 150 tokens in one step, then the same prompt with its
    last 40 tokens one by one."""
    from gisilix_models import one_layer, write_config
    from sharpinference_b200 import StepEntry
    _, std, seed = CASES[name]
    for variant, mlp in (("bare", None), ("own", "same")):
        cfg = one_layer(name, index, mlp)
        if variant == "own" and cfg["layers"][-1]["mlp"] is None:
            continue
        folder = write_config(cfg, std, seed + index, str(tmp_path / variant))
        cfg, w = plain.load_folder(folder)
        toks = traces.random_tokens(cfg["vocab"], 150, seed=index)
        after = []
        plain.forward(cfg, w, toks, layers_out=after)
        # the last layer by hand from its mechanism's function
        x = after[-2] if len(after) > 1 else w["embed"][torch.tensor(toks)]
        last = len(cfg["layers"]) - 1
        layer, p = cfg["layers"][last], f"l{last}."
        h = plain.layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], cfg["norm"]["eps"])
        if layer["type"] == "attention":
            kv = None
            if last:
                h0 = plain.layer_norm(w["embed"][torch.tensor(toks)], w["l0.norm1"], w["l0.norm1.b"], cfg["norm"]["eps"])
                kv = plain.attention_keys_values(h0, cfg["layers"][0]["mixer"], w, "l0.mix.", cfg["norm"]["eps"])
            want = x + plain.attention(h, layer["mixer"], w, p + "mix.", cfg["norm"]["eps"], kv=kv)
        else:
            want = x + plain.latent_attention(h, layer["mixer"], w, p + "mix.", cfg["norm"]["eps"])
        if layer["mlp"] is not None:
            h2 = plain.layer_norm(want, w[p + "norm2"], w[p + "norm2.b"], cfg["norm"]["eps"])
            want = want + plain.feed_forward(h2, layer["mlp"], w, p + "mlp.")[0]
        assert float((want - after[-1]).abs().max()) < 1e-9
        eng = engine_for(folder, "float32", 256)
        eng.runner.trace_streams = True
        scale = float(want.abs().max())
        eng.open_request("a")
        eng.forward_step([StepEntry("a", toks, [])])
        got = eng.runner.last_layer_streams[-1].double().cpu()
        assert float((got - want).abs().max()) < 3e-5 * scale, (variant, "prompt")
        eng.close_request("a")
        eng.open_request("b")
        eng.forward_step([StepEntry("b", toks[:110], [])])
        for t in range(110, 150):
            eng.forward_step([StepEntry("b", [toks[t]], [])])
            got = eng.runner.last_layer_streams[-1].double().cpu()
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
    after = []
    plain.forward(cfg, w, toks, layers_out=after)
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
    """The last 110 tokens one by one: windows of 1 to 100 positions pass wholly over decoded tokens, the query factor
    changes several times among them, and the borrowing layers read what single-row steps of their sources wrote."""
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
    """Up to three live requests for three slots and a pool sized for the schedule's peak: every later request runs
    on pages that an earlier one left behind."""
    steps = traces.mixed(requests_for(name), max_live=3)
    eng = run_and_compare(folders[name], name, dtype, steps, expected, max_batch=3)
    assert eng.cache.state_slots.free_count == 3
    run_and_compare(folders[name], name, dtype, traces.drawn(requests_for(name), seed=5, max_live=4), expected)
    run_and_compare(folders[name], name, dtype, traces.drawn(requests_for(name), seed=6, max_live=4), expected, page_size=16)


@pytest.mark.parametrize("name", sorted(CASES))
def test_pages_used_again_hold_nothing_of_the_request_before(folders, expected, name):
    """One request's worth of pages for all requests in turn."""
    reqs = requests_for(name)
    eng = engine_for(folders[name], "float32", 256, max_batch=1)
    for rid, toks in reqs.items():
        got = traces.replay(eng, traces.whole({rid: toks}))
        err, where = traces.worst_error(got, expected[name])
        assert err < TOL["float32"], (rid, err, where)


@pytest.mark.parametrize("name", ["A", "C", "E"])
def test_a_window_one_position_off_would_show(folders, name):
    """The comparison is sharp enough: the plain model with every window one position longer or shorter differs from
    the engine by far more than the tolerance, in prompts and in decoded tokens, once a sequence is longer than the
    window, and not at all before."""
    cfg, w = plain.load_folder(folders[name])
    windows = [c["mixer"]["mask"]["size"] for c in cfg["layers"] if c["mixer"].get("mask")]
    reqs = {"r": traces.random_tokens(cfg["vocab"], 230, seed=77)}
    eng = engine_for(folders[name], "float32", 256)
    got = traces.replay(eng, traces.tail_decode(reqs, tail=80))
    right = {"r": plain.forward(cfg, w, reqs["r"])}
    assert traces.worst_error(got, right)[0] < TOL["float32"]
    scale = float(right["r"].abs().max())
    for delta in (-1, 1):
        other = copy.deepcopy(cfg)
        for c in other["layers"]:
            if c["mixer"].get("mask"):
                c["mixer"]["mask"]["size"] += delta
        wrong = plain.forward(other, w, reqs["r"])
        early = min(windows) + min(delta, 0)
        assert float((wrong[:early] - right["r"][:early]).abs().max()) / scale < 1e-9
        late_prompt = float((wrong[early:150] - right["r"][early:150]).abs().max()) / scale
        late_decode = float((wrong[150:] - right["r"][150:]).abs().max()) / scale
        assert late_prompt > 20 * TOL["float32"] and late_decode > 20 * TOL["float32"], (delta, late_prompt, late_decode)


def _aim(w, cfg, marked, asking, layer=0):
    """Edit a layer's weights so that the query of token ``asking`` meets the key of token ``marked`` with a score far
    above every other: a rank-one term in the key projection along what sets the marked token's normed embedding apart
    from the average one, and one in the query's for the asking token.  In latent attention the term goes into the
    rotated key part's last element, which the configuration leaves unrotated and which passes no norm."""
    m, p = cfg["layers"][layer]["mixer"], f"l{layer}.mix."
    h = plain.layer_norm(w["embed"], w[f"l{layer}.norm1"], w[f"l{layer}.norm1.b"], cfg["norm"]["eps"])
    vk, vq = h[marked] - h.mean(0), h[asking] - h.mean(0)
    if cfg["layers"][layer]["type"] == "attention":
        d = m["dim"]
        w[p + "k"][1] += 8.0 * vk / (vk @ vk)                                   # element 1 of the first key head
        w[p + "k.norm"][1] = 1.0
        for hd in range(m["heads"]):
            w[p + "q"][hd * d + 1] += 40.0 * vq / (vq @ vq)
            w[p + "q.norm"][hd * d + 1] = 1.0
    else:
        r, d, dr = m["kv_rank"], m["dim"], m["rot_dim"]
        assert m["rot"]["dims"] < dr
        w[p + "dkv"][r + dr - 1] += 6.0 * vk / (vk @ vk)
        for hd in range(m["heads"]):
            w[p + "q"][hd * (d + dr) + d + dr - 1] += 6.0 * vq / (vq @ vq)
    return w


@pytest.mark.parametrize("kind", ["attention", "borrowed", "latent"])
def test_a_far_key_among_hundreds_carries_the_output(tmp_path, kind):
    """Models whose weights are edited so that the last token's query meets the key of one early token with a score far
    above all others: 400 positions back and across six pages, in a prompt's last row and in a decoded token.
    Exchanging that early token then changes the layer's output at the end by a visible part of its size.  For the
    windowed latent layer a token outside the window leaves no trace, the first one inside it does, and the place
    before that is seen by the prompt's last row and not by the decoded one."""
    from gisilix_models import att, lat2, top, write_config
    from safetensors.torch import save_file
    from sharpinference_b200 import StepEntry
    if kind == "latent":
        layers = [lat2(2, 8, 6, 8, 16, 1.0, (4, 1000.0, (4.0, 32, 4.0, 1.0)), 300, None)]
    elif kind == "attention":
        layers = [att(2, 1, 16, 16, 0.6, 50.0, (0.3, 64), None)]
    else:
        layers = [att(2, 1, 16, 16, 0.6, 50.0, (0.3, 64), None), att(2, 1, 16, 16, 0.6, 50.0, (0.3, 64), None, kv_from=0)]
    folder = write_config(top(40, 32, 1e-5, layers), 0.3, 5, str(tmp_path / "base"))
    cfg, w = plain.load_folder(folder)
    w = _aim(w, cfg, marked=37, asking=39, layer=0)
    if kind == "borrowed":                       # the second layer asks with its own queries, of the first layer's keys
        w["l0.mix.o"] *= 0.0                     # its input is the embedding again: the aimed query fits
        w["l1.mix.q"], w["l1.mix.q.norm"] = w["l0.mix.q"].clone(), w["l0.mix.q.norm"].clone()
        w["l1.norm1"], w["l1.norm1.b"] = w["l0.norm1"].clone(), w["l0.norm1.b"].clone()
    variant = str(tmp_path / "aimed")
    os.makedirs(variant)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in w.items()}, os.path.join(variant, "model.safetensors"))
    with open(os.path.join(variant, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    cfg, w = plain.load_folder(variant)
    n = 403
    eng = engine_for(variant, "float32", 512)
    for place in (2, n - 300, n - 301):          # far back; the first place the last row's window holds; the one before
        toks = [t % 30 for t in traces.random_tokens(30, n, seed=3)]
        toks[place], toks[-2], toks[-1] = 37, 39, 39                 # the asking token as a prompt's last row and decoded
        after, other = [], []
        want = plain.forward(cfg, w, toks, layers_out=after)
        plain.forward(cfg, w, toks[:place] + [5] + toks[place + 1:], layers_out=other)
        for row in (n - 2, n - 1):
            reaches = kind != "latent" or row - place < 300
            moved = float((after[-1][row] - other[-1][row]).abs().max()) / float(after[-1].abs().max())
            assert (moved > 0.01) == reaches, (place, row, moved)
            if not reaches:
                assert moved < 1e-12
        eng.open_request("a")
        lg = eng.forward_step([StepEntry("a", toks[:-1], [n - 2])]).double().cpu()
        assert float((lg[0] - want[n - 2]).abs().max()) < TOL["float32"] * float(want.abs().max()), place
        lg = eng.forward_step([StepEntry("a", toks[-1:], [0])]).double().cpu()
        assert float((lg[0] - want[n - 1]).abs().max()) < TOL["float32"] * float(want.abs().max()), place
        eng.close_request("a")


@pytest.mark.parametrize("seed", [3, 14, 15, 92, 65])
def test_drawn_configurations(tmp_path, seed):
    """Configurations drawn at random (layer order, sizes, windows, constants) with requests of 2 to 700 tokens: whole,
    with decoded tails, and in drawn mixed batches, in 32-bit; bfloat16 whole, held to what rounding does."""
    from gisilix_models import drawn_config, write_config
    cfg = drawn_config(seed)
    folder = write_config(cfg, 0.1, seed, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    reqs = {f"q{i}": traces.random_tokens(cfg["vocab"], n, seed=seed * 7 + i) for i, n in enumerate([330, 37, 150, 700, 2])}
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    for steps in (traces.whole(reqs), traces.tail_decode(reqs, tail=40), traces.drawn(reqs, seed=seed, max_live=4)):
        eng = engine_for(folder, "float32", traces.max_tokens(steps))
        err, where = traces.worst_error(traces.replay(eng, steps), ref)
        eng.runner.flush_status()
        assert err < TOL["float32"], (err, where)
    steps = traces.whole(reqs)
    eng = engine_for(folder, "bfloat16", traces.max_tokens(steps))
    routing, slack = {}, {}
    got = traces.replay(eng, steps, routing)
    excess, where = worst_excess(got, reference_for(folder, reqs, routing, None, "bfloat16", slack), TOL["bfloat16"], slack)
    assert excess < 2.0, (excess, where)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_latent_row_longer_than_the_tensor_core_kernels_take(tmp_path, dtype):
    """A latent of 560 with 16 rotated elements: a cached row of 576 elements runs the general attention kernel in both
    precisions, whole, in portions and token by token."""
    from gisilix_models import lat2, top, write_config
    cfg = top(40, 64, 1e-5, [lat2(2, 16, 16, 24, 560, 0.3, (16, 1000.0, (4.0, 64, 8.0, 1.0)), 90, None)])
    folder = write_config(cfg, 0.1, 7, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    reqs = {"a": traces.random_tokens(40, 150, seed=1), "b": traces.random_tokens(40, 70, seed=2)}
    ref = {rid: plain.forward(cfg, w, toks) for rid, toks in reqs.items()}
    for steps in (traces.whole(reqs), traces.mixed(reqs, max_live=2, tail=40)):
        eng = engine_for(folder, dtype, traces.max_tokens(steps))
        err, where = traces.worst_error(traces.replay(eng, steps), ref)
        assert err < TOL[dtype], (err, where)


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
        slack = {}
        ref = reference_for(folders[name], reqs, routing, None, dtype, slack)
    excess, where = worst_excess(got, ref, TOL[dtype], slack if routing is not None else None)
    assert excess < 1.0, (excess, where)


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
    """``sharpi-cli`` generates greedily on a Gisilix folder, and ``bin/trace_run`` as a child process replays a mixed
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
    assert "layernorm" in part_kinds("norm") and "latent_attention" in part_kinds("mixer")
