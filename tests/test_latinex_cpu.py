"""Latinex without a GPU: the configuration reader, the tensor declaration, the pages and state that the cache manager
hands to the layers, the distance table, and the plain implementation checked against each mechanism's defining
property."""
import copy
import math

import pytest
import torch

import plain_latinex as plain
import traces
from latinex_models import CASE_A, CASE_B, CASE_C, CASE_D, CASE_E, CASES, write

from sharpinference_b200.config import ConfigError, LatinexConfig
from sharpinference_b200.registry import get_architecture, resolve
from sharpinference_b200.weights.loading import declared_tensors

F64 = torch.float64


def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# -- configuration -------------------------------------------------------------------------
@pytest.mark.parametrize("case", [CASE_A, CASE_B, CASE_C, CASE_D, CASE_E])
def test_config_round_trip(case):
    arch, cfg = resolve(copy.deepcopy(case), "test")
    assert arch.name == "Latinex" and isinstance(cfg, LatinexConfig)
    assert LatinexConfig.from_dict(cfg.to_dict()) == cfg
    assert [layer.type for layer in cfg.layers] == [c["type"] for c in case["layers"]]
    assert cfg.eps == case["norm"]["eps"] and cfg.embedding_scale == case["embedding"]["scale"]
    for layer, raw in zip(cfg.layers, case["layers"]):
        assert (layer.mlp is None) == (raw["mlp"] is None)
        if raw["mlp"]:
            assert (layer.mlp.experts, layer.mlp.top) == (raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"])
            assert layer.mlp.shared_ff == (raw["mlp"]["shared"] or {"ff": 0})["ff"]


def test_defaults_of_absent_keys():
    case = copy.deepcopy(CASE_A)
    lat, att, ssd = (layer["mixer"] for layer in case["layers"])
    del lat["scale"], lat["rot"], lat["vdim"]
    del att["kv_heads"], att["mask"], att["scale"], att["vdim"]
    del ssd["groups"], ssd["norm_groups"]
    del case["embedding"], case["logit_scale"]
    _, cfg = resolve(case, "test")
    a, b, c = cfg.layers
    assert a.scale == pytest.approx((16 + 8) ** -0.5) and a.rot_dims == 0 and a.vdim == 16
    assert b.kv_heads == 4 and b.window == 0 and b.keep_first == 0 and b.scale == pytest.approx(0.25) and b.vdim == 16
    assert c.groups == 1 and c.norm_groups == 1
    assert cfg.embedding_scale == 1.0 and cfg.logit_scale == 1.0


def test_config_problems_are_listed_together():
    bad = copy.deepcopy(CASE_A)
    del bad["width"]
    bad["layers"][0]["mixer"]["rot"]["dims"] = 10               # beyond rot_dim
    bad["layers"][1]["mixer"]["kv_heads"] = 3                   # 4 heads are no multiple of 3
    bad["layers"][2]["mixer"]["norm_groups"] = 5                # does not divide heads * vdim
    bad["layers"][0]["mlp"]["router"]["top"] = 9                # more than there are experts
    bad["layers"].append({"type": "conv", "mixer": {}, "mlp": None})
    with pytest.raises(ConfigError) as err:
        resolve(bad, "test")
    text = str(err.value)
    for piece in ("width", "rot.dims", "kv_heads", "norm_groups", "router.top", "conv"):
        assert piece in text, (piece, text)


def test_declared_tensors_follow_the_configuration():
    arch = get_architecture("Latinex")
    _, cfg = resolve(copy.deepcopy(CASE_A), "test")
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg)}
    assert decls["embed"] == (97, 64) and decls["head"] == (97, 64) and decls["final.norm.alpha"] == ()
    assert decls["l0.norm1"] == (64,) and decls["l0.norm2.b"] == (64,)
    assert decls["l0.mix.dq"] == (32, 64) and decls["l0.mix.uq"] == (4 * 24, 32) and decls["l0.mix.dkv"] == (48, 64)
    assert decls["l0.mix.dkv.norm"] == (40,) and decls["l0.mix.uk"] == (64, 40) and decls["l0.mix.uv"] == (96, 40)
    assert decls["l0.mix.o"] == (64, 96)
    assert decls["l0.mlp.router"] == (4, 64) and decls["l0.mlp.e3.gate"] == (24, 64) and decls["l0.mlp.e0.down"] == (64, 24)
    assert decls["l0.mlp.shared.up"] == (40, 64) and "l1.mlp.shared.up" not in decls and "l0.mlp.e4.gate" not in decls
    assert decls["l1.mix.q"] == (64, 64) and decls["l1.mix.k"] == (32, 64) and decls["l1.mix.k.b"] == (32,)
    assert decls["l1.mix.rel"] == (8, 4) and decls["l1.mix.g"] == (64, 64) and "l1.mix.v" not in decls
    assert decls["l2.mix.in"] == (2 * 32 + 2 * 2 * 16 + 4, 64) and decls["l2.mix.conv"] == (32 + 64, 3)
    assert decls["l2.mix.A_log"] == (4,) and decls["l2.mix.norm"] == (32,) and decls["l2.mix.o"] == (64, 32)
    assert not any(n.startswith("l2.mlp") for n in decls)


def test_the_distance_table_size_comes_from_the_stored_tensor_when_the_configuration_is_silent():
    arch = get_architecture("Latinex")
    case = copy.deepcopy(CASE_A)
    del case["layers"][1]["mixer"]["bias_buckets"]
    _, cfg = resolve(case, "test")
    with pytest.raises(ValueError, match="rel"):
        declared_tensors(arch, cfg)
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg, stored_names={"l1.mix.rel": (12, 4)})}
    assert decls["l1.mix.rel"] == (12, 4)


def test_pages_and_state_in_the_cache_manager():
    """A latent layer caches one row a token in keys-only pages, a windowed layer its keys only with the kept
    positions in its group's rule, a state-space layer holds matrix state and convolution inputs; a slot that is
    handed out again is zero."""
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.weights.source import DeclaringWeights
    arch = get_architecture("Latinex")
    _, cfg = resolve(copy.deepcopy(CASE_A), "test")
    model = arch.build(cfg, DeclaringWeights(torch.float32))
    cache = CacheManager(model.schedule, model.blocks, page_size=4, num_pages=8, max_requests=2, dtype=torch.float32,
                         device="cpu", model_state_specs=model.state_specs)
    specs = sorted((g.spec.kind, g.spec.span, g.spec.num_kv_heads, g.spec.head_dim, g.spec.planes, g.spec.keep_first)
                   for g in cache.groups)
    assert specs == [("full", 0, 1, 48, 1, 0), ("window", 33, 2, 16, 1, 5)]
    slots = cache.layer_slots()
    assert set(slots[2].states) == {"S", "conv"} and not slots[0].states and not slots[1].states
    assert slots[2].states["S"].shape == (2, 4 * 16 * 8) and slots[2].states["conv"].shape == (2, 2 * (32 + 64))
    a = cache.add_request("a")
    for t in slots[2].states.values():
        t[a.state_slot] = 3
    cache.free_request("a")
    b = cache.add_request("b")
    assert b.state_slot == a.state_slot
    assert all(float(t[b.state_slot].abs().sum()) == 0 for t in slots[2].states.values())


def test_a_window_with_kept_positions_holds_their_pages():
    """Pages that lie wholly between the kept positions and the window are given back; the kept ones stay."""
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.weights.source import DeclaringWeights
    arch = get_architecture("Latinex")
    _, cfg = resolve(copy.deepcopy(CASE_A), "test")
    model = arch.build(cfg, DeclaringWeights(torch.float32))
    cache = CacheManager(model.schedule, model.blocks, page_size=4, num_pages=64, max_requests=2, dtype=torch.float32,
                         device="cpu", model_state_specs=model.state_specs)
    group = next(i for i, g in enumerate(cache.groups) if g.spec.kind == "window")
    rc = cache.add_request("a")
    at = 0
    for n in (30, 1, 1, 40, 1, 1, 1, 57, 1):
        cache.reserve([("a", n)])
        cache.commit("a", n)
        at += n
        lo = max(at - 33 + 1, 0)                          # the lowest position the next row sees through its window
        held = [b for b, p in enumerate(rc.tables[group]) if p >= 0]
        want = [b for b in range((at + 3) // 4) if b * 4 < 5 or (b + 1) * 4 > lo]
        assert held == want, (at, held, want)
    full = next(i for i, g in enumerate(cache.groups) if g.spec.kind == "full")
    assert all(p >= 0 for p in rc.tables[full]) and len(rc.tables[full]) == (at + 3) // 4
    cache.free_request("a")
    cache.check_invariants()
    assert all(g.pages.held_count == 0 for g in cache.groups)


# -- the distance table -------------------------------------------------------------------------
@pytest.mark.parametrize("rows,far", [(2, 2), (2, 3), (4, 9), (8, 40), (32, 150), (16, 200), (12, 64), (10, 16), (6, 3)])
def test_distance_table_rows_are_the_plain_buckets(rows, far):
    from sharpinference_b200.parts import distance_bias_table
    rel = torch.arange(rows * 3, dtype=torch.float32).view(rows, 3)
    table = distance_bias_table(rel, far)
    n = table.shape[0] - 1
    assert n <= max(far, rows)
    for dist in range(0, 3 * far + 5):
        want = rows - 1 if far <= rows // 2 and dist >= rows // 2 else plain.distance_bucket(dist, rows, far)
        assert torch.equal(table[min(dist, n)], rel[want]), (dist, want)


def test_plain_buckets_are_exact_near_and_logarithmic_far():
    rows, far = 32, 150
    assert [plain.distance_bucket(n, rows, far) for n in range(16)] == list(range(16))
    got = [plain.distance_bucket(n, rows, far) for n in range(16, 400)]
    assert got == sorted(got) and got[0] == 16 and got[-1] == 31
    first_last = next(n for n in range(16, 400) if plain.distance_bucket(n, rows, far) == 31)
    assert 16 * (150 / 16) ** (15 / 16) <= first_last <= 150


# -- the plain implementation against itself ---------------------------------------------------
def test_plain_norm_rotation_and_window():
    x = _rand(3, 8, seed=1, scale=2.0)
    w, b = _rand(8, seed=2), _rand(8, seed=3)
    assert torch.allclose(plain.dyt(x, 0.7, w, b), torch.tanh(0.7 * x) * w + b)
    assert torch.allclose((plain.rms(x, 0.0) ** 2).mean(-1), torch.ones(3, dtype=F64))
    q, k = _rand(1, 1, 12, seed=4), _rand(1, 1, 12, seed=5)
    dots = []
    for shift in (0, 23):
        qr = plain.rotate_pairs(q, torch.tensor([5 + shift]), 100.0, 8)
        kr = plain.rotate_pairs(k, torch.tensor([2 + shift]), 100.0, 8)
        assert torch.equal(qr[..., 8:], q[..., 8:])
        dots.append(float((qr * kr).sum()))
    assert dots[0] == pytest.approx(dots[1], abs=1e-12)
    one = plain.rotate_pairs(q, torch.tensor([1]), 100.0, 4)
    assert float(one[0, 0, 0]) == pytest.approx(float(q[0, 0, 0] * math.cos(1.0) - q[0, 0, 1] * math.sin(1.0)))
    assert float(one[0, 0, 3]) == pytest.approx(float(q[0, 0, 3] * math.cos(0.1) + q[0, 0, 2] * math.sin(0.1)))
    vis = plain.window_with_first(12, 3, 2)
    assert vis[9].tolist() == [True, True] + [False] * 5 + [True] * 3 + [False] * 2
    assert vis[1].tolist() == [True, True] + [False] * 10


def test_plain_window_attention_sees_window_and_kept_positions_only(tmp_path):
    folder = write("A", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    m = cfg["layers"][1]["mixer"]                            # a window of 33 with 5 kept positions
    h = _rand(60, cfg["width"], seed=6)
    full = plain.window_attention(h, m, w, "l1.mix.")
    h2 = h.clone()
    h2[5:20] = _rand(15, cfg["width"], seed=7)               # positions 5 .. 19: outside the window of rows >= 52
    other = plain.window_attention(h2, m, w, "l1.mix.")
    assert torch.allclose(full[52:], other[52:]) and not torch.allclose(full[51], other[51])
    h3 = h.clone()
    h3[4] = _rand(cfg["width"], seed=8)                      # a kept position reaches the last row
    assert not torch.allclose(plain.window_attention(h3, m, w, "l1.mix.")[59], full[59])
    assert not torch.allclose(plain.window_attention(h, m, w, "l1.mix.", window_delta=1)[52], full[52])
    assert not torch.allclose(plain.window_attention(h, m, w, "l1.mix.", keep_delta=-1)[59], full[59])


def test_plain_mixture_weights_the_input_of_the_chosen_experts(tmp_path):
    folder = write("A", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    mlp = cfg["layers"][0]["mlp"]                            # two of four experts, a shared one
    h = _rand(6, cfg["width"], seed=9)
    out, scores, chosen = plain.mixture(h, mlp, w, "l0.mlp.")
    assert chosen.shape == (6, 2) and torch.equal(chosen, scores.topk(2, dim=-1).indices)
    def expert(name, u):
        return (plain.silu(u @ w[name + ".gate"].T) * (u @ w[name + ".up"].T)) @ w[name + ".down"].T
    for t in range(6):
        want = expert("l0.mlp.shared", h[t])
        for e in chosen[t].tolist():
            want = want + expert(f"l0.mlp.e{e}", scores[t, e] * h[t])
        assert torch.allclose(out[t], want, atol=1e-12)
    assert float(scores.min()) > 0 and float(scores.max()) < 1 and not torch.allclose(scores.sum(-1), torch.ones(6, dtype=F64))


def test_plain_state_space_layer_equals_its_sum_form(tmp_path):
    """The recurrence, unrolled: y_t = sum_{s<=t} (prod_{s<r<=t} a_r) dt_s (C_t . B_s) x_s + D x_t."""
    folder = write("A", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    m, p = cfg["layers"][2]["mixer"], "l2.mix."
    nh, dv, N, G, T = m["heads"], m["vdim"], m["state"], m["groups"], 9
    h = _rand(T, cfg["width"], seed=10)
    inner = nh * dv
    proj = h @ w[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = plain.causal_conv_silu(xbc, w[p + "conv"], w[p + "conv.b"])
    x, B, C = xbc[:, :inner].view(T, nh, dv), xbc[:, inner:inner + G * N].view(T, G, N), xbc[:, inner + G * N:].view(T, G, N)
    dt = plain.softplus(dt + w[p + "dt_bias"])
    log_a = -torch.exp(w[p + "A_log"]) * dt
    y = torch.zeros(T, nh, dv, dtype=F64)
    for hd in range(nh):
        g = hd // (nh // G)
        for t in range(T):
            for s in range(t + 1):
                y[t, hd] += torch.exp(log_a[s + 1:t + 1, hd].sum()) * dt[s, hd] * (C[t, g] @ B[s, g]) * x[s, hd]
            y[t, hd] += w[p + "D"][hd] * x[t, hd]
    u = y.reshape(T, inner) * plain.silu(z)
    parts = m["norm_groups"]
    want = (plain.rms(u.view(T, parts, inner // parts), cfg["norm"]["eps"]).reshape(T, inner) * w[p + "norm"]) @ w[p + "o"].T
    assert torch.allclose(plain.mamba2(h, m, w, p, cfg["norm"]["eps"]), want, atol=1e-10)
    # the convolution sees zeros before the start and the current token through its last column
    one = torch.zeros(4, 2, dtype=F64)
    one[1, 0] = 1.0
    cw, cb = torch.tensor([[1.0, 2.0, 3.0], [0.0, 0.0, 0.0]], dtype=F64), torch.tensor([0.0, 0.5], dtype=F64)
    got = plain.causal_conv_silu(one, cw, cb)
    assert torch.allclose(got[:, 0], plain.silu(torch.tensor([0.0, 3.0, 2.0, 1.0], dtype=F64)))
    assert torch.allclose(got[:, 1], plain.silu(torch.full((4,), 0.5, dtype=F64)))


@pytest.mark.parametrize("name", sorted(CASES))
def test_random_folder_loads_and_runs_plain(tmp_path, name):
    folder = write(name, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    arch, typed = resolve(cfg, "test")
    assert {d.name for d in declared_tensors(arch, typed)} == set(w)
    toks = traces.random_tokens(cfg["vocab"], 12, seed=1)
    logits, layers, _ = plain.forward(cfg, w, toks, want_layers=True)
    assert logits.shape == (12, cfg["vocab"]) and len(layers) == len(cfg["layers"]) and bool(torch.isfinite(logits).all())
    # a prefix gives the same logits: everything is causal
    assert torch.allclose(plain.forward(cfg, w, toks[:7]), logits[:7], atol=1e-12)
