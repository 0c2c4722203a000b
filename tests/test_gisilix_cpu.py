"""Gisilix without a GPU: the configuration reader, the tensor declaration, the schedule and the pages that the cache
manager hands to the layers, the stretched rotation frequencies, and the plain implementation checked against each
mechanism's defining property."""
import copy
import math

import pytest
import torch

import plain_gisilix as plain
import traces
from gisilix_models import CASE_A, CASE_B, CASE_C, CASE_D, CASE_E, CASES, write

from sharpinference_b200.config import ConfigError, GisilixConfig
from sharpinference_b200.registry import get_architecture, resolve
from sharpinference_b200.weights.loading import declared_tensors

F64 = torch.float64


def _rand(*shape, seed=0, scale=1.0):
    return scale * torch.randn(*shape, generator=torch.Generator().manual_seed(seed), dtype=F64)


# -- configuration -------------------------------------------------------------------------
@pytest.mark.parametrize("case", [CASE_A, CASE_B, CASE_C, CASE_D, CASE_E])
def test_config_round_trip(case):
    arch, cfg = resolve(copy.deepcopy(case), "test")
    assert arch.name == "Gisilix" and isinstance(cfg, GisilixConfig)
    assert GisilixConfig.from_dict(cfg.to_dict()) == cfg
    assert cfg.to_dict() == case
    assert [layer.type for layer in cfg.layers] == [c["type"] for c in case["layers"]]
    for layer, raw in zip(cfg.layers, case["layers"]):
        assert (layer.mlp is None) == (raw["mlp"] is None)
        assert layer.kv_from == raw["mixer"].get("kv_from")
        if raw["mlp"] and raw["mlp"]["kind"] == "moe":
            assert (layer.mlp.experts, layer.mlp.top) == (raw["mlp"]["router"]["experts"], raw["mlp"]["router"]["top"])
            assert layer.mlp.shared_ff == (raw["mlp"]["shared"] or {"ff": 0})["ff"]


def test_defaults_of_absent_keys():
    case = copy.deepcopy(CASE_A)
    a0, _, l2, l3 = (layer["mixer"] for layer in case["layers"])
    del a0["kv_heads"], a0["vdim"], a0["scale"], a0["softcap"], a0["q_temp"]
    case["layers"][1]["mixer"]["kv_heads"], case["layers"][1]["mixer"]["vdim"] = 4, 16
    del l2["mask"], l2["scale"], l2["rot"]["scaling"], l2["rot"]["dims"]
    del l3["vdim"]
    _, cfg = resolve(case, "test")
    a, _, b, c = cfg.layers
    assert a.kv_heads == 4 and a.vdim == 16 and a.scale == pytest.approx(0.25) and a.softcap == 0 and a.temp_every == 0
    assert b.window == 0 and b.scale == pytest.approx(0.25) and b.yarn is None and b.rot_dims == 8 and b.head_gate
    assert c.vdim == 16 and c.rot_dim == 0 and not c.head_gate


def test_config_problems_are_listed_together():
    bad = copy.deepcopy(CASE_A)
    del bad["width"]
    bad["layers"][0]["mixer"]["kv_heads"] = 3                   # 4 heads are no multiple of 3
    bad["layers"][1]["mixer"]["kv_from"] = 2                    # not an earlier attention layer
    bad["layers"][2]["mixer"]["rot"]["dims"] = 10               # beyond rot_dim
    bad["layers"][3]["mlp"]["router"]["top"] = 9                # more than there are experts
    bad["layers"].append({"type": "conv", "mixer": {}, "mlp": None})
    with pytest.raises(ConfigError) as err:
        resolve(bad, "test")
    text = str(err.value)
    for piece in ("width", "kv_heads", "rot.dims", "router.top", "conv"):
        assert piece in text, (piece, text)
    bad = copy.deepcopy(CASE_A)
    bad["layers"][1]["mixer"]["kv_from"] = 2
    with pytest.raises(ConfigError, match="kv_from"):
        resolve(bad, "test")
    bad = copy.deepcopy(CASE_A)
    bad["layers"][1]["mixer"]["dim"] = 8                        # the borrowed keys have another size
    with pytest.raises(ConfigError, match="must agree"):
        resolve(bad, "test")


def test_declared_tensors_follow_the_configuration():
    arch = get_architecture("Gisilix")
    _, cfg = resolve(copy.deepcopy(CASE_A), "test")
    decls = {d.name: d.shape for d in declared_tensors(arch, cfg)}
    assert decls["embed"] == (97, 64) and "head" not in decls and decls["final.norm.b"] == (64,)
    assert decls["l0.mix.q"] == (64, 64) and decls["l0.mix.k"] == (32, 64) and decls["l0.mix.v"] == (48, 64)
    assert decls["l0.mix.q.norm"] == (64,) and decls["l0.mix.k.norm"] == (32,) and decls["l0.mix.sink"] == (4,)
    assert decls["l0.mix.g"] == (96, 64) and decls["l0.mix.o"] == (64, 96)
    assert decls["l0.mlp.gate"] == (40, 64) and decls["l0.mlp.down"] == (64, 40)
    # the borrowing layer has queries, their norm, sink, gate and output only
    assert decls["l1.mix.q"] == (64, 64) and decls["l1.mix.q.norm"] == (64,) and decls["l1.mix.g"] == (96, 64)
    assert not any(n in decls for n in ("l1.mix.k", "l1.mix.v", "l1.mix.k.norm"))
    assert decls["l1.mlp.router"] == (4, 64) and decls["l1.mlp.router.b"] == (4,) and decls["l1.mlp.e3.gate"] == (24, 64)
    assert decls["l1.mlp.shared.up"] == (40, 64) and "l1.mlp.e4.gate" not in decls
    assert decls["l2.mix.q"] == (2 * 16, 64) and decls["l2.mix.dkv"] == (32, 64) and decls["l2.mix.dkv.norm"] == (24,)
    assert decls["l2.mix.uk"] == (16, 24) and decls["l2.mix.uv"] == (24, 24) and decls["l2.mix.g"] == (2, 64)
    assert "l2.norm2" not in decls and "l2.mlp.gate" not in decls            # no feed-forward, no second norm
    assert decls["l3.mix.q"] == (64, 64) and decls["l3.mix.dkv"] == (40, 64) and "l3.mix.g" not in decls
    assert "l3.mlp.shared.up" not in decls


def test_schedule_and_pages_in_the_cache_manager():
    """A borrowing layer is a schedule entry that reads another entry's cache; attention layers of equal shape share a
    group of pages with two planes, latent layers cache one row a token in keys-only pages, windowed ones in a group
    of their own."""
    from sharpinference_b200.cache import CacheManager
    from sharpinference_b200.weights.source import DeclaringWeights
    arch = get_architecture("Gisilix")
    _, cfg = resolve(copy.deepcopy(CASE_C), "test")
    model = arch.build(cfg, DeclaringWeights(torch.float32))
    assert [e.cache_from for e in model.schedule] == [None, None, None, 0, None, None]
    cache = CacheManager(model.schedule, model.blocks, page_size=4, num_pages=8, max_requests=2, dtype=torch.float32,
                         device="cpu", model_state_specs=model.state_specs)
    specs = sorted((g.spec.kind, g.spec.span, g.spec.num_kv_heads, g.spec.head_dim, g.spec.planes) for g in cache.groups)
    assert specs == [("full", 0, 1, 64, 2), ("full", 0, 1, 128, 1), ("full", 0, 2, 128, 2), ("window", 64, 1, 128, 1),
                     ("window", 130, 1, 80, 1)]
    slots = cache.layer_slots()
    assert slots[3].kv.data_ptr() == slots[0].kv.data_ptr() and not slots[3].writes_cache and slots[0].writes_cache
    # values wider than keys: both padded to one head size, the norm's mean still over the keys' own size
    _, cfg = resolve(copy.deepcopy(CASE_A), "test")
    model = arch.build(cfg, DeclaringWeights(torch.float32))
    mixer = model.blocks[0].mixer
    assert (mixer.key_dim, mixer.value_dim, mixer.head_dim) == (16, 24, 32)
    assert mixer.qkv.out_features == (4 + 2 + 2 + 4) * 32 and model.blocks[1].mixer.qkv.out_features == (4 + 4) * 32


# -- stretched frequencies -----------------------------------------------------------------
@pytest.mark.parametrize("dims,base,scaling", [(24, 40000.0, (3.0, 1024, 24.0, 1.5)), (4, 100.0, (4.0, 16, 4.0, 1.0)),
                                               (2, 10.0, (8.0, 4, 1.0, 0.25)), (64, 10000.0, (4.0, 128, 32.0, 1.0)),
                                               (32, 30000.0, (4.0, 64, 8.0, 1.0)), (16, 1000.0, (16.0, 32, 16.0, 2.0))])
def test_stretched_frequencies(dims, base, scaling):
    from sharpinference_b200.parts import yarn_inv_freq
    got, amp = yarn_inv_freq(dims, base, *scaling)
    want, want_amp = plain.yarn_frequencies(dims, base, dict(zip(("factor", "original", "fast", "slow"), scaling)))
    assert torch.allclose(got.double(), want, rtol=1e-6, atol=0) and amp == pytest.approx(want_amp)
    plain_f = base ** (-2.0 * torch.arange(dims // 2, dtype=F64) / dims)
    # every frequency lies between the plain one and the plain one divided by the factor
    assert bool(((want <= plain_f * (1 + 1e-12)) & (want >= plain_f / scaling[0] * (1 - 1e-12))).all())
    assert amp == pytest.approx(0.1 * math.log(scaling[0]) + 1.0)


def test_stretched_frequencies_blend_between_fast_and_slow_waves():
    """A wave that makes many turns over the original span keeps its frequency, one that makes less than one turn is
    slowed by the factor, and the pairs between are blended linearly in the pair index."""
    f, _ = plain.yarn_frequencies(24, 40000.0, {"factor": 5.0, "original": 1024, "fast": 24.0, "slow": 1.5})
    plain_f = 40000.0 ** (-2.0 * torch.arange(12, dtype=F64) / 24)
    ratio = f / plain_f
    assert ratio[0] == 1.0 and ratio[-1] == pytest.approx(0.2)
    assert bool((ratio[1:] <= ratio[:-1] + 1e-12).all())
    inner = [float(r) for r in ratio if 0.2 + 1e-9 < float(r) < 1 - 1e-9]
    assert len(inner) >= 2
    steps = [inner[i] - inner[i + 1] for i in range(len(inner) - 1)]
    assert max(steps) - min(steps) < 1e-9                       # equal steps: linear in the pair index


# -- the plain implementation --------------------------------------------------------------
def test_plain_norms_and_softmax_with_a_sink():
    x, w, b = _rand(5, 12, seed=1, scale=3.0), _rand(12, seed=2), _rand(12, seed=3)
    y = plain.layer_norm(x, w, b, 1e-5)
    assert torch.allclose(y, torch.nn.functional.layer_norm(x, (12,), w, b, 1e-5), atol=1e-12)
    r = plain.rms(x, w, 1e-5)
    assert torch.allclose(r, x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5) * w, atol=1e-12)
    s = _rand(2, 4, 4, seed=4)
    sink = torch.tensor([0.5, -1.0], dtype=F64)
    p = plain.softmax_rows(s, plain.causal(4), sink)
    # a sink is a key with score `sink` whose value is zero: append it and drop its column
    ext = torch.cat([s.masked_fill(~plain.causal(4), -math.inf), sink.view(2, 1, 1).expand(2, 4, 1)], dim=-1)
    assert torch.allclose(p, torch.softmax(ext, dim=-1)[..., :4], atol=1e-12)
    assert float(p.sum(-1).max()) < 1.0 and float(p[0, 0, 1:].abs().max()) == 0.0
    vis = plain.causal(6, 3)
    assert vis[5].tolist() == [False, False, False, True, True, True] and vis[1].tolist() == [True, True] + [False] * 4


def test_plain_query_factor_and_rotation():
    f = plain.query_temperature(300, 0.25, 100)
    assert f[98] == 1.0 and f[99] == pytest.approx(1 + 0.25 * math.log(2)) and f[199] == pytest.approx(1 + 0.25 * math.log(3))
    v = _rand(7, 3, 6, seed=5)
    freqs = torch.tensor([0.5, 0.1], dtype=F64)
    out = plain.rotate_pairs(v, freqs, 1.2, 4)
    assert torch.equal(out[..., 4:], v[..., 4:]) and torch.allclose(out[0], v[0] * torch.tensor([1.2] * 4 + [1, 1], dtype=F64))
    # the dot product of two rotated vectors depends on the distance of their positions alone
    a, b = _rand(1, 4, seed=6), _rand(1, 4, seed=7)
    ra, rb = plain.rotate_pairs(a.expand(9, 4), freqs, 1.0, 4), plain.rotate_pairs(b.expand(9, 4), freqs, 1.0, 4)
    assert float(ra[5] @ rb[2]) == pytest.approx(float(ra[8] @ rb[5]), abs=1e-12)


def test_plain_mixture_weights_the_outputs_by_the_softmax_over_the_chosen(tmp_path):
    folder = write("A", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    mlp = cfg["layers"][1]["mlp"]
    h = _rand(6, 64, seed=8)
    out, idx, z = plain.mixture(h, mlp, w, "l1.mlp.")
    assert torch.equal(idx, z.topk(2, dim=-1).indices)
    for t in range(6):
        zt = z[t, idx[t]]
        wt = torch.exp(zt) / torch.exp(zt).sum()
        want = sum(wt[j] * plain.gated(h[t:t + 1], w, f"l1.mlp.e{int(idx[t, j])}.") for j in range(2))
        want = want + plain.gated(h[t:t + 1], w, "l1.mlp.shared.")
        assert torch.allclose(out[t:t + 1], want, atol=1e-12)
    # the bias takes part in the choice and in the weights
    w2 = dict(w)
    w2["l1.mlp.router.b"] = w["l1.mlp.router.b"] + torch.tensor([0.0, 0.0, 0.0, 50.0], dtype=F64)
    assert bool((plain.mixture(h, mlp, w2, "l1.mlp.")[1][:, 0] == 3).all())


@pytest.mark.parametrize("name", sorted(CASES))
def test_random_folder_loads_and_runs_plain(tmp_path, name):
    folder = write(name, str(tmp_path))
    cfg, w = plain.load_folder(folder)
    toks = traces.random_tokens(cfg["vocab"], 40, seed=1)
    layers = []
    logits = plain.forward(cfg, w, toks, layers_out=layers)
    assert logits.shape == (40, cfg["vocab"]) and len(layers) == len(cfg["layers"]) and bool(torch.isfinite(logits).all())
    # causal: a prefix gives the same logits
    assert torch.allclose(plain.forward(cfg, w, toks[:17]), logits[:17], atol=1e-9)


def test_every_constant_shows_in_the_plain_logits(tmp_path):
    """The comparison with the plain model is sharp: dropping the sink, the cap, the query factor, the amplitude or the
    stretching of the rotation, or moving a window by one, changes the plain logits by far more than the tolerance."""
    folder = write("A", str(tmp_path))
    cfg, w = plain.load_folder(folder)
    toks = traces.random_tokens(cfg["vocab"], 90, seed=2)
    right = plain.forward(cfg, w, toks)
    scale = float(right.abs().max())

    def moved(other_cfg=None, other_w=None):
        wrong = plain.forward(other_cfg or cfg, other_w or w, toks)
        return float((wrong - right).abs().max()) / scale

    for key in ("softcap", "q_temp"):
        c = copy.deepcopy(cfg)
        del c["layers"][0]["mixer"][key]
        assert moved(c) > 1e-2, key
    c = copy.deepcopy(cfg)
    del c["layers"][2]["mixer"]["rot"]["scaling"]
    assert moved(c) > 1e-3
    for delta in (-1, 1):
        c = copy.deepcopy(cfg)
        c["layers"][2]["mixer"]["mask"]["size"] += delta
        assert moved(c) > 1e-3
        early = min(33, 33 + delta)
        assert float((plain.forward(c, w, toks)[:early] - right[:early]).abs().max()) == 0.0
    w2 = {k: v for k, v in w.items() if not k.endswith(".sink")}
    assert moved(None, w2) > 1e-2
    w3 = dict(w)
    w3["l1.mix.sink"] = w["l1.mix.sink"] + 1.0
    assert moved(None, w3) > 1e-3
