"""``bench.py --preset gisilix``: prefill and decode throughput of the Gisilix architecture at layer sizes that
resemble a real model's, beside Latinex (the framework's closest architecture: latent attention and gated attention
beside mixtures of gated experts with a shared expert) at equal width and depth, both with random bfloat16 weights on
one B200.

Per width W, Gisilix has ten layers in the order attention, windowed latent attention, latent attention, attention
that borrows the keys and values of the attention layer three before it, and so on: attention with W / 128 heads of
128 (a quarter as many key/value heads), a norm over the whole q and k, scores capped at 30, sinks, a query factor
every 1024 positions and an element-wise gate; latent attention with W / 128 heads of 128 unrotated (and, in the
windowed layers, 64 rotated) elements, values of 128 and a cached latent of 256 (a row of 320 with the rotated part),
a window of 1024 positions and stretched frequencies; every layer has 16 experts of W / 2 with two a row and a shared
expert of W / 2, as Latinex has (``--preset latinex``).

Timing as in ``bench_notedra.py``: CUDA events after warm-up, a step's weights and cache exceed the L2 cache.
"""
from __future__ import annotations

import json
import time

from bench_latinex import latinex_config
from bench_notedra import _measure


def gisilix_config(W: int, vocab: int = 32768) -> dict:
    ah = max(1, W // 128)
    attn = {"heads": ah, "kv_heads": max(1, ah // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "softcap": 30.0,
            "q_temp": {"coef": 0.1, "every": 1024}}
    lat = {"heads": ah, "dim": 128, "vdim": 128, "kv_rank": 256, "scale": 128 ** -0.5}
    lat2 = {"heads": ah, "dim": 128, "rot_dim": 64, "vdim": 128, "kv_rank": 256, "scale": 192 ** -0.5,
            "rot": {"dims": 64, "base": 500000.0, "scaling": {"factor": 8.0, "original": 8192, "fast": 32.0, "slow": 1.0}},
            "mask": {"size": 1024}}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": W // 2}, "shared": {"ff": W // 2}}
    kinds = ["attention", "latent_attention_2", "latent_attention", "borrow"]
    layers, last_own = [], None
    for i in range(10):
        kind = kinds[i % 4]
        if kind == "attention":
            last_own = i
            layers.append({"type": "attention", "mixer": dict(attn), "mlp": dict(moe)})
        elif kind == "borrow":
            layers.append({"type": "attention", "mixer": dict(attn, kv_from=last_own), "mlp": dict(moe)})
        else:
            layers.append({"type": kind, "mixer": dict(lat2 if kind == "latent_attention_2" else lat), "mlp": dict(moe)})
    return {"architecture": "Gisilix", "vocab": vocab, "width": W, "norm": {"eps": 1e-6}, "layers": layers}


def run(ns, pk, pk_kind) -> int:
    widths = [int(w) for w in ns.widths.split(",") if w.strip()]
    batches = [int(b) for b in ns.points.split(",") if b.strip()] or [8]
    t0 = time.time()
    sizes = {}
    for W in widths:
        sizes[str(W)] = {
            "gisilix": _measure("gisilix", gisilix_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
            "latinex": _measure("latinex", latinex_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
        }
    first = sizes[str(widths[0])]["gisilix"]["decode"][str(batches[0])]
    print(json.dumps({
        "metric": "decode tokens/s, Gisilix layer sizes beside Latinex at equal width (random bf16 weights)",
        "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": ns.steps, "warmup": max(ns.warmup, 3),
        "ms_per_step": first["ms_per_step"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"preset": "gisilix", "widths": widths, "prefill_tokens": ns.prefill_tokens, "context": ns.context,
                   "batches": batches, "l2": "weights and cache of a step exceed the L2 cache"},
        "peaks": dict(pk, kind=pk_kind), "sizes": sizes, "seconds": round(time.time() - t0, 1)}))
    return 0
