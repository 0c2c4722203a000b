"""``bench.py --preset latinex``: prefill and decode throughput of the Latinex architecture at layer sizes that
resemble a real model's, beside Notedra (the framework's closest architecture: masked attention beside a recurrent
mixer with per-request state, routed experts) at equal width and depth, both with random bfloat16 weights on one B200.

Per width W, Latinex has ten layers, latent attention, windowed attention and state-space duality in turn: latent
attention with W / 128 heads of 128 unrotated and 64 rotated elements and values of 128, a query latent of 3 W / 8
and a cached row of 256 + 64; windowed attention with W / 128 heads of 128 whose keys (a quarter as many heads) are
the values, a window of 1024 positions that keeps the first 4, a distance table of 32 rows; a state-space layer of
2 W / 64 heads of 64 with 128 states in one group, four taps; every layer has 16 experts of W / 2 with two a row and
a shared expert of W / 2.  Notedra is the configuration of ``--preset notedra`` (five layers that run twice).

Timing as in ``bench_notedra.py``: CUDA events after warm-up, a step's weights, state and cache exceed the L2 cache.
"""
from __future__ import annotations

import json
import time

from bench_notedra import _measure, notedra_config


def latinex_config(W: int, vocab: int = 32768) -> dict:
    ah = max(1, W // 128)
    latent = {"heads": ah, "dim": 128, "rot_dim": 64, "vdim": 128, "q_rank": 3 * W // 8, "kv_rank": 256,
              "scale": 192 ** -0.5, "rot": {"dims": 64, "base": 500000.0}}
    attn = {"heads": ah, "kv_heads": max(1, ah // 4), "dim": 128, "vdim": 128, "scale": 128 ** -0.5, "bias_max": 1024,
            "bias_buckets": 32, "mask": {"size": 1024, "keep_first": 4}}
    ssd = {"heads": max(1, 2 * W // 64), "vdim": 64, "state": 128, "groups": 1, "conv": 4, "norm_groups": 1}
    moe = {"kind": "moe", "router": {"experts": 16, "top": 2}, "expert": {"ff": W // 2}, "shared": {"ff": W // 2}}
    kinds = ["latent_attention", "attention", "mamba2"]
    mixers = {"latent_attention": latent, "attention": attn, "mamba2": ssd}
    layers = [{"type": kinds[i % 3], "mixer": dict(mixers[kinds[i % 3]]), "mlp": dict(moe)} for i in range(10)]
    return {"architecture": "Latinex", "vocab": vocab, "width": W, "logit_scale": 1.0, "embedding": {"scale": 1.0},
            "norm": {"eps": 1e-6}, "layers": layers}


def run(ns, pk, pk_kind) -> int:
    widths = [int(w) for w in ns.widths.split(",") if w.strip()]
    batches = [int(b) for b in ns.points.split(",") if b.strip()] or [8]
    t0 = time.time()
    sizes = {}
    for W in widths:
        sizes[str(W)] = {
            "latinex": _measure("latinex", latinex_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
            "notedra": _measure("notedra", notedra_config(W), ns.prefill_tokens, batches, ns.context, ns.steps, max(ns.warmup, 3)),
        }
    first = sizes[str(widths[0])]["latinex"]["decode"][str(batches[0])]
    print(json.dumps({
        "metric": "decode tokens/s, Latinex layer sizes beside Notedra at equal width (random bf16 weights)",
        "value": first["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "steps": ns.steps, "warmup": max(ns.warmup, 3),
        "ms_per_step": first["ms_per_step"], "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"preset": "latinex", "widths": widths, "prefill_tokens": ns.prefill_tokens, "context": ns.context,
                   "batches": batches, "l2": "weights, state and cache of a step exceed the L2 cache"},
        "peaks": dict(pk, kind=pk_kind), "sizes": sizes, "seconds": round(time.time() - t0, 1)}))
    return 0
