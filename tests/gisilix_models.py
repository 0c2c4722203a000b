"""Small Gisilix configurations for the tests, and folders with random weights for them.

The configurations differ from each other in every size; between them they cover: attention with one key head, one per
query head and groups, values wider and narrower than keys, head sizes that the tensor-core kernels take (64, 128) and
that they do not, layers that borrow the keys and values of an earlier layer (directly behind it and three layers on),
query factors that change every 3 to 40 positions, caps from 1.5 to 30 and none; latent attention whose cached row
(latent plus rotated part) is and is not a multiple of 16, with a rotation of all and of part of the rotated elements,
with stretched frequencies whose blend range lies inside, below and above the pairs, and with plain ones; windows of 1,
2, 5, 33, 64, 70, 100 and 130 positions; layers without a feed-forward, dense ones, one to three experts a row, a single
expert, no shared expert; widths that are no multiple of 8; sizes of one and two everywhere.

Random weights alone would hide some faults, so ``write`` edits a few tensors afterwards: the sinks get values of both
signs around the size of a score, router biases are spread so that they decide choices, and the score factors in the
configurations are large (single keys carry a row's output, so a window that is one position off shows, and the cap
bends the scores that matter).
"""
from __future__ import annotations

import os

import torch


def dense(ff):
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared} if shared else None}


def att(heads, kv, dim, vdim, scale, cap, temp, mlp, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if cap:
        m["softcap"] = cap
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "attention", "mixer": m, "mlp": mlp}


def lat(heads, dim, vdim, kv_rank, scale, mlp):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale}, "mlp": mlp}


def lat2(heads, dim, rot_dim, vdim, kv_rank, scale, rot, window, mlp):
    """``rot`` = (dims, base, scaling or None) with scaling = (factor, original, fast, slow)."""
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
         "rot": {"dims": rot[0], "base": rot[1]}}
    if rot[2]:
        m["rot"]["scaling"] = dict(zip(("factor", "original", "fast", "slow"), rot[2]))
    if window:
        m["mask"] = {"size": window}
    return {"type": "latent_attention_2", "mixer": m, "mlp": mlp}


def top(vocab, width, eps, layers):
    return {"architecture": "Gisilix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# A: every mixer; grouped key heads with values wider than keys; a layer that borrows from the layer right before it;
# a cached latent row of 24 + 8 = 32 elements of which 4 turn; a window of 33; two experts a row with a shared expert;
# a layer without a feed-forward.
CASE_A = top(97, 64, 1e-5, [
    att(4, 2, 16, 24, 0.9, 3.0, (0.4, 8), dense(40)),
    att(4, 2, 16, 24, 1.1, 2.0, (0.2, 5), moe(4, 2, 24, 40), kv_from=0),
    lat2(2, 8, 8, 12, 24, 0.8, (4, 100.0, (4.0, 16, 4.0, 1.0)), 33, None),
    lat(4, 16, 8, 40, 0.7, moe(3, 1, 16, 0)),
])

# B: a width that is no multiple of 8 (no library product and no tensor-core expert product anywhere); head sizes
# of 10; a latent row of 20 + 6 = 26 elements; windows of 70 (longer than a page), 1 and 2; three experts a row out
# of three; no cap on one layer and no query factor on another; latent attention first.
CASE_B = top(61, 52, 1e-4, [
    lat2(3, 10, 6, 10, 20, 0.8, (6, 50.0, None), 70, moe(3, 3, 12, 20)),
    att(3, 3, 10, 10, 0.5, 0.0, (0.25, 3), None),
    lat2(2, 12, 4, 6, 14, 1.2, (2, 300.0, (2.0, 8, 2.0, 0.5)), 1, dense(30)),
    lat(2, 6, 10, 9, 1.5, None),
    lat2(1, 4, 2, 4, 7, 1.0, (2, 10.0, (8.0, 4, 1.0, 0.25)), 2, moe(5, 2, 10, 0)),
    att(3, 3, 10, 10, 1.3, 1.5, None, dense(17), kv_from=1),
])

# C: sizes that the tensor-core kernels take: attention heads of 64 (one key head for four) and of 128 (two for two),
# a latent row of 96 + 32 = 128; a window of exactly a page and one of 130; a borrowing layer three layers on;
# a single expert; eight experts.
CASE_C = top(131, 128, 1e-6, [
    att(4, 1, 64, 64, 0.4, 6.0, (0.3, 40), moe(1, 1, 32, 32)),
    lat2(4, 32, 32, 48, 96, 0.35, (32, 30000.0, (4.0, 64, 8.0, 1.0)), 64, moe(8, 2, 32, 48)),
    att(2, 2, 128, 128, 0.25, 30.0, (0.1, 16), dense(96)),
    att(4, 1, 64, 64, 0.5, 4.0, (0.6, 7), None, kv_from=0),
    lat2(2, 64, 16, 32, 64, 0.3, (16, 1000.0, (16.0, 32, 16.0, 2.0)), 130, None),
    lat(8, 16, 16, 128, 0.5, dense(64)),
])

# D: ones and twos wherever a size can be one or two.
CASE_D = top(23, 16, 1e-5, [
    att(1, 1, 2, 1, 1.2, 2.0, (1.0, 1), moe(2, 2, 1, 1)),
    lat2(1, 2, 2, 2, 2, 1.2, (2, 10.0, (2.0, 2, 1.0, 0.5)), 2, None),
    lat(2, 1, 1, 1, 0.9, dense(2)),
    att(2, 1, 2, 2, 1.4, 1.0, (0.5, 2), moe(1, 1, 2, 0)),
    att(1, 1, 2, 1, 0.7, 0.0, None, None, kv_from=0),
])

# E: the largest sizes: a latent row of 192 + 64 = 256 elements with a window of 100; attention heads of 128 with
# values of 64; a latent of 300 (a row of 304); a window of 5; values narrower than keys in a borrowing pair.
CASE_E = top(50, 96, 1e-5, [
    lat2(2, 48, 64, 40, 192, 0.2, (64, 10000.0, (4.0, 128, 32.0, 1.0)), 100, moe(4, 3, 16, 8)),
    att(2, 1, 128, 64, 0.25, 10.0, (0.3, 32), None),
    lat(3, 24, 32, 300, 0.3, dense(48)),
    lat2(3, 16, 8, 16, 40, 1.0, (8, 20.0, None), 5, moe(2, 1, 24, 24)),
    att(2, 1, 128, 64, 0.2, 10.0, (0.3, 32), dense(24), kv_from=1),
])

# config, std of the weights, seed
CASES = {"A": (CASE_A, 0.15, 41), "B": (CASE_B, 0.13, 42), "C": (CASE_C, 0.1, 43), "D": (CASE_D, 0.5, 44),
         "E": (CASE_E, 0.1, 45)}


def drawn_config(seed: int) -> dict:
    """A configuration drawn from a seeded generator: three to nine layers in any order, widths of 64 to 320, grouped
    and plain key heads of 16 to 128 elements with values of their own size, borrowing layers wherever an earlier
    attention layer exists, latents of 32 to 512, windows from 17 to 600 or none, every kind of feed-forward."""
    import random
    r = random.Random(seed)
    W = r.choice([64, 96, 128, 192, 256, 320])
    layers, own = [], []

    def mlp():
        k = r.random()
        if k < 0.15:
            return None
        if k < 0.5:
            return dense(r.choice([48, 72, 128, 200]))
        E = r.choice([2, 3, 5, 8, 12])
        return moe(E, r.randint(1, min(E, 4)), r.choice([16, 24, 40, 64]), r.choice([0, 32, 64]))

    def cap_and_temp():
        return r.choice([0, 5.0, 20.0, 50.0]), r.choice([None, (0.3, r.choice([16, 128, 100]))])

    for i in range(r.randint(3, 9)):
        k = r.random()
        if k < 0.4:
            if own and r.random() < 0.4:
                j = r.choice(own)
                m = layers[j]["mixer"]
                cap, temp = cap_and_temp()
                layers.append(att(m["heads"], m["kv_heads"], m["dim"], m["vdim"], r.choice([0.1, 0.2, 0.3]), cap, temp, mlp(),
                                  kv_from=j))
            else:
                G = r.choice([1, 2, 4])
                d = r.choice([16, 32, 64, 64, 128, 40])
                cap, temp = cap_and_temp()
                layers.append(att(G * r.choice([1, 2, 3]), G, d, r.choice([d, d, 64, 32]), r.choice([0.1, 0.15, 0.2]), cap,
                                  temp, mlp()))
                own.append(i)
        elif k < 0.7:
            dr = r.choice([8, 16, 32, 64])
            scaling = r.choice([None, (r.choice([2.0, 4.0, 8.0]), r.choice([64, 256, 2048]), r.choice([8.0, 32.0]),
                                       r.choice([1.0, 2.0]))])
            layers.append(lat2(r.choice([1, 2, 4, 6]), r.choice([16, 32, 64]), dr, r.choice([16, 32, 64]),
                               r.choice([32, 64, 128, 100, 256]), r.choice([0.08, 0.12, 0.2]),
                               (r.choice([dr, dr, dr // 2]), r.choice([1000.0, 50000.0]), scaling),
                               r.choice([0, 17, 96, 256, 300, 600]), mlp()))
        else:
            layers.append(lat(r.choice([1, 2, 4, 8]), r.choice([16, 32, 64]), r.choice([16, 32, 64]),
                              r.choice([32, 64, 128, 100, 512]), r.choice([0.1, 0.18]), mlp()))
    return top(r.choice([100, 333, 1000]), W, r.choice([1e-6, 1e-5]), layers)


def one_layer(name: str, index: int, mlp="same") -> dict:
    """A case's configuration cut down to one of its layers (``mlp``: the layer's own, or a replacement); a layer that
    borrows keys and values comes with the layer it borrows from, as layers 0 and 1."""
    cfg = dict(CASES[name][0])
    layer = {**cfg["layers"][index], "mixer": dict(cfg["layers"][index]["mixer"])}
    if mlp != "same":
        layer["mlp"] = mlp
    src = layer["mixer"].get("kv_from")
    if src is not None:
        layer["mixer"]["kv_from"] = 0
        cfg["layers"] = [{**cfg["layers"][src], "mlp": None}, layer]
    else:
        cfg["layers"] = [layer]
    return cfg


def write(name: str, out_dir: str) -> str:
    """``config.json`` and ``model.safetensors`` for a case: seeded random weights, then the edits named above."""
    cfg, std, seed = CASES[name]
    return write_config(cfg, std, seed, out_dir)


def write_config(cfg: dict, std: float, seed: int, out_dir: str) -> str:
    from safetensors.torch import load_file

    from sharpinference_b200.weights import safetensors_io, write_random_model
    write_random_model(dict(cfg), out_dir, seed, std=std, norm_std=0.1)
    path = os.path.join(out_dir, "model.safetensors")
    tensors = load_file(path)
    g = torch.Generator().manual_seed(seed + 1000)
    for key in list(tensors):
        t = tensors[key]
        rnd = torch.rand(t.shape, generator=g)
        if key.endswith(".sink"):
            new = 4.0 * (rnd - 0.5)                      # -2 .. 2: a sink takes a visible share of a row's weight
        elif key.endswith(".router.b"):
            new = 1.0 * (rnd - 0.5)
        elif key.endswith(".norm1.b") or key.endswith(".norm2.b") or key == "final.norm.b":
            new = 0.4 * (rnd - 0.5)
        else:
            continue
        tensors[key] = new.to(t.dtype)
    safetensors_io.save_file(sorted(tensors.items()), path, metadata={"format": "pt"})
    return out_dir
