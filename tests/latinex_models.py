"""Small Latinex configurations for the tests, and folders with random weights for them.

The configurations differ from each other in every size; between them they cover: latent attention whose cached row
(latent plus rotated part) is and is not a multiple of 16, with a rotation of all and of part of the rotated
elements and of none, one head and several, values wider and narrower than keys; windowed attention with one key
head, one per query head and groups, windows of 1, 2, 5, 33, 64, 70, 100 and 130 positions, none to 70 kept first
positions (fewer and more than a page, more than the window), distance tables of 2 to 32 rows; state-space layers
with one to three groups, one to three norm groups, 1 to 200 states and one to five taps; layers without a
feed-forward; one to three experts a row, a single expert, no shared expert; widths that are no multiple of 8.

Random weights alone would hide some faults, so ``write`` edits a few tensors afterwards: ``A_log`` and ``dt_bias`` of
the state-space layers are lowered (memories that keep what they saw hundreds of tokens ago), the distance tables
get entries of both signs and size 1, the norms' ``alpha`` stay below 1 so that the squashing does not saturate, and
the attention score factors in the configurations are large (single keys carry a row's output, so a window that is
one position off shows).
"""
from __future__ import annotations

import os

import torch


def _moe(experts, top, ff, shared):
    return {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff},
            "shared": {"ff": shared} if shared else None}


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot, mlp):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank, "scale": scale}
    if rot:
        m["rot"] = {"dims": rot[0], "base": rot[1]}
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _att(heads, kv, dim, scale, buckets, far, window, keep, mlp):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "bias_max": far, "bias_buckets": buckets}
    if window:
        m["mask"] = {"size": window, "keep_first": keep}
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _ssd(heads, vdim, state, groups, conv, norm_groups, mlp):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp}


def _top(vocab, width, eps, emb_scale, logit_scale, layers):
    return {"architecture": "Latinex", "vocab": vocab, "width": width, "logit_scale": logit_scale,
            "embedding": {"scale": emb_scale}, "norm": {"eps": eps}, "layers": layers}


# A: every mixer once; a cached latent row of 40 + 8 = 48 elements; a window of 33 with 5 kept positions; two experts
# a row with a shared expert; a state-space layer without a feed-forward.
CASE_A = _top(97, 64, 1e-5, 2.0, 0.7, [
    _lat(4, 16, 8, 24, 32, 40, 0.9, (8, 100.0), _moe(4, 2, 24, 40)),
    _att(4, 2, 16, 1.1, 8, 40, 33, 5, _moe(3, 1, 16, 0)),
    _ssd(4, 8, 16, 2, 3, 2, None),
])

# B: a width that is no multiple of 8 (no library product and no tensor-core expert product anywhere); a latent row
# of 20 + 6 = 26 elements of which 4 are rotated; a window of 70 (longer than a page) with 70 kept positions; windows
# of 1 and 2; three experts a row out of three.
CASE_B = _top(61, 52, 1e-4, 1.0, 1.0, [
    _att(3, 3, 10, 0.8, 4, 9, 70, 70, _moe(3, 3, 12, 20)),
    _lat(2, 12, 6, 10, 14, 20, 0.7, (4, 300.0), None),
    _ssd(2, 13, 5, 1, 1, 1, _moe(2, 1, 18, 6)),
    _att(2, 1, 6, 1.5, 2, 3, 1, 0, None),
    _att(4, 2, 8, 1.2, 6, 30, 2, 1, _moe(5, 2, 10, 0)),
])

# C: head sizes that the tensor-core attention kernels take (64 for windowed attention; a latent row of 96 + 32 =
# 128), a window of exactly a page with 3 kept positions and one of 130 with 64, a table of 32 rows; two groups
# of 64 states; a single expert.
CASE_C = _top(131, 128, 1e-6, 4.0, 0.5, [
    _lat(4, 32, 32, 48, 64, 96, 0.35, (32, 30000.0), _moe(1, 1, 32, 32)),
    _att(4, 1, 64, 0.4, 32, 150, 64, 3, _moe(8, 2, 32, 48)),
    _ssd(4, 32, 64, 2, 4, 1, _moe(4, 1, 64, 0)),
    _att(2, 2, 64, 0.3, 16, 200, 130, 64, None),
    _lat(2, 64, 16, 32, 48, 64, 0.3, (16, 1000.0), None),
])

# D: ones and twos wherever a size can be one or two.
CASE_D = _top(23, 16, 1e-5, 1.5, 2.0, [
    _lat(1, 2, 2, 2, 2, 2, 1.2, (2, 10.0), _moe(2, 2, 1, 1)),
    _ssd(1, 2, 1, 1, 2, 1, None),
    _att(1, 1, 2, 1.4, 2, 2, 2, 2, _moe(1, 1, 2, 0)),
    _lat(2, 2, 0, 1, 1, 1, 0.9, None, None),
])

# E: the largest sizes: 200 states with five taps and three norm groups; a latent row of 192 + 64 = 256 elements;
# attention heads of 128 with a window of 100 and 20 kept positions; a window of 5.
CASE_E = _top(50, 96, 1e-5, 3.0, 1.0, [
    _ssd(3, 16, 200, 3, 5, 3, _moe(4, 3, 16, 8)),
    _lat(2, 48, 64, 40, 24, 192, 0.2, (64, 10000.0), None),
    _att(2, 1, 128, 0.25, 12, 64, 100, 20, _moe(2, 1, 24, 24)),
    _att(3, 1, 16, 1.0, 10, 16, 5, 2, None),
])

# config, std of the weights, seed
CASES = {"A": (CASE_A, 0.15, 41), "B": (CASE_B, 0.18, 42), "C": (CASE_C, 0.1, 43), "D": (CASE_D, 0.5, 44),
         "E": (CASE_E, 0.1, 45)}


def one_layer(name: str, index: int, mlp="same") -> dict:
    """A case's configuration cut down to one of its layers (``mlp``: the layer's own, or a replacement)."""
    cfg = dict(CASES[name][0])
    layer = dict(cfg["layers"][index])
    if mlp != "same":
        layer["mlp"] = mlp
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
        if key.endswith(".A_log"):
            new = -4.0 + 3.5 * rnd                       # decay rates exp(-4) to exp(-0.5) per unit step
        elif key.endswith(".dt_bias"):
            new = -3.0 + 3.0 * rnd
        elif key.endswith(".rel"):
            new = 2.0 * (rnd - 0.5)
        elif key.endswith(".alpha"):
            new = 0.3 + 0.5 * rnd
        elif key.endswith(".conv.b") or key.endswith(".q.b") or key.endswith(".k.b"):
            new = 0.6 * (rnd - 0.5)
        else:
            continue
        tensors[key] = new.to(t.dtype)
    safetensors_io.save_file(sorted(tensors.items()), path, metadata={"format": "pt"})
    return out_dir
