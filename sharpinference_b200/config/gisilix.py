"""``GisilixConfig``: the typed configuration of the Gisilix architecture.

A Gisilix ``config.json`` gives ``vocab``, ``width``, ``norm.eps`` (of the layer norms and of the RMS norms inside the
mixers) and ``layers``: a list of ``{"type", "mixer", "mlp"}`` with ``type`` one of

* ``"attention"``: ``heads``, ``kv_heads``, ``dim`` (query/key size a head), ``vdim``, ``scale`` (of the scores),
  ``softcap`` (scores become ``softcap * tanh(score / softcap)``), ``q_temp.coef`` / ``q_temp.every`` (the query factor
  ``1 + coef * ln(floor((p + 1) / every) + 1)`` at position ``p``), and optionally ``kv_from``: the index of an earlier
  attention layer whose cached keys and values this layer reads instead of forming its own;
* ``"latent_attention"``: ``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``; every earlier position is visible and
  there is no rotated part;
* ``"latent_attention_2"``: the same plus ``rot_dim`` rotated query/key elements a head, ``rot.base`` / ``rot.dims`` /
  ``rot.scaling`` (``factor``, ``original``, ``fast``, ``slow``: stretched frequencies with an amplitude), ``mask.size``
  (a sliding window) and a gate per head.

``mlp`` is null, ``{"kind": "dense", "ff"}`` or ``{"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"},
"shared": {"ff"} or null}``.

No size stands in code; every layer has sizes of its own.  Defaults for what a file may leave out: ``kv_heads`` =
``heads``, ``vdim`` = ``dim``, ``scale`` = (``dim`` + ``rot_dim``)^(-1/2), no ``softcap`` / ``q_temp`` / ``mask`` /
``rot.scaling`` = none of it, ``rot.dims`` = ``rot_dim``, ``rot.base`` = 10000, no ``shared`` = no shared expert.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .notedra import _merge

LAYER_TYPES = ("attention", "latent_attention", "latent_attention_2")


@dataclass(frozen=True)
class GisilixMLP:
    kind: str                   # "dense" or "moe"
    ff: int                     # dense: the hidden size; moe: an expert's
    experts: int = 0
    top: int = 0
    shared_ff: int = 0          # 0: no shared expert

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return {"kind": "dense", "ff": self.ff}
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff},
                "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass(frozen=True)
class GisilixYarn:
    factor: float
    original: float
    fast: float
    slow: float

    def to_dict(self) -> dict:
        return {"factor": self.factor, "original": self.original, "fast": self.fast, "slow": self.slow}


@dataclass(frozen=True)
class GisilixLayer:
    type: str
    mlp: Optional[GisilixMLP] = None
    heads: int = 0
    dim: int = 0                # attention: the query/key size a head; latent: the unrotated query/key elements a head
    vdim: int = 0
    scale: float = 0.0
    # attention
    kv_heads: int = 0
    softcap: float = 0.0        # 0: scores are not capped
    temp_coef: float = 0.0
    temp_every: float = 0.0     # 0: no query factor
    kv_from: Optional[int] = None
    # latent attention
    kv_rank: int = 0
    rot_dim: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    yarn: Optional[GisilixYarn] = None
    window: int = 0             # 0: every earlier position

    @property
    def head_gate(self) -> bool:
        return self.type == "latent_attention_2"

    def to_dict(self) -> dict:
        if self.type == "attention":
            mixer = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                     "scale": self.scale}
            if self.softcap:
                mixer["softcap"] = self.softcap
            if self.temp_every:
                mixer["q_temp"] = {"coef": self.temp_coef, "every": self.temp_every}
            if self.kv_from is not None:
                mixer["kv_from"] = self.kv_from
        else:
            mixer = {"heads": self.heads, "dim": self.dim, "vdim": self.vdim, "kv_rank": self.kv_rank, "scale": self.scale}
            if self.rot_dim:
                mixer["rot_dim"] = self.rot_dim
                mixer["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
                if self.yarn is not None:
                    mixer["rot"]["scaling"] = self.yarn.to_dict()
            if self.window:
                mixer["mask"] = {"size": self.window}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class GisilixConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[GisilixLayer, ...]

    architecture = "Gisilix"

    @classmethod
    def from_dict(cls, obj: dict, where: str = "config.json") -> "GisilixConfig":
        r = ConfigReader(obj, where)
        vocab, width = r.int("vocab"), r.int("width")
        eps = None
        norm = r.object("norm")
        if norm is not None:
            nr = ConfigReader(norm, f"{where}[norm]")
            eps = nr.float("eps")
            _merge(r, nr)
        raw_layers = obj.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            r.problem("key 'layers': expected a non-empty list of layer descriptions")
            raw_layers = []
        layers = []
        for i, entry in enumerate(raw_layers):
            layer = _read_layer(entry, f"{where}[layers][{i}]", r)
            if layer is not None:
                layers.append(layer)
        if r.ok:
            r.require(vocab > 0 and width > 0, f"vocab ({vocab}) and width ({width}) must be positive")
            r.require(eps >= 0, f"norm.eps must not be negative, found {eps}")
            for i, layer in enumerate(layers):
                if layer.kv_from is None:
                    continue
                j = layer.kv_from
                ok = 0 <= j < i and layers[j].type == "attention" and layers[j].kv_from is None
                r.require(ok, f"layers[{i}].mixer.kv_from ({j}) must name an earlier attention layer that forms its own "
                              f"keys and values")
                if ok:
                    src = layers[j]
                    r.require((src.kv_heads, src.dim, src.vdim) == (layer.kv_heads, layer.dim, layer.vdim),
                              f"layers[{i}] reads the keys and values of layers[{j}]: kv_heads, dim and vdim must agree "
                              f"({(layer.kv_heads, layer.dim, layer.vdim)} against {(src.kv_heads, src.dim, src.vdim)})")
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
                "layers": [layer.to_dict() for layer in self.layers]}


def _read_mlp(mlp, where: str, r: ConfigReader) -> Optional[GisilixMLP]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        r.problem(f"key 'mlp': expected an object or null, found {type(mlp).__name__}")
        return None
    mr = ConfigReader(mlp, f"{where}[mlp]")
    kind = mr.str("kind")
    out = None
    if kind == "dense":
        ff = mr.int("ff")
        if mr.ok:
            mr.require(ff > 0, f"ff ({ff}) must be positive")
            if mr.ok:
                out = GisilixMLP("dense", ff)
    elif kind == "moe":
        router, expert, shared = mr.object("router"), mr.object("expert"), mr.object("shared", None)
        experts = top = ff = None
        shared_ff = 0
        if router is not None:
            rr = ConfigReader(router, f"{where}[mlp][router]")
            experts, top = rr.int("experts"), rr.int("top")
            _merge(mr, rr)
        if expert is not None:
            xr = ConfigReader(expert, f"{where}[mlp][expert]")
            ff = xr.int("ff")
            _merge(mr, xr)
        if shared is not None:
            sr = ConfigReader(shared, f"{where}[mlp][shared]")
            shared_ff = sr.int("ff")
            _merge(mr, sr)
        if mr.ok:
            mr.require(experts > 0 and 1 <= top <= experts, f"router.top ({top}) must be 1 .. router.experts ({experts})")
            mr.require(ff > 0 and shared_ff >= 0, f"expert.ff ({ff}) must be positive and shared.ff ({shared_ff}) not negative")
            if mr.ok:
                out = GisilixMLP("moe", ff, experts=experts, top=top, shared_ff=shared_ff)
    elif kind is not None:
        mr.problem(f"key 'kind': expected 'dense' or 'moe', found {kind!r}")
    _merge(r, mr)
    return out


def _read_layer(entry, where: str, top: ConfigReader) -> Optional[GisilixLayer]:
    if not isinstance(entry, dict):
        top.problem(f"{where}: expected an object, found {type(entry).__name__}")
        return None
    r = ConfigReader(entry, where)
    kind, mixer = r.str("type"), r.object("mixer")
    mlp = _read_mlp(entry.get("mlp"), where, r)
    layer = None
    if kind is not None and kind not in LAYER_TYPES:
        r.problem(f"key 'type': expected one of {', '.join(LAYER_TYPES)}, found {kind!r}")
    elif kind is not None and mixer is not None:
        m = ConfigReader(mixer, f"{where}[mixer]")
        heads, dim = m.int("heads"), m.int("dim")
        vdim, scale = m.int("vdim", dim), m.float("scale", None)
        if kind == "attention":
            kv_heads, softcap = m.int("kv_heads", heads), m.float("softcap", 0.0)
            temp, kv_from = m.object("q_temp", None), m.int("kv_from", None)
            coef = every = 0.0
            if temp is not None:
                tr = ConfigReader(temp, f"{where}[mixer][q_temp]")
                coef, every = tr.float("coef"), tr.float("every")
                _merge(m, tr)
            if m.ok:
                m.require(heads > 0 and dim > 0 and vdim > 0, f"heads ({heads}), dim ({dim}) and vdim ({vdim}) must be positive")
                m.require(kv_heads > 0 and heads % max(kv_heads, 1) == 0,
                          f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
                m.require(softcap >= 0, f"softcap ({softcap}) must not be negative")
                m.require(temp is None or every > 0, f"q_temp.every ({every}) must be positive")
                if m.ok:
                    layer = GisilixLayer(kind, mlp, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                                         scale=float(dim) ** -0.5 if scale is None else scale, softcap=softcap,
                                         temp_coef=coef, temp_every=every, kv_from=kv_from)
        else:
            kv_rank, rot_dim = m.int("kv_rank"), m.int("rot_dim", 0)
            rot, mask = m.object("rot", None), m.object("mask", None)
            rot_dims, rot_base, yarn, window = 0, 10000.0, None, 0
            if rot is not None:
                rr = ConfigReader(rot, f"{where}[mixer][rot]")
                rot_dims, rot_base = rr.int("dims", rot_dim), rr.float("base", 10000.0)
                scaling = rr.object("scaling", None)
                if scaling is not None:
                    sr = ConfigReader(scaling, f"{where}[mixer][rot][scaling]")
                    factor, original = sr.float("factor"), sr.float("original")
                    fast, slow = sr.float("fast"), sr.float("slow")
                    if sr.ok:
                        sr.require(min(factor, original, fast, slow) > 0, "factor, original, fast and slow must be positive")
                        if sr.ok:
                            yarn = GisilixYarn(factor, original, fast, slow)
                    _merge(rr, sr)
                _merge(m, rr)
            if mask is not None:
                kr = ConfigReader(mask, f"{where}[mixer][mask]")
                window = kr.int("size")
                _merge(m, kr)
            if m.ok:
                m.require(min(heads, dim, vdim, kv_rank) > 0 and rot_dim >= 0,
                          f"heads ({heads}), dim ({dim}), vdim ({vdim}) and kv_rank ({kv_rank}) must be positive and "
                          f"rot_dim ({rot_dim}) not negative")
                m.require(rot_dims % 2 == 0 and 0 <= rot_dims <= rot_dim,
                          f"rot.dims ({rot_dims}) must be even and at most rot_dim ({rot_dim})")
                m.require(rot_base > 1, f"rot.base ({rot_base}) must be above 1")
                m.require(window >= 0, f"mask.size ({window}) must not be negative")
                if m.ok:
                    layer = GisilixLayer(kind, mlp, heads=heads, dim=dim, vdim=vdim, kv_rank=kv_rank, rot_dim=rot_dim,
                                         rot_dims=rot_dims if rot_dim else 0, rot_base=rot_base,
                                         yarn=yarn if rot_dim else None, window=window,
                                         scale=float(dim + rot_dim) ** -0.5 if scale is None else scale)
        _merge(r, m)
    _merge(top, r)
    return layer if r.ok else None
