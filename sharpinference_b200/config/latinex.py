"""``LatinexConfig``: the typed configuration of the Latinex architecture.

A Latinex ``config.json`` gives

* ``vocab``, ``width``, ``logit_scale``, ``embedding.scale`` (the embedding row is multiplied by it), ``norm.eps``
  (of the RMS norms inside the mixers; the layers' own norm is an element-wise ``tanh`` norm and has none);
* ``layers``: a list of ``{"type", "mixer", "mlp"}`` with ``type`` one of

  - ``"latent_attention"``: ``heads``, ``dim`` (unrotated) and ``rot_dim`` (rotated) query/key elements a head,
    ``vdim``, the latent sizes ``q_rank`` and ``kv_rank``, ``scale`` (of the scores), ``rot.base`` / ``rot.dims``;
  - ``"attention"``: ``heads``, ``kv_heads``, ``dim``, ``vdim`` (the values are the keys, so ``vdim`` = ``dim``),
    ``scale``, ``bias_max`` (the distance at which the learned distance bias reaches its last bucket; the number of
    buckets is the stored table's, or ``bias_buckets`` where there is no file),
    ``mask.size`` (sliding window) and ``mask.keep_first`` (first positions that stay visible);
  - ``"mamba2"``: ``heads``, ``vdim``, ``state``, ``groups``, ``conv`` (taps), ``norm_groups``;

  ``mlp`` is null or ``{"kind": "moe", "router": {"experts", "top"}, "expert": {"ff"}, "shared": {"ff"} or null}``.

No size stands in code; every layer has sizes of its own.  Defaults for what a file may leave out: ``kv_heads`` =
``heads``, ``vdim`` = ``dim``, ``scale`` = (``dim`` + ``rot_dim``)^(-1/2), no ``rot`` = no rotation, ``rot.dims`` =
``rot_dim``, ``rot.base`` = 10000, no ``mask`` = every earlier position, ``keep_first`` = 0, ``groups`` =
``norm_groups`` = 1, no ``shared`` = no shared expert, ``logit_scale`` = ``embedding.scale`` = 1.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

from .base import ConfigReader
from .notedra import _merge

LAYER_TYPES = ("latent_attention", "attention", "mamba2")


@dataclass(frozen=True)
class LatinexMoE:
    experts: int
    top: int
    ff: int
    shared_ff: int = 0          # 0: no shared expert

    def to_dict(self) -> dict:
        return {"kind": "moe", "router": {"experts": self.experts, "top": self.top}, "expert": {"ff": self.ff},
                "shared": {"ff": self.shared_ff} if self.shared_ff else None}


@dataclass(frozen=True)
class LatinexLayer:
    type: str
    mlp: Optional[LatinexMoE] = None
    heads: int = 0
    dim: int = 0                # latent_attention: unrotated elements a head; attention: the head size
    vdim: int = 0
    scale: float = 0.0
    # latent_attention
    rot_dim: int = 0
    q_rank: int = 0
    kv_rank: int = 0
    rot_dims: int = 0
    rot_base: float = 10000.0
    # attention
    kv_heads: int = 0
    bias_max: int = 0
    bias_buckets: int = 0       # rows of the distance table (0: as stored)
    window: int = 0             # 0: every earlier position
    keep_first: int = 0
    # mamba2
    state: int = 0
    groups: int = 1
    conv: int = 0
    norm_groups: int = 1

    def to_dict(self) -> dict:
        if self.type == "latent_attention":
            mixer = {"heads": self.heads, "dim": self.dim, "rot_dim": self.rot_dim, "vdim": self.vdim,
                     "q_rank": self.q_rank, "kv_rank": self.kv_rank, "scale": self.scale,
                     "rot": {"base": self.rot_base, "dims": self.rot_dims}}
        elif self.type == "attention":
            mixer = {"heads": self.heads, "kv_heads": self.kv_heads, "dim": self.dim, "vdim": self.vdim,
                     "scale": self.scale, "bias_max": self.bias_max}
            if self.bias_buckets:
                mixer["bias_buckets"] = self.bias_buckets
            if self.window:
                mixer["mask"] = {"size": self.window, "keep_first": self.keep_first}
        else:
            mixer = {"heads": self.heads, "vdim": self.vdim, "state": self.state, "groups": self.groups,
                     "conv": self.conv, "norm_groups": self.norm_groups}
        return {"type": self.type, "mixer": mixer, "mlp": None if self.mlp is None else self.mlp.to_dict()}


@dataclass(frozen=True)
class LatinexConfig:
    vocab: int
    width: int
    eps: float
    embedding_scale: float
    logit_scale: float
    layers: Tuple[LatinexLayer, ...]

    architecture = "Latinex"

    @classmethod
    def from_dict(cls, obj: dict, where: str = "config.json") -> "LatinexConfig":
        r = ConfigReader(obj, where)
        vocab, width, logit_scale = r.int("vocab"), r.int("width"), r.float("logit_scale", 1.0)
        eps, emb_scale = None, 1.0
        norm = r.object("norm")
        if norm is not None:
            nr = ConfigReader(norm, f"{where}[norm]")
            eps = nr.float("eps")
            _merge(r, nr)
        emb = r.object("embedding", None)
        if emb is not None:
            er = ConfigReader(emb, f"{where}[embedding]")
            emb_scale = er.float("scale", 1.0)
            _merge(r, er)
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
        r.finish()
        return cls(vocab=vocab, width=width, eps=eps, embedding_scale=emb_scale, logit_scale=logit_scale,
                   layers=tuple(layers))

    def to_dict(self) -> dict:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width,
                "logit_scale": self.logit_scale, "embedding": {"scale": self.embedding_scale},
                "norm": {"eps": self.eps}, "layers": [layer.to_dict() for layer in self.layers]}


def _read_mlp(mlp, where: str, r: ConfigReader) -> Optional[LatinexMoE]:
    if mlp is None:
        return None
    if not isinstance(mlp, dict):
        r.problem(f"key 'mlp': expected an object or null, found {type(mlp).__name__}")
        return None
    mr = ConfigReader(mlp, f"{where}[mlp]")
    kind, router, expert, shared = mr.str("kind"), mr.object("router"), mr.object("expert"), mr.object("shared", None)
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
    out = None
    if mr.ok:
        mr.require(kind == "moe", f"key 'kind': expected 'moe', found {kind!r}")
        mr.require(experts > 0 and 1 <= top <= experts, f"router.top ({top}) must be 1 .. router.experts ({experts})")
        mr.require(ff > 0 and shared_ff >= 0, f"expert.ff ({ff}) must be positive and shared.ff ({shared_ff}) not negative")
        if mr.ok:
            out = LatinexMoE(experts, top, ff, shared_ff)
    _merge(r, mr)
    return out


def _read_layer(entry, where: str, top: ConfigReader) -> Optional[LatinexLayer]:
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
        if kind == "latent_attention":
            heads, dim, rot_dim = m.int("heads"), m.int("dim"), m.int("rot_dim", 0)
            vdim, q_rank, kv_rank = m.int("vdim", dim), m.int("q_rank"), m.int("kv_rank")
            scale, rot = m.float("scale", None), m.object("rot", None)
            rot_dims, rot_base = 0, 10000.0
            if rot is not None:
                rr = ConfigReader(rot, f"{where}[mixer][rot]")
                rot_dims, rot_base = rr.int("dims", rot_dim), rr.float("base", 10000.0)
                _merge(m, rr)
            if m.ok:
                m.require(min(heads, dim, vdim, q_rank, kv_rank) > 0 and rot_dim >= 0,
                          f"heads ({heads}), dim ({dim}), vdim ({vdim}), q_rank ({q_rank}) and kv_rank ({kv_rank}) must "
                          f"be positive and rot_dim ({rot_dim}) not negative")
                m.require(rot_dims % 2 == 0 and 0 <= rot_dims <= rot_dim,
                          f"rot.dims ({rot_dims}) must be even and at most rot_dim ({rot_dim})")
                if m.ok:
                    layer = LatinexLayer(kind, mlp, heads=heads, dim=dim, vdim=vdim, rot_dim=rot_dim, q_rank=q_rank,
                                         kv_rank=kv_rank, rot_dims=rot_dims, rot_base=rot_base,
                                         scale=float(dim + rot_dim) ** -0.5 if scale is None else scale)
        elif kind == "attention":
            heads, dim = m.int("heads"), m.int("dim")
            kv_heads, vdim, scale = m.int("kv_heads", heads), m.int("vdim", dim), m.float("scale", None)
            bias_max, mask, buckets = m.int("bias_max"), m.object("mask", None), m.int("bias_buckets", 0)
            window = keep_first = 0
            if mask is not None:
                kr = ConfigReader(mask, f"{where}[mixer][mask]")
                window, keep_first = kr.int("size"), kr.int("keep_first", 0)
                _merge(m, kr)
            if m.ok:
                m.require(heads > 0 and dim > 0, f"heads ({heads}) and dim ({dim}) must be positive")
                m.require(kv_heads > 0 and heads % kv_heads == 0,
                          f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
                m.require(vdim == dim, f"the values are the keys: vdim ({vdim}) must equal dim ({dim})")
                m.require(dim % 2 == 0, f"dim ({dim}) must be even")
                m.require(bias_max > 0 and window >= 0 and keep_first >= 0,
                          f"bias_max ({bias_max}) must be positive, mask.size ({window}) and mask.keep_first "
                          f"({keep_first}) not negative")
                if m.ok:
                    layer = LatinexLayer(kind, mlp, heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim,
                                         scale=float(dim) ** -0.5 if scale is None else scale, bias_max=bias_max,
                                         bias_buckets=max(buckets, 0),
                                         window=window, keep_first=keep_first if window else 0)
        else:
            heads, vdim, state = m.int("heads"), m.int("vdim"), m.int("state")
            groups, conv, norm_groups = m.int("groups", 1), m.int("conv"), m.int("norm_groups", 1)
            if m.ok:
                m.require(min(heads, vdim, state, groups, conv, norm_groups) > 0,
                          "heads, vdim, state, groups, conv and norm_groups must be positive")
                m.require(groups > 0 and heads % max(groups, 1) == 0,
                          f"heads ({heads}) must be a multiple of groups ({groups})")
                m.require(norm_groups > 0 and (heads * vdim) % max(norm_groups, 1) == 0,
                          f"norm_groups ({norm_groups}) must divide heads * vdim ({heads * vdim})")
                if m.ok:
                    layer = LatinexLayer(kind, mlp, heads=heads, vdim=vdim, state=state, groups=groups, conv=conv,
                                         norm_groups=norm_groups)
        _merge(r, m)
    _merge(top, r)
    return layer if r.ok else None
