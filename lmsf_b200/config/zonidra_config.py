"""The typed configuration of the Zonidra design, read from config.json.

config.json of this design is nested: `layers` lists every layer with its `type` (which mixer), the mixer's sizes and constants
(`mixer`: heads, sizes per head, `rot`, `mask`, `scale`, and `kv_from` for a layer that reads another layer's keys and values)
and its feed-forward (`mlp`: dense, routed experts, or null for none); `embedding` holds the scale and the hashed pair table;
`norm.eps`, `vocab` and `width` are global.  Every size and every constant that may differ between models of the design is
read from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ConfigError

MIXER_TYPES = ("attention",)
MLP_KINDS = ("dense", "moe")


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _int(v, what: str, least: int = 1) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v < least:
        raise ConfigError(f"config.json: {what} must be an integer of at least {least}, got {v!r}")
    return v


@dataclass
class ZonidraRotation:
    dims: int                                            # how many values at the front of every head are rotated
    base: float
    scaling: Optional[Dict[str, float]] = None           # factor, low, high, original: frequencies stretched by wavelength


@dataclass
class ZonidraMixer:
    heads: int
    kv_heads: int
    dim: int                                             # query/key values per head
    vdim: int                                            # values per value head
    scale: float
    rot: Optional[ZonidraRotation] = None
    window: Optional[int] = None                         # mask.size; None: every earlier token is seen
    keep_first: int = 0                                  # mask.keep_first: the first tokens stay visible behind the window
    kv_from: Optional[int] = None                        # the layer whose cached keys and values this one reads


@dataclass
class ZonidraFeedForward:
    kind: str
    ff: int                                              # dense: hidden size; moe: an expert's hidden size
    experts: int = 0
    top: int = 0
    identity: int = 0                                    # router outputs behind the experts that return the input
    route_scale: float = 1.0
    shared_ff: int = 0                                   # 0: no shared expert


@dataclass
class ZonidraLayer:
    mixer: ZonidraMixer
    mlp: Optional[ZonidraFeedForward]


@dataclass
class ZonidraConfig:
    vocab: int
    width: int
    eps: float
    layers: List[ZonidraLayer]
    embed_scale: float = 1.0
    pair_buckets: int = 0                                # 0: no pair table
    pair_mul_prev: int = 0
    pair_mul_cur: int = 0
    max_model_len: int = 1 << 20                         # bounded by the cache alone
    torch_dtype: str = "bfloat16"
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "ZonidraConfig":
        vocab = _int(_need(d, "vocab", "the model"), "vocab")
        width = _int(_need(d, "width", "the model"), "width")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        if not (eps > 0):
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[ZonidraLayer] = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
            m, wm = _need(L, "mixer", where), where + ".mixer"
            heads = _int(_need(m, "heads", wm), "heads")
            kv_heads = _int(m.get("kv_heads") or heads, "kv_heads")
            if heads % kv_heads:
                raise ConfigError(f"config.json: {wm}: {heads} heads over {kv_heads} kv heads")
            dim = _int(_need(m, "dim", wm), "dim")
            mixer = ZonidraMixer(heads, kv_heads, dim, _int(m.get("vdim") or dim, "vdim"),
                                 float(m["scale"]) if m.get("scale") is not None else dim ** -0.5)
            rot = m.get("rot")
            if rot and rot.get("dims"):
                dims = _int(rot["dims"], "rot.dims")
                if dims % 2 or dims > dim:
                    raise ConfigError(f"config.json: {wm}.rot.dims must be even and at most dim ({dim})")
                base = float(rot.get("base", 10000.0))
                if not (base > 0):
                    raise ConfigError(f"config.json: {wm}.rot.base must be positive")
                sc = rot.get("scaling")
                if sc:
                    sc = {k: float(_need(sc, k, wm + ".rot.scaling")) for k in ("factor", "low", "high", "original")}
                    if not (sc["high"] > sc["low"] and sc["factor"] > 0 and sc["original"] > 0):
                        raise ConfigError(f"config.json: {wm}.rot.scaling {sc!r} is not a stretch of wavelengths")
                mixer.rot = ZonidraRotation(dims, base, sc or None)
            mask = m.get("mask")
            if mask and mask.get("size") is not None:
                mixer.window = _int(mask["size"], "mask.size")
                mixer.keep_first = _int(mask.get("keep_first") or 0, "mask.keep_first", 0)
            if m.get("kv_from") is not None:
                j = _int(m["kv_from"], "kv_from", 0)
                if j >= i or layers[j].mixer.kv_from is not None:
                    raise ConfigError(f"config.json: {wm}.kv_from {j} must name an earlier layer with keys and values of its own")
                o = layers[j].mixer
                if (o.kv_heads, o.dim, o.vdim) != (mixer.kv_heads, mixer.dim, mixer.vdim):
                    raise ConfigError(f"config.json: {wm}.kv_from {j}: the key/value heads and sizes of the two layers differ")
                mixer.kv_from = j
            f = L.get("mlp")
            mlp = None
            if f:
                wf = where + ".mlp"
                kind_f = _need(f, "kind", wf)
                if kind_f not in MLP_KINDS:
                    raise ConfigError(f"config.json: {wf}.kind {kind_f!r} is not a feed-forward of this design ({', '.join(MLP_KINDS)})")
                if kind_f == "dense":
                    mlp = ZonidraFeedForward("dense", _int(_need(f, "ff", wf), "ff"))
                else:
                    r = _need(f, "router", wf)
                    mlp = ZonidraFeedForward("moe", _int(_need(_need(f, "expert", wf), "ff", wf + ".expert"), "ff"),
                                             _int(_need(r, "experts", wf + ".router"), "experts"),
                                             _int(_need(r, "top", wf + ".router"), "top"),
                                             _int(r.get("identity") or 0, "identity", 0),
                                             float(r["scale"]) if r.get("scale") is not None else 1.0)
                    if mlp.top > mlp.experts + mlp.identity:
                        raise ConfigError(f"config.json: {wf}.router: top {mlp.top} of {mlp.experts + mlp.identity} outputs")
                    sh = f.get("shared")
                    if sh:
                        mlp.shared_ff = _int(_need(sh, "ff", wf + ".shared"), "ff")
            layers.append(ZonidraLayer(mixer, mlp))
        cfg = ZonidraConfig(vocab, width, eps, layers, raw=dict(d))
        e = d.get("embedding") or {}
        if e.get("scale") is not None:
            cfg.embed_scale = float(e["scale"])
        b = e.get("bigram")
        if b:
            cfg.pair_buckets = _int(_need(b, "buckets", "embedding.bigram"), "buckets")
            cfg.pair_mul_prev = _int(_need(b, "mul_prev", "embedding.bigram"), "mul_prev", 0)
            cfg.pair_mul_cur = _int(_need(b, "mul_cur", "embedding.bigram"), "mul_cur", 0)
        if d.get("max_len"):
            cfg.max_model_len = _int(d["max_len"], "max_len")
        dt = d.get("torch_dtype", d.get("dtype"))
        if dt is not None:
            cfg.torch_dtype = str(dt).replace("torch.", "")
        eos = d.get("eos_token_id")
        if eos is not None:
            cfg.eos_token_ids = [int(x) for x in (eos if isinstance(eos, (list, tuple)) else [eos])]
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)
