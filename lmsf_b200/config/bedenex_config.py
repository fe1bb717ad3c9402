"""The typed configuration of the Bedenex design, read from config.json.

config.json of this design is nested: `layers` lists every layer with its `type` (which mixer), the mixer's sizes
(`mixer`) and its feed-forward (`mlp`: dense, routed experts, or null for none); `loop` names a span of layers that runs
several times; `norm.eps`, `vocab` and `width` are global.  Every size and every constant that may differ between models
of the design is read from there; nothing is assumed equal between layers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .model_config import ConfigError

MIXER_TYPES = ("attention", "latent_attention")
MLP_KINDS = ("dense", "moe")


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks {key!r}")
    return d[key]


def _pos_int(v, what: str) -> int:
    if isinstance(v, bool) or not isinstance(v, int) or v <= 0:
        raise ConfigError(f"config.json: {what} must be a positive integer, got {v!r}")
    return v


@dataclass
class BedenexMixer:
    type: str
    heads: int
    dim: int                                             # unrotated query/key values per head
    vdim: int
    scale: Optional[float] = None                        # None: (query/key values per head) ** -0.5
    kv_heads: int = 0                                    # attention: key/value heads
    chunk: Optional[int] = None                          # attention: mask.size; None: every earlier token is seen
    kv_rank: int = 0                                     # latent attention: size of the cached vector
    rot_dim: int = 0                                     # latent attention: rotated query/key values per head
    rot_dims: int = 0                                    # how many of those are rotated (the rest pass unchanged)
    rot_base: float = 10000.0


@dataclass
class BedenexFeedForward:
    kind: str
    ff: int                                              # dense: hidden size; moe: an expert's hidden size
    experts: int = 0
    top: int = 0


@dataclass
class BedenexLayer:
    mixer: BedenexMixer
    mlp: Optional[BedenexFeedForward]


@dataclass
class BedenexConfig:
    vocab: int
    width: int
    eps: float
    layers: List[BedenexLayer]
    loop_start: int = 0
    loop_stop: int = 0
    loop_times: int = 1                                  # a span [start, stop) that runs `times` times; no span: stop == start
    has_loop: bool = False
    max_model_len: int = 1 << 20                         # bounded by the cache alone
    torch_dtype: str = "bfloat16"
    eos_token_ids: List[int] = field(default_factory=list)
    raw: Dict[str, Any] = field(default_factory=dict)

    @staticmethod
    def from_dict(d: Dict[str, Any]) -> "BedenexConfig":
        vocab = _pos_int(_need(d, "vocab", "the model"), "vocab")
        width = _pos_int(_need(d, "width", "the model"), "width")
        eps = float(_need(_need(d, "norm", "the model"), "eps", "norm"))
        if not (eps > 0):
            raise ConfigError(f"config.json: norm.eps must be positive, got {eps!r}")
        raw_layers = _need(d, "layers", "the model")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = _need(L, "type", where)
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design ({', '.join(MIXER_TYPES)})")
            m = _need(L, "mixer", where)
            mixer = BedenexMixer(kind, _pos_int(_need(m, "heads", where + ".mixer"), "heads"),
                                 _pos_int(_need(m, "dim", where + ".mixer"), "dim"),
                                 _pos_int(_need(m, "vdim", where + ".mixer"), "vdim"))
            mixer.scale = float(m["scale"]) if m.get("scale") is not None else None
            if kind == "attention":
                mixer.kv_heads = _pos_int(m.get("kv_heads") or mixer.heads, "kv_heads")
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {where}.mixer: {mixer.heads} heads over {mixer.kv_heads} kv heads")
                mask = m.get("mask")
                if mask and mask.get("size") is not None:
                    mixer.chunk = _pos_int(mask["size"], "mask.size")
            else:
                mixer.kv_rank = _pos_int(_need(m, "kv_rank", where + ".mixer"), "kv_rank")
                mixer.rot_dim = _pos_int(_need(m, "rot_dim", where + ".mixer"), "rot_dim")
                rot = m.get("rot") or {}
                mixer.rot_dims = _pos_int(rot.get("dims", mixer.rot_dim), "rot.dims")
                if mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most rot_dim ({mixer.rot_dim})")
                mixer.rot_base = float(rot.get("base", 10000.0))
                if not (mixer.rot_base > 0):
                    raise ConfigError(f"config.json: {where}.mixer.rot.base must be positive")
            f = L.get("mlp")
            mlp = None
            if f:
                kind_f = _need(f, "kind", where + ".mlp")
                if kind_f not in MLP_KINDS:
                    raise ConfigError(f"config.json: {where}.mlp.kind {kind_f!r} is not a feed-forward of this design "
                                      f"({', '.join(MLP_KINDS)})")
                if kind_f == "dense":
                    mlp = BedenexFeedForward("dense", _pos_int(_need(f, "ff", where + ".mlp"), "ff"))
                else:
                    r = _need(f, "router", where + ".mlp")
                    mlp = BedenexFeedForward("moe", _pos_int(_need(_need(f, "expert", where + ".mlp"), "ff", where + ".mlp.expert"), "ff"),
                                             _pos_int(_need(r, "experts", where + ".mlp.router"), "experts"),
                                             _pos_int(_need(r, "top", where + ".mlp.router"), "top"))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"config.json: {where}.mlp.router: top {mlp.top} of {mlp.experts} experts")
            layers.append(BedenexLayer(mixer, mlp))
        cfg = BedenexConfig(vocab, width, eps, layers, raw=dict(d))
        loop = d.get("loop")
        if loop:
            start, stop, times = int(_need(loop, "start", "loop")), int(_need(loop, "stop", "loop")), int(_need(loop, "times", "loop"))
            if not (0 <= start <= stop <= len(layers)) or times < 1:
                raise ConfigError(f"config.json: loop {loop!r} does not fit {len(layers)} layers")
            if stop > start:
                cfg.loop_start, cfg.loop_stop, cfg.loop_times, cfg.has_loop = start, stop, times, True
        if d.get("max_len"):
            cfg.max_model_len = _pos_int(d["max_len"], "max_len")
        dt = d.get("torch_dtype", d.get("dtype"))
        if dt is not None:
            cfg.torch_dtype = str(dt).replace("torch.", "")
        eos = d.get("eos_token_id")
        if eos is not None:
            cfg.eos_token_ids = [int(e) for e in (eos if isinstance(eos, (list, tuple)) else [eos])]
        return cfg

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)
