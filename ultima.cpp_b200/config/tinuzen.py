"""Tinuzen: the typed configuration, read from the design's own config.json keys.

    architecture  "Tinuzen"
    vocab, width  sizes of the embedding table
    embedding     {"scale": constant on the token rows,
                   "bigram": {"buckets", "mul_prev", "mul_cur"}: the hashed table of token pairs}
    norm.eps      the eps of every RMS norm of the model
    loop          optional {"start", "stop", "times"}: layers start .. stop-1 run ``times`` times in a row
    layers        a list; each entry has
        type      "attention" or "parallel"
        mixer     the mixer's sizes and constants (below)
        mlp       null, or {"kind": "dense", "ff": inner size}
    attention mixer:  heads, kv_heads, dim, vdim, scale, mask {"size", "keep_first"} (optional)
    parallel mixer:   left_scale, right_scale,
        left      heads, kv_heads, dim, vdim (= dim: the values are the keys), scale,
                  rot {"base", "dims"} (optional)
        right     heads, vdim, state, groups, conv (taps), norm_groups
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from .base import ConfigError
from .sugizen import _int, _num

ATTENTION, PARALLEL = "attention", "parallel"


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int] = None
    keep_first: int = 0


@dataclass(frozen=True)
class SinkAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    scale: float
    rot_base: Optional[float] = None
    rot_dims: Optional[int] = None


@dataclass(frozen=True)
class StateSpaceConfig:
    heads: int
    vdim: int
    state: int
    groups: int
    conv: int
    norm_groups: int


@dataclass(frozen=True)
class ParallelConfig:
    left: SinkAttentionConfig
    right: StateSpaceConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class TinuzenLayer:
    kind: str
    mixer: object
    ff: Optional[int]


@dataclass(frozen=True)
class TinuzenConfig:
    vocab: int
    width: int
    eps: float
    embed_scale: float
    buckets: int
    mul_prev: int
    mul_cur: int
    layers: tuple
    loop: Optional[tuple] = None              # (start, stop, times)
    max_position_embeddings: int = 131072
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    architecture: str = "Tinuzen"
    model_type: str = "tinuzen"

    @classmethod
    def from_dict(cls, d: dict) -> "TinuzenConfig":
        vocab, width = _int(d, "vocab", ""), _int(d, "width", "")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(norm, "eps", "norm.")
        emb = d.get("embedding")
        if not isinstance(emb, dict) or not isinstance(emb.get("bigram"), dict):
            raise ConfigError("config.json: 'embedding' must be an object with 'scale' and 'bigram'")
        big = emb["bigram"]
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where}mixer must be an object")
            m, kind = L["mixer"], L.get("type")
            if kind == ATTENTION:
                heads, kv_heads = _int(m, "heads", where + "mixer."), _int(m, "kv_heads", where + "mixer.")
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {where}mixer.heads must be a multiple of kv_heads")
                window, keep = None, 0
                if m.get("mask") is not None:
                    window = _int(m["mask"], "size", where + "mixer.mask.")
                    keep = _int(m["mask"], "keep_first", where + "mixer.mask.", 0) if "keep_first" in m["mask"] else 0
                mixer = WindowAttentionConfig(heads, kv_heads, _int(m, "dim", where + "mixer."), _int(m, "vdim", where + "mixer."),
                                              _num(m, "scale", where + "mixer."), window, keep)
            elif kind == PARALLEL:
                if not isinstance(m.get("left"), dict) or not isinstance(m.get("right"), dict):
                    raise ConfigError(f"config.json: {where}mixer must hold 'left' and 'right'")
                a, r = m["left"], m["right"]
                wl, wr = where + "mixer.left.", where + "mixer.right."
                heads, kv_heads = _int(a, "heads", wl), _int(a, "kv_heads", wl)
                if heads % kv_heads:
                    raise ConfigError(f"config.json: {wl}heads must be a multiple of kv_heads")
                dim = _int(a, "dim", wl)
                if "vdim" in a and a["vdim"] != dim:
                    raise ConfigError(f"config.json: {wl}vdim must equal dim: the values are the keys")
                rot_base = rot_dims = None
                if a.get("rot") is not None:
                    rot_base, rot_dims = _num(a["rot"], "base", wl + "rot."), _int(a["rot"], "dims", wl + "rot.", 2)
                    if rot_dims % 2 or rot_dims > dim:
                        raise ConfigError(f"config.json: {wl}rot.dims must be even and at most dim")
                left = SinkAttentionConfig(heads, kv_heads, dim, _num(a, "scale", wl), rot_base, rot_dims)
                right = StateSpaceConfig(_int(r, "heads", wr), _int(r, "vdim", wr), _int(r, "state", wr), _int(r, "groups", wr),
                                         _int(r, "conv", wr), _int(r, "norm_groups", wr))
                if right.heads % right.groups:
                    raise ConfigError(f"config.json: {wr}heads must be a multiple of groups")
                if (right.heads * right.vdim) % right.norm_groups:
                    raise ConfigError(f"config.json: {wr}heads * vdim must be a multiple of norm_groups")
                mixer = ParallelConfig(left, right, _num(m, "left_scale", where + "mixer."), _num(m, "right_scale", where + "mixer."))
            else:
                raise ConfigError(f"config.json: {where}type must be '{ATTENTION}' or '{PARALLEL}', got {kind!r}")
            ff = None
            if L.get("mlp") is not None:
                f = L["mlp"]
                if f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {f.get('kind')!r}")
                ff = _int(f, "ff", where + "mlp.")
            layers.append(TinuzenLayer(kind, mixer, ff))
        loop = None
        if d.get("loop") is not None:
            lp = d["loop"]
            loop = (_int(lp, "start", "loop.", 0), _int(lp, "stop", "loop.", 0), _int(lp, "times", "loop."))
            if not (loop[0] < loop[1] <= len(layers)):
                raise ConfigError("config.json: loop.start < loop.stop <= number of layers is needed")
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width, eps=eps, embed_scale=_num(emb, "scale", "embedding.") if "scale" in emb else 1.0,
                   buckets=_int(big, "buckets", "embedding.bigram."), mul_prev=_int(big, "mul_prev", "embedding.bigram.", 0),
                   mul_cur=_int(big, "mul_cur", "embedding.bigram.", 0), layers=tuple(layers), loop=loop,
                   max_position_embeddings=int(d.get("max_positions", 131072)),
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")), eos_token_id=eos)

    def to_dict(self) -> dict:
        out = []
        for L in self.layers:
            m = L.mixer
            if L.kind == ATTENTION:
                d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
                if m.window is not None:
                    d["mask"] = {"size": m.window, "keep_first": m.keep_first}
            else:
                a, r = m.left, m.right
                left = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.dim, "scale": a.scale}
                if a.rot_dims is not None:
                    left["rot"] = {"base": a.rot_base, "dims": a.rot_dims}
                d = {"left": left, "left_scale": m.left_scale, "right_scale": m.right_scale,
                     "right": {"heads": r.heads, "vdim": r.vdim, "state": r.state, "groups": r.groups, "conv": r.conv,
                               "norm_groups": r.norm_groups}}
            out.append({"type": L.kind, "mixer": d, "mlp": None if L.ff is None else {"kind": "dense", "ff": L.ff}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "embedding": {"scale": self.embed_scale,
                           "bigram": {"buckets": self.buckets, "mul_prev": self.mul_prev, "mul_cur": self.mul_cur}},
             "layers": out, "max_positions": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.loop is not None:
            d["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
