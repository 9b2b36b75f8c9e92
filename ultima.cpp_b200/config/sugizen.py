"""Sugizen: the typed configuration, read from the design's own config.json keys.

    architecture  "Sugizen"
    vocab, width  sizes of the embedding table
    norm.eps      the eps of every RMS norm of the model
    layers        a list; each entry has
        type      "channel_delta" (gated delta-rule mixer) or "attention"
        mixer     the mixer's sizes and constants (below)
        mlp       null, or {"kind": "dense", "ff": inner size, "limit": clamp}
    channel_delta mixer:  heads, kv_heads, dim (key size), vdim (value size), conv (taps)
    attention mixer:      heads, kv_heads, dim, vdim, scale, and optionally
        rot       {"base", "dims", "scaling": {"factor", "low", "high", "original"} (optional)}
        mask      {"size": positions a block}: a token sees the earlier tokens of its own block
        kv_from   index of an earlier attention layer whose keys and values this layer reads

The inner sizes of the delta mixer's two low-rank products stand in no key: they are the shapes of
the stored tensors (``with_tensor_shapes``); a configuration written by this package carries them as
``decay_rank`` and ``gate_rank`` so that a random model can be made from it.
"""
from __future__ import annotations

from dataclasses import dataclass, replace
from typing import Optional

from .base import ConfigError

DELTA, ATTENTION = "channel_delta", "attention"


def _int(d: dict, key: str, where: str, minimum: int = 1) -> int:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, int):
        raise ConfigError(f"config.json: {where}'{key}' must be an integer, got {v!r}")
    if v < minimum:
        raise ConfigError(f"config.json: {where}'{key}' must be >= {minimum}, got {v}")
    return v


def _num(d: dict, key: str, where: str) -> float:
    v = d.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}'{key}' must be a number, got {v!r}")
    return float(v)


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int
    scaling: Optional[tuple] = None          # (factor, low, high, original)


@dataclass(frozen=True)
class MixerConfig:
    kind: str
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: Optional[int] = None               # delta
    decay_rank: Optional[int] = None         # delta; from the tensors' shapes when the file has no key
    gate_rank: Optional[int] = None
    scale: Optional[float] = None            # attention
    rot: Optional[RotaryConfig] = None
    block: Optional[int] = None
    kv_from: Optional[int] = None


@dataclass(frozen=True)
class DenseConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class SugizenLayer:
    mixer: MixerConfig
    mlp: Optional[DenseConfig]


@dataclass(frozen=True)
class SugizenConfig:
    vocab: int
    width: int
    eps: float
    layers: tuple
    max_position_embeddings: int = 131072
    torch_dtype: str = "bfloat16"
    eos_token_id: tuple = ()
    architecture: str = "Sugizen"
    model_type: str = "sugizen"

    # ---- reading ---------------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: dict) -> "SugizenConfig":
        vocab, width = _int(d, "vocab", ""), _int(d, "width", "")
        norm = d.get("norm")
        if not isinstance(norm, dict):
            raise ConfigError("config.json: 'norm' must be an object with 'eps'")
        eps = _num(norm, "eps", "norm.")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]."
            if not isinstance(L, dict) or not isinstance(L.get("mixer"), dict):
                raise ConfigError(f"config.json: {where}mixer must be an object")
            m, kind = L["mixer"], L.get("type")
            heads, kv_heads = _int(m, "heads", where + "mixer."), _int(m, "kv_heads", where + "mixer.")
            if heads % kv_heads:
                raise ConfigError(f"config.json: {where}mixer.heads must be a multiple of kv_heads")
            dim, vdim = _int(m, "dim", where + "mixer."), _int(m, "vdim", where + "mixer.")
            if kind == DELTA:
                mixer = MixerConfig(kind, heads, kv_heads, dim, vdim, conv=_int(m, "conv", where + "mixer."),
                                    decay_rank=m.get("decay_rank"), gate_rank=m.get("gate_rank"))
            elif kind == ATTENTION:
                rot = None
                if m.get("rot") is not None:
                    r = m["rot"]
                    dims = _int(r, "dims", where + "mixer.rot.", 2)
                    if dims % 2 or dims > dim:
                        raise ConfigError(f"config.json: {where}mixer.rot.dims must be even and at most dim")
                    sc = None
                    if r.get("scaling") is not None:
                        sc = tuple(_num(r["scaling"], k, where + "mixer.rot.scaling.")
                                   for k in ("factor", "low", "high", "original"))
                        if sc[1] == sc[2]:
                            raise ConfigError(f"config.json: {where}mixer.rot.scaling: low and high must differ")
                    rot = RotaryConfig(_num(r, "base", where + "mixer.rot."), dims, sc)
                block = _int(m["mask"], "size", where + "mixer.mask.") if m.get("mask") is not None else None
                kv_from = m.get("kv_from")
                if kv_from is not None:
                    src = layers[kv_from].mixer if isinstance(kv_from, int) and 0 <= kv_from < i else None
                    if src is None or src.kind != ATTENTION or src.kv_from is not None:
                        raise ConfigError(f"config.json: {where}mixer.kv_from must name an earlier attention layer "
                                          f"with keys and values of its own")
                    if (src.kv_heads, src.dim, src.vdim) != (kv_heads, dim, vdim):
                        raise ConfigError(f"config.json: {where}mixer shares layer {kv_from}'s keys and values "
                                          f"but differs from it in kv_heads, dim or vdim")
                mixer = MixerConfig(kind, heads, kv_heads, dim, vdim,
                                    scale=_num(m, "scale", where + "mixer.") if "scale" in m else dim ** -0.5,
                                    rot=rot, block=block, kv_from=kv_from)
            else:
                raise ConfigError(f"config.json: {where}type must be '{DELTA}' or '{ATTENTION}', got {kind!r}")
            mlp = None
            if L.get("mlp") is not None:
                f = L["mlp"]
                if f.get("kind") != "dense":
                    raise ConfigError(f"config.json: {where}mlp.kind must be 'dense', got {f.get('kind')!r}")
                mlp = DenseConfig(_int(f, "ff", where + "mlp."), _num(f, "limit", where + "mlp."))
            layers.append(SugizenLayer(mixer, mlp))
        eos = d.get("eos_token_id")
        eos = () if eos is None else ((eos,) if isinstance(eos, int) else tuple(eos))
        return cls(vocab=vocab, width=width, eps=eps, layers=tuple(layers),
                   max_position_embeddings=int(d.get("max_positions", 131072)),
                   torch_dtype=str(d.get("torch_dtype", "bfloat16")), eos_token_id=eos)

    # ---- sizes that only the tensors give ------------------------------------------------------
    @property
    def needs_tensor_shapes(self) -> bool:
        return any(L.mixer.kind == DELTA and (L.mixer.decay_rank is None or L.mixer.gate_rank is None)
                   for L in self.layers)

    def with_tensor_shapes(self, shapes: dict) -> "SugizenConfig":
        """The configuration with the low-rank sizes read from the stored tensors' shapes
        (``shapes``: stored name -> shape)."""
        layers = []
        for i, L in enumerate(self.layers):
            m = L.mixer
            if m.kind == DELTA:
                for field, name in (("decay_rank", f"l{i}.mix.a1"), ("gate_rank", f"l{i}.mix.g1")):
                    if getattr(m, field) is None:
                        if name not in shapes or len(shapes[name]) != 2:
                            raise ConfigError(f"the model's files hold no matrix '{name}' to take the layer's "
                                              f"{field} from")
                        m = replace(m, **{field: int(shapes[name][0])})
            layers.append(SugizenLayer(m, L.mlp))
        return replace(self, layers=tuple(layers))

    # ---- writing ---------------------------------------------------------------------------
    def to_dict(self) -> dict:
        out = []
        for L in self.layers:
            m = L.mixer
            d = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim}
            if m.kind == DELTA:
                d["conv"] = m.conv
                if m.decay_rank is not None:
                    d["decay_rank"] = m.decay_rank
                if m.gate_rank is not None:
                    d["gate_rank"] = m.gate_rank
            else:
                d["scale"] = m.scale
                if m.rot is not None:
                    d["rot"] = {"base": m.rot.base, "dims": m.rot.dims}
                    if m.rot.scaling is not None:
                        d["rot"]["scaling"] = dict(zip(("factor", "low", "high", "original"), m.rot.scaling))
                if m.block is not None:
                    d["mask"] = {"size": m.block}
                if m.kv_from is not None:
                    d["kv_from"] = m.kv_from
            out.append({"type": m.kind, "mixer": d,
                        "mlp": None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff, "limit": L.mlp.limit}})
        d = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": {"eps": self.eps},
             "layers": out, "max_positions": self.max_position_embeddings, "torch_dtype": self.torch_dtype}
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
