"""Small Sugizen configurations for the tests.  They differ from one another in every size and option:
order of layers, widths (one not a multiple of 8), heads and groups, key and value sizes (equal and not,
multiples of 8, 16, 32 and not), taps, low-rank sizes, rotation of part or all of a head, with and
without frequency scaling, with and without a block mask, blocks that end on and off a page's border, a
layer without feed-forward, and layers that read another layer's keys and values."""


def _attention(heads, kv_heads, dim, vdim, scale, rot=None, mask=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    if mask is not None:
        m["mask"] = {"size": mask}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _delta(heads, kv_heads, dim, vdim, conv, decay_rank, gate_rank):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "conv": conv, "decay_rank": decay_rank,
            "gate_rank": gate_rank}


def _layer(kind, mixer, ff=None, limit=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


_ROT_A = {"base": 10000.0, "dims": 16, "scaling": {"factor": 8.0, "low": 1.0, "high": 3.0, "original": 64}}
_ROT_B = {"base": 300.0, "dims": 20}
_ROT_C = {"base": 50000.0, "dims": 64, "scaling": {"factor": 2.0, "low": 2.0, "high": 8.0, "original": 256}}

MIXED = {"architecture": "Sugizen", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "layers": [
    _layer("attention", _attention(4, 2, 32, 16, 0.2, _ROT_A, 24), 96, 2.0),
    _layer("channel_delta", _delta(4, 2, 24, 40, 3, 5, 7), 80, 1.0),
    _layer("attention", _attention(4, 2, 32, 16, 0.3, _ROT_A, 24, kv_from=0), 96, 2.0),
    _layer("channel_delta", _delta(3, 3, 16, 32, 2, 4, 4)),
    _layer("attention", _attention(6, 2, 32, 16, 0.25, _ROT_A, 10, kv_from=0)),
]}

ODD = {"architecture": "Sugizen", "vocab": 257, "width": 100, "norm": {"eps": 3e-6}, "layers": [
    _layer("channel_delta", _delta(2, 1, 72, 33, 5, 3, 9), 131, 0.7),
    _layer("attention", _attention(3, 3, 20, 20, 0.22, _ROT_B), 60, 5.0),
    _layer("attention", _attention(3, 1, 28, 12, 0.2), 60, 5.0),
    _layer("channel_delta", _delta(4, 4, 130, 8, 1, 2, 2), 64, 1.5),
]}

WIDE = {"architecture": "Sugizen", "vocab": 384, "width": 128, "norm": {"eps": 1e-6}, "layers": [
    _layer("channel_delta", _delta(4, 2, 64, 64, 4, 16, 8), 256, 1.5),
    _layer("attention", _attention(4, 1, 64, 64, 0.125, _ROT_C, 64), 256, 1.5),
    _layer("attention", _attention(8, 1, 64, 64, 0.125, _ROT_C, 64, kv_from=1), 256, 1.5),
    _layer("attention", _attention(2, 2, 128, 128, 0.09, {"base": 1000.0, "dims": 128}, 100), 128, 3.0),
    _layer("attention", _attention(6, 3, 48, 48, 0.15, {"base": 1000.0, "dims": 24}, 40), 128, 3.0),
]}

# only one kind of layer: a model without any keys and values, and one without any state
DELTA_ONLY = {"architecture": "Sugizen", "vocab": 130, "width": 48, "norm": {"eps": 1e-5}, "layers": [
    _layer("channel_delta", _delta(2, 2, 32, 32, 4, 8, 8), 64, 1.2),
    _layer("channel_delta", _delta(6, 3, 16, 12, 3, 6, 3)),
]}
ATTENTION_ONLY = {"architecture": "Sugizen", "vocab": 210, "width": 72, "norm": {"eps": 2e-5}, "layers": [
    _layer("attention", _attention(3, 1, 24, 40, 0.2, {"base": 777.0, "dims": 24}, 33), 100, 1.0),
    _layer("attention", _attention(6, 1, 24, 40, 0.21, {"base": 777.0, "dims": 24}, 50, kv_from=0)),
    _layer("attention", _attention(2, 2, 16, 16, 0.25), 40, 9.0),
]}

CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "delta_only": DELTA_ONLY, "attention_only": ATTENTION_ONLY}
