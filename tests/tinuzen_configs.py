"""Small Tinuzen configurations for the tests.  They differ from one another in every size and option: order
of layers, widths (one not a multiple of 8), heads and groups, key and value sizes (equal and not), windows
with and without kept first positions (fewer than a page, more than a page, none at all), rotation of part or
all of a head or none, state sizes that are and are not multiples of 8, taps from 1 to 5, parts of the
state-space norm, scales, a repeated group at the start, in the middle, over all layers or absent, one pass
only, layers without feed-forward, hash constants (one bucket; a multiplier of zero)."""


def _attention(heads, kv_heads, dim, vdim, scale, size=None, keep_first=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if size is not None:
        m["mask"] = {"size": size}
        if keep_first is not None:
            m["mask"]["keep_first"] = keep_first
    return m


def _parallel(left, right, left_scale, right_scale):
    return {"left": left, "right": right, "left_scale": left_scale, "right_scale": right_scale}


def _left(heads, kv_heads, dim, scale, rot=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot is not None:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return m


def _right(heads, vdim, state, groups, conv, norm_groups):
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv, "norm_groups": norm_groups}


def _layer(kind, mixer, ff=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def _emb(scale, buckets, mul_prev, mul_cur):
    return {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mul_prev, "mul_cur": mul_cur}}


MIXED = {"architecture": "Tinuzen", "vocab": 300, "width": 64, "norm": {"eps": 1e-5}, "embedding": _emb(4.0, 97, 5, 3),
         "loop": {"start": 1, "stop": 3, "times": 2}, "layers": [
    _layer("attention", _attention(4, 2, 32, 16, 0.2, 24, 3), 96),
    _layer("parallel", _parallel(_left(4, 2, 32, 0.18, (10000.0, 16)), _right(4, 16, 16, 2, 3, 2), 0.7, 1.3), 80),
    _layer("attention", _attention(6, 2, 16, 24, 0.25, 10, 0)),
    _layer("parallel", _parallel(_left(2, 1, 24, 0.2), _right(6, 8, 12, 3, 2, 3), 1.5, 0.5)),
]}

ODD = {"architecture": "Tinuzen", "vocab": 257, "width": 100, "norm": {"eps": 3e-6}, "embedding": _emb(1.0, 1, 7, 11), "layers": [
    _layer("parallel", _parallel(_left(3, 1, 28, 0.19, (300.0, 28)), _right(3, 10, 5, 3, 1, 1), 1.0, 1.0), 131),
    _layer("attention", _attention(3, 3, 20, 12, 0.22), 60),
    _layer("attention", _attention(5, 1, 12, 20, 0.3, 7, 2), 60),
    _layer("parallel", _parallel(_left(5, 5, 20, 0.22, (50.0, 6)), _right(2, 33, 20, 1, 5, 2), 0.9, 1.1), 64),
]}

WIDE = {"architecture": "Tinuzen", "vocab": 384, "width": 128, "norm": {"eps": 1e-6}, "embedding": _emb(8.0, 1000, 0, 13),
        "loop": {"start": 0, "stop": 3, "times": 3}, "layers": [
    _layer("attention", _attention(4, 1, 64, 64, 0.125, 100, 70), 256),
    _layer("parallel", _parallel(_left(4, 2, 64, 0.125, (50000.0, 64)), _right(4, 32, 64, 2, 4, 1), 1.2, 0.8), 256),
    _layer("parallel", _parallel(_left(2, 2, 128, 0.09, (1000.0, 64)), _right(2, 64, 128, 1, 4, 4), 1.0, 1.0), 128),
]}

ONE_PASS = {"architecture": "Tinuzen", "vocab": 130, "width": 48, "norm": {"eps": 1e-5}, "embedding": _emb(2.0, 31, 3, 0),
            "loop": {"start": 1, "stop": 2, "times": 1}, "layers": [
    _layer("parallel", _parallel(_left(2, 2, 16, 0.25, (100.0, 8)), _right(3, 16, 8, 1, 4, 3), 1.1, 0.9), 64),
    _layer("attention", _attention(2, 2, 24, 24, 0.2, 64, 1), 40),
]}

CONFIGS = {"mixed": MIXED, "odd": ODD, "wide": WIDE, "one_pass": ONE_PASS}
