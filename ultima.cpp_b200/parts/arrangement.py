"""How a layer's parts are arranged around the residual stream."""
from __future__ import annotations

from ..kernels import ops
from .base import Arrangement, register_part


@register_part("arrangement", "pre_norm")
class PreNorm(Arrangement):
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x in float32
    (reference: src/model/qwen_block.cpp:621-628, :782-792, :811-812)."""

    roles = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm",
             "feed_forward": "feed_forward"}

    def __init__(self):
        pass

    def run(self, layer, x, batch, cache, rt):
        mark = rt.arena.mark()
        h = layer.mixer_norm.forward(x, rt)
        layer.mixer.forward(h, x, batch, cache, rt)
        rt.arena.reset(mark)
        h = layer.feed_forward_norm.forward(x, rt)
        layer.feed_forward.forward(h, x, batch, rt)
        rt.arena.reset(mark)


class _NormAfter(Arrangement):
    """x += norm(mixer(x)); x += norm(feed_forward(x)): the sublayers read the residual stream itself
    and the norm stands on what they put out.  A sublayer adds its output into the stream it is handed;
    here that is a cleared float32 buffer y, which the norm then folds into x.  The same kernel writes
    the next sublayer's input (x in the activation type) and clears y again, and both buffers are kept
    from layer to layer of a pass, so a layer costs no conversion or clearing kernel of its own after
    the first."""

    def _buffers(self, x, rt):
        carry = getattr(rt, "_norm_after_carry", None)
        if carry is not None and carry[0] == (rt.pass_id, x.data_ptr(), tuple(x.shape)):
            return carry[1], carry[2]
        y = rt.arena.alloc(tuple(x.shape), x.dtype)
        y.zero_()
        if rt.dtype == x.dtype:
            h = x                                   # 32-bit run: the sublayers read x in place
        else:
            h = rt.arena.alloc(tuple(x.shape), rt.dtype)
            rt.launches += 1
            ops.convert(x, h)
        rt._norm_after_carry = ((rt.pass_id, x.data_ptr(), tuple(x.shape)), h, y)
        return h, y

    def run(self, layer, x, batch, cache, rt):
        h, y = self._buffers(x, rt)
        hn = None if h is x else h
        mark = rt.arena.mark()
        layer.mixer.forward(h, y, batch, cache, rt)
        layer.mixer_norm.add_normed(y, x, rt, h=hn, clear=True)
        rt.arena.reset(mark)
        ff = getattr(layer, "feed_forward", None)
        if ff is not None:
            ff.forward(h, y, batch, rt)
            layer.feed_forward_norm.add_normed(y, x, rt, h=hn, clear=True)
            rt.arena.reset(mark)


@register_part("arrangement", "norm_after")
class NormAfter(_NormAfter):
    roles = {"mixer": "mixer", "mixer_norm": "norm", "feed_forward": "feed_forward", "feed_forward_norm": "norm"}

    def __init__(self):
        pass


@register_part("arrangement", "norm_after_mixer_only")
class NormAfterMixerOnly(_NormAfter):
    """The same layer without a feed-forward."""
    roles = {"mixer": "mixer", "mixer_norm": "norm"}

    def __init__(self):
        pass
