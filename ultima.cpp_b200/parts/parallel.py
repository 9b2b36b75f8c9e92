"""Two mixers side by side."""
from __future__ import annotations

from .base import KVNeed, Mixer, PartSpec, StateNeed, build_part, register_part


@register_part("mixer", "side_by_side")
class SideBySide(Mixer):
    """left_scale * left(h) + right_scale * right(h): two mixers of any kind read the same input and add
    into the same stream.  Each applies its scale itself (its ``out_scale`` parameter, a constant on what
    goes into its output projection), so no buffer lies between them and the stream.  The tensors of the
    two stand under ``left.`` and ``right.``.  The run's cache is shared out: keys and values to the one
    that asks for them (at most one may), states in the order left, right."""

    def __init__(self, left: PartSpec, right: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0):
        self.left = build_part("mixer", PartSpec(left.kind, tuple(sorted({**left.as_dict(), "out_scale": float(left_scale)}.items()))))
        self.right = build_part("mixer", PartSpec(right.kind, tuple(sorted({**right.as_dict(), "out_scale": float(right_scale)}.items()))))
        self._needs = [self._list(self.left.cache_need()), self._list(self.right.cache_need())]
        if sum(isinstance(n, KVNeed) for ns in self._needs for n in ns) > 1:
            raise ValueError("side_by_side: at most one of the two mixers may keep keys and values")

    @staticmethod
    def _list(need):
        if need is None:
            return []
        return list(need) if isinstance(need, tuple) else [need]

    @property
    def graph_safe(self) -> bool:
        return bool(self.left.graph_safe and self.right.graph_safe)

    def weight_specs(self):
        from ..weights.spec import WeightSpec
        return [WeightSpec(side + s.name, s.shape, s.kind, s.init)
                for side, m in (("left.", self.left), ("right.", self.right)) for s in m.weight_specs()]

    def cache_need(self):
        needs = tuple(n for ns in self._needs for n in ns)
        return needs or None

    def kernel_needs(self, run_dtype):
        return list(self.left.kernel_needs(run_dtype)) + list(self.right.kernel_needs(run_dtype))

    def bind(self, tensors, rt):
        for side, m in (("left.", self.left), ("right.", self.right)):
            m.bind({n[len(side):]: t for n, t in tensors.items() if n.startswith(side)}, rt)

    def input_weight(self):
        """Both sides' input matrices stacked, if both have one."""
        import torch
        a, b = self.left.input_weight(), self.right.input_weight()
        if a is None or b is None or a.dtype != b.dtype or a.shape[1] != b.shape[1]:
            return None
        return torch.cat([a, b], dim=0)

    def adopt_input_weight(self, w):
        n = self.left.input_weight().shape[0]
        self.left.adopt_input_weight(w[:n])
        self.right.adopt_input_weight(w[n:])

    def _share(self, cache, which: int):
        """The part of the run's cache that belongs to one side."""
        if cache is None:
            return None
        before = sum(isinstance(n, StateNeed) for n in self._needs[0]) if which == 1 else 0
        mine = sum(isinstance(n, StateNeed) for n in self._needs[which])
        states = tuple(cache.states[before:before + mine])
        kv = cache.kv if any(isinstance(n, KVNeed) for n in self._needs[which]) else None
        return type(cache)(kv=kv, state=states[0] if states else None, owner=cache.owner, states=states)

    def forward(self, h, residual, batch, cache, rt, projected=None):
        mark = rt.arena.mark()
        if projected is not None:
            n = self.left.input_weight().shape[0]
            self.left.forward(h, residual, batch, self._share(cache, 0), rt, projected=projected[..., :n])
            rt.arena.reset(mark)
            self.right.forward(h, residual, batch, self._share(cache, 1), rt, projected=projected[..., n:])
        else:
            self.left.forward(h, residual, batch, self._share(cache, 0), rt)
            rt.arena.reset(mark)
            self.right.forward(h, residual, batch, self._share(cache, 1), rt)
        rt.arena.reset(mark)
