"""Tinuzen as data: layers of two kinds in the order the configuration lists them, a group of them run
several times with a cache of its own each time; the tensor names of its files.

A layer is h = norm1(x); x += gate1(h) * mixer(h) + gate2(h) * feed_forward(h) (arrangement
``parallel_gated``, gates ``sigmoid_linear``).  The mixer is either attention with a q/k norm over all heads
at once, a bias by distance and a window that keeps the sequence's first positions (part ``attention`` with
``norm_whole``, ``distance_slope``, ``window``, ``keep_first``), or two mixers side by side (part
``side_by_side``): attention whose values are its keys, with neighbouring columns rotated, a softmax with a
sink and a gate an output element (``values_are_keys``, ``sink``, ``wide_gate``), and a state-space mixer
(part ``state_space_dual``).  The feed-forward is ``gated_relu``.  The embedding adds a hashed table of token
pairs (``token_table_hashed_pairs``); a pass of the repeated group opens with a ``pass_marker``.
"""
from __future__ import annotations

from ..config.base import ArchitectureEntry, register_architecture
from ..config.tinuzen import ATTENTION, PARALLEL, TinuzenConfig
from ..parts.base import ModelSpec, Run, layer, part

DISTANCE_SLOPE = 8.0          # head h of H takes 2^(-8 (h + 1) / H) a position of distance off its scores

_ROLE_NAMES = (("norm", "norm1."), ("mixer", "mix."), ("mixer_gate", "rg1."), ("feed_forward", "mlp."),
               ("feed_forward_gate", "rg2."))
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm"}
_LEFT_NAMES = {"left.q_proj.weight": "left.q", "left.k_proj.weight": "left.k", "left.gate_proj.weight": "left.g",
               "left.o_proj.weight": "left.o"}
_RIGHT_NAMES = {"right.in_proj.weight": "right.in", "right.conv.weight": "right.conv", "right.conv.bias": "right.conv.b",
                "right.dt_bias": "right.dt_bias", "right.a_log": "right.A_log", "right.d_skip": "right.D",
                "right.o_norm.weight": "right.norm", "right.o_proj.weight": "right.o"}
_DENSE_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def run_order(n_layers: int, loop) -> list:
    """[(layer, number of the pass this run opens or None), ...]"""
    if loop is None:
        return [(i, None) for i in range(n_layers)]
    start, stop, times = loop
    order = [(i, None) for i in range(start)]
    for t in range(times):
        order += [(i, t if i == start else None) for i in range(start, stop)]
    return order + [(i, None) for i in range(stop, n_layers)]


def build_spec(cfg: TinuzenConfig, max_positions: int | None = None) -> ModelSpec:
    max_pos = int(max_positions or cfg.max_position_embeddings)
    norm = part("rms", width=cfg.width, eps=cfg.eps)
    gate = part("sigmoid_linear", width=cfg.width, bias=True)
    layers = []
    renames = [("embed.weight", "embed"), ("embed.pairs", "bigram"), ("final.norm.weight", "final.norm"),
               ("head.weight", "head")]
    for i, L in enumerate(cfg.layers):
        m, pre = L.mixer, f"l{i}."
        if L.kind == ATTENTION:
            mixer = part("attention", width=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim, qk_norm=True,
                         eps=cfg.eps, position=None, window=m.window, scale=m.scale, v_head_dim=m.vdim, norm_whole=True,
                         keep_first=m.keep_first if m.window is not None else 0, distance_slope=DISTANCE_SLOPE)
            names = _ATTENTION_NAMES
        elif L.kind == PARALLEL:
            a, r = m.left, m.right
            position = None
            if a.rot_dims is not None:
                position = part("rotary_interleaved", head_dim=a.dim, theta=a.rot_base, max_positions=max_pos,
                                rotary_dim=a.rot_dims)
            left = part("attention", width=cfg.width, n_heads=a.heads, n_kv_heads=a.kv_heads, head_dim=a.dim, qk_norm=False,
                        eps=cfg.eps, position=position, window=None, scale=a.scale, values_are_keys=True, sink=True,
                        wide_gate=True)
            right = part("state_space_dual", width=cfg.width, n_heads=r.heads, head_dim=r.vdim, state=r.state,
                         n_groups=r.groups, conv=r.conv, norm_groups=r.norm_groups, eps=cfg.eps)
            mixer = part("side_by_side", left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
            names = {**_LEFT_NAMES, **_RIGHT_NAMES}
        else:
            raise ValueError(f"Tinuzen: unknown layer type {L.kind!r}")
        renames += [(f"{pre}mix.{a}", f"{pre}mix.{b}") for a, b in names.items()]
        renames += [(f"{pre}norm1.weight", f"{pre}norm1"), (f"{pre}rg1.weight", f"{pre}rg1"), (f"{pre}rg1.bias", f"{pre}rg1.b")]
        if L.ff is not None:
            layers.append(layer(part("parallel_gated"), prefix=pre, names=_ROLE_NAMES, norm=norm, mixer=mixer, mixer_gate=gate,
                                feed_forward=part("gated_relu", width=cfg.width, inner=L.ff), feed_forward_gate=gate))
            renames += [(f"{pre}mlp.{a}", f"{pre}mlp.{b}") for a, b in _DENSE_NAMES.items()]
            renames += [(f"{pre}rg2.weight", f"{pre}rg2"), (f"{pre}rg2.bias", f"{pre}rg2.b")]
        else:
            layers.append(layer(part("parallel_gated_mixer_only"), prefix=pre, names=_ROLE_NAMES[:3], norm=norm, mixer=mixer,
                                mixer_gate=gate))
    entries, runs = [], []
    for i, opens in run_order(len(cfg.layers), cfg.loop):
        entry = None
        if opens is not None:
            entry = len(entries)
            entries.append((part("pass_marker", width=cfg.width, times=cfg.loop[2], index=opens), "loop."))
        runs.append(Run(i, entry=entry))
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=part("token_table_hashed_pairs", vocab_size=cfg.vocab, width=cfg.width, scale=cfg.embed_scale,
                       buckets=cfg.buckets, mul_prev=cfg.mul_prev, mul_cur=cfg.mul_cur), embedding_name="embed.",
        layers=tuple(layers), runs=tuple(runs), final_norm=norm, final_norm_name="final.norm.",
        head=part("linear", vocab_size=cfg.vocab, width=cfg.width, tied=False), head_name="head.",
        stop_token_ids=tuple(cfg.eos_token_id), renames=tuple(renames), entries=tuple(entries))


register_architecture(ArchitectureEntry(
    name="Tinuzen", model_type="tinuzen", supported=True,
    notes="Tinuzen: gated parallel layers of windowed attention or attention beside a state-space mixer, a group of layers "
          "run several times, a hashed table of token pairs in the embedding",
    config_cls=TinuzenConfig, build_spec=build_spec))
