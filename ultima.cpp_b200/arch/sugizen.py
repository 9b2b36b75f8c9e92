"""Sugizen as data: layers of two kinds in the order the configuration lists them, each with the norm
on its sublayers' outputs; the tensor names of its files.

A layer is x += norm1(mixer(x)); x += norm2(feed_forward(x)) (arrangement ``norm_after``), the mixer
either the gated delta rule (part ``gated_delta``) or attention with per-head q/k norm, a rotation of
part of the head with wavelength-scaled frequencies, a mask by blocks of positions, a sigmoid gate a
head, and optionally another layer's keys and values (part ``attention`` with ``block``, ``head_gate``,
``v_head_dim``, ``own_kv``; the run list's ``cache_from``).  The feed-forward is ``gated_clamped``.
"""
from __future__ import annotations

from ..config.base import ArchitectureEntry, register_architecture
from ..config.sugizen import ATTENTION, DELTA, SugizenConfig
from ..parts.base import ModelSpec, Run, layer, part

_ROLE_NAMES = (("mixer", "mix."), ("feed_forward", "mlp."), ("mixer_norm", "norm1."), ("feed_forward_norm", "norm2."))

# part's own tensor name -> the name below the role's prefix in the files
_ATTENTION_NAMES = {"q_proj.weight": "q", "k_proj.weight": "k", "v_proj.weight": "v", "o_proj.weight": "o",
                    "q_norm.weight": "q.norm", "k_norm.weight": "k.norm", "gate_proj.weight": "g"}
_DELTA_NAMES = {"q_proj.weight": "q", "q_conv.weight": "q.conv", "k_proj.weight": "k", "k_conv.weight": "k.conv",
                "v_proj.weight": "v", "v_conv.weight": "v.conv", "b_proj.weight": "b", "a_log": "A_log",
                "o_norm.weight": "norm", "decay_down.weight": "a1", "decay_up.weight": "a2", "dt_bias": "dt_bias",
                "gate_down.weight": "g1", "gate_up.weight": "g2", "o_proj.weight": "o"}
_DENSE_NAMES = {"gate_proj.weight": "gate", "up_proj.weight": "up", "down_proj.weight": "down"}


def build_spec(cfg: SugizenConfig, max_positions: int | None = None) -> ModelSpec:
    if cfg.needs_tensor_shapes:
        raise ValueError("Sugizen: the delta layers' low-rank sizes are not known; read the configuration with "
                         "config_from_dir (which takes them from the tensors' shapes) or give decay_rank and gate_rank")
    max_pos = int(max_positions or cfg.max_position_embeddings)
    norm = part("rms", width=cfg.width, eps=cfg.eps)
    layers, runs, renames = [], [], [("embed.weight", "embed"), ("final.norm.weight", "final.norm"), ("head.weight", "head")]
    for i, L in enumerate(cfg.layers):
        m, pre = L.mixer, f"l{i}."
        if m.kind == DELTA:
            mixer = part("gated_delta", width=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         v_head_dim=m.vdim, conv=m.conv, decay_rank=m.decay_rank, gate_rank=m.gate_rank, eps=cfg.eps)
            names = _DELTA_NAMES
        elif m.kind == ATTENTION:
            position = None
            if m.rot is not None:
                position = part("rotary_half_split", head_dim=m.dim, theta=m.rot.base, max_positions=max_pos,
                                rotary_dim=m.rot.dims, wavelength_scaling=m.rot.scaling)
            mixer = part("attention", width=cfg.width, n_heads=m.heads, n_kv_heads=m.kv_heads, head_dim=m.dim,
                         qk_norm=True, eps=cfg.eps, position=position, window=None, scale=m.scale,
                         v_head_dim=m.vdim, block=m.block, head_gate=True, own_kv=m.kv_from is None)
            names = _ATTENTION_NAMES
        else:
            raise ValueError(f"Sugizen: unknown layer type {m.kind!r}")
        renames += [(f"{pre}mix.{a}", f"{pre}mix.{b}") for a, b in names.items()]
        renames.append((f"{pre}norm1.weight", f"{pre}norm1"))
        if L.mlp is not None:
            ffn = part("gated_clamped", width=cfg.width, inner=L.mlp.ff, limit=L.mlp.limit, alpha=1.702, shift=1.0)
            layers.append(layer(part("norm_after"), prefix=pre, names=_ROLE_NAMES, mixer=mixer, mixer_norm=norm,
                                feed_forward=ffn, feed_forward_norm=norm))
            renames += [(f"{pre}mlp.{a}", f"{pre}mlp.{b}") for a, b in _DENSE_NAMES.items()]
            renames.append((f"{pre}norm2.weight", f"{pre}norm2"))
        else:
            layers.append(layer(part("norm_after_mixer_only"), prefix=pre, names=_ROLE_NAMES[:1] + _ROLE_NAMES[2:3],
                                mixer=mixer, mixer_norm=norm))
        runs.append(Run(i, cache_from=m.kv_from))
    return ModelSpec(
        width=cfg.width, vocab_size=cfg.vocab, max_positions=max_pos,
        embedding=part("token_table", vocab_size=cfg.vocab, width=cfg.width), embedding_name="embed.",
        layers=tuple(layers), runs=tuple(runs), final_norm=norm, final_norm_name="final.norm.",
        head=part("linear", vocab_size=cfg.vocab, width=cfg.width, tied=False), head_name="head.",
        stop_token_ids=tuple(cfg.eos_token_id), renames=tuple(renames))


register_architecture(ArchitectureEntry(
    name="Sugizen", model_type="sugizen", supported=True,
    notes="Sugizen: gated delta-rule and block-masked gated attention layers, norm on the sublayers' outputs",
    config_cls=SugizenConfig, build_spec=build_spec))
