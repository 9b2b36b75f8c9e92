"""Tinuzen on the GPU against the plain implementation (tests/plain_tinuzen.py): each mechanism's kernels
alone, then whole models from small configurations with random weights: prompts, token-by-token decoding,
portions, batches of unequal requests, slots used again, long decoding, greedy generation, trace replay."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, close_enough, has_gpu
from tinuzen_configs import CONFIGS

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not has_gpu(), reason="needs a CUDA device")]
DEV = "cuda:0"


def _ops():
    from ultima_b200.kernels import ops
    return ops


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max() / max(1e-30, float(ref.abs().max())))


class _Seqs:
    """The few fields of a step's batch that the kernels read."""

    def __init__(self, starts, slots, ids=None):
        self.seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.n_seqs = len(slots)
        seq = []
        for i in range(len(slots)):
            seq += [i] * (starts[i + 1] - starts[i])
        self.tok_seq = torch.tensor(seq, dtype=torch.int32, device=DEV)
        self.max_new = max(b - a for a, b in zip(starts[:-1], starts[1:]))
        if ids is not None:
            self.tok_ids = torch.tensor(ids, dtype=torch.int32, device=DEV)


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("sizes", [(50, 24, 7, 3, 5, 2.5), (300, 100, 1, 11, 0, 1.0), (64, 2048, 1000, 0, 13, 16.0)])
def test_embedding_with_the_hashed_table_of_pairs_and_its_state(sizes, dtype):
    import plain_tinuzen as P
    ops = _ops()
    vocab, width, buckets, mp, mc, scale = sizes
    g = torch.Generator().manual_seed(vocab)
    table = torch.randn(vocab, width, generator=g).to(dtype)
    pairs = torch.randn(buckets + 1, width, generator=g).to(dtype)
    e = {"scale": scale, "bigram": {"buckets": buckets, "mul_prev": mp, "mul_cur": mc}}
    W = {"embed": table.double(), "bigram": pairs.double()}
    a = torch.randint(0, vocab, (23,), generator=g).tolist()
    b = torch.randint(0, vocab, (9,), generator=g).tolist()
    ref_a, ref_b = P.embedding(a, W, e), P.embedding(b, W, e)
    last = torch.zeros(4, dtype=torch.int32, device=DEV)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    tol = 1e-6 if dtype == torch.float32 else 1e-6          # the sum itself is float32 either way

    def run(parts, slots):
        """parts: for each sequence its tokens of this step."""
        ids = [t for p in parts for t in p]
        starts = np.concatenate([[0], np.cumsum([len(p) for p in parts])]).tolist()
        out = torch.empty(len(ids), width, device=DEV)
        ops.embed_pairs(table.to(DEV), pairs.to(DEV), torch.tensor(ids, dtype=torch.int32, device=DEV),
                        _Seqs(starts, slots), last, out, status, scale, buckets, mp, mc)
        return out
    # two sequences of unequal length together, then cut in portions, then token by token; slots 2 and 0
    o = run([a[:10], b[:1]], [2, 0])
    assert rel_err(o[:10], ref_a[:10]) < tol and rel_err(o[10:], ref_b[:1]) < tol
    assert last.tolist() == [b[0] + 1, 0, a[9] + 1, 0]
    o = run([a[10:12], b[1:8]], [2, 0])
    assert rel_err(o[:2], ref_a[10:12]) < tol and rel_err(o[2:], ref_b[1:8]) < tol
    for t in range(12, 23):
        o = run([[a[t]]] + ([[b[8]]] if t == 12 else []), [2, 0][:2 if t == 12 else 1])
        assert rel_err(o[:1], ref_a[t:t + 1]) < tol
        if t == 12:
            assert rel_err(o[1:], ref_b[8:9]) < tol
    # a slot that is used again starts from "no token before": the cache zeroes the state on acquire
    last[2] = 0
    o = run([a[:3]], [2])
    assert rel_err(o, ref_a[:3]) < tol and int(status.item()) == 0


def test_gated_join_pass_marker_and_gate_an_element():
    ops = _ops()
    g = torch.Generator().manual_seed(4)
    for T, width in ((5, 64), (3, 100), (7, 30)):
        x, y = torch.randn(T, width, generator=g), torch.randn(T, width, generator=g)
        parts, b = torch.randn(3, T, width, generator=g), torch.randn(width, generator=g)
        ref = x.double() + torch.sigmoid(parts.double().sum(0) + b.double()) * y.double()
        xd, yd = x.to(DEV), y.to(DEV)
        ops.gated_add(parts.to(DEV), b.to(DEV), yd, xd, clear_y=True)
        assert rel_err(xd, ref) < 1e-6 and float(yd.abs().max()) == 0.0
        xd, yd = x.to(DEV), y.to(DEV)
        ops.gated_add(parts[0].contiguous().to(DEV), None, yd, xd)
        assert rel_err(xd, x.double() + torch.sigmoid(parts[0].double()) * y.double()) < 1e-6 and torch.equal(yd.cpu(), y)
        xd = x.to(DEV)
        ops.add_rows(xd, y.to(DEV), b.to(DEV))
        assert rel_err(xd, x.double() + y.double() + b.double()) < 1e-6
        xd = x.to(DEV)
        ops.add_rows(xd, None, b.to(DEV))
        assert rel_err(xd, x.double() + b.double()) < 1e-6
        for dt in (torch.float32, torch.bfloat16):
            o = x.to(dt).to(DEV)
            wide = torch.randn(T, width + 8, generator=g).to(DEV)
            ops.elem_gate(o, wide[:, 3:3 + width], 1.7)
            ref = x.to(dt).double() * 1.7 * torch.sigmoid(wide[:, 3:3 + width].double().cpu())
            assert rel_err(o, ref) < (1e-6 if dt == torch.float32 else 2 ** -7)


@pytest.mark.parametrize("T", [5, 300])
def test_rectified_gate_product_on_both_paths(T):
    from ultima_b200.engine.runtime import Runtime
    from ultima_b200.parts.mlp import GatedReLU
    g = torch.Generator().manual_seed(T)
    for dtype, width, F in ((torch.float32, 40, 37), (torch.bfloat16, 128, 192), (torch.bfloat16, 100, 50)):
        rt = Runtime(DEV, dtype)
        ff = GatedReLU(width, F)
        w = {n: (torch.randn(*s, generator=g) * 0.2).to(dtype) for n, s in
             (("gate_proj.weight", (F, width)), ("up_proj.weight", (F, width)), ("down_proj.weight", (width, F)))}
        ff.bind({n: t.to(DEV) for n, t in w.items()}, rt)
        h = torch.randn(T, width, generator=g).to(dtype)
        h[0] = 0                                         # a gate of exactly zero
        res = torch.zeros(T, width, device=DEV)
        ff.forward(h.to(DEV), res, None, rt)
        rt.check_status()
        hd, wd = h.double(), {n: t.double() for n, t in w.items()}
        inner = torch.relu(hd @ wd["gate_proj.weight"].T) * (hd @ wd["up_proj.weight"].T)
        if dtype == torch.bfloat16:
            inner = inner.to(torch.bfloat16).double()
        ref = inner @ wd["down_proj.weight"].T
        assert torch.isfinite(res).all() and rel_err(res, ref) < (1e-5 if dtype == torch.float32 else 2 ** -6), (dtype, width)


def _paged(k, v, ring_pages, seed):
    """k [n, nkv, hd], v [n, nkv, hdv] into shuffled pages of 64 positions."""
    n, nkv, hd = k.shape
    perm = torch.randperm(ring_pages + 2, generator=torch.Generator().manual_seed(seed))[:ring_pages]
    kc = torch.full((ring_pages + 2, nkv, 64, hd), float("nan"), dtype=k.dtype)
    vc = torch.full((ring_pages + 2, nkv, 64, v.shape[2]), float("nan"), dtype=v.dtype)
    for p in range(n):
        kc[perm[p // 64], :, p % 64], vc[perm[p // 64], :, p % 64] = k[p], v[p]
    return kc.to(DEV), vc.to(DEV), perm.to(torch.int32).view(1, -1).to(DEV)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48, rd=48, whole=True), dict(nh=2, nkv=2, hd=16, rd=0, whole=True),
                                 dict(nh=4, nkv=1, hd=96, rd=32, whole=False), dict(nh=3, nkv=3, hd=20, rd=6, whole=True),
                                 dict(nh=32, nkv=8, hd=128, rd=128, whole=True)])
def test_placement_by_rows_norm_over_all_heads_neighbour_rotation_values_from_keys(cfg, dtype):
    """q and k normed over the whole projection (or not at all), neighbouring columns rotated, the values taken from
    the key columns as they are, a wide gate copied out; from one piece and from K slices."""
    import plain_tinuzen as P
    ops = _ops()
    nh, nkv, hd, rd, whole = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["rd"], cfg["whole"]
    T, eps = 70, 1e-5
    g = torch.Generator().manual_seed(hd + nh)
    qw, kw, gw = nh * hd, nkv * hd, nh * hd
    x = torch.randn(2, T, qw + kw + gw + 3, generator=g)
    row = x.double().sum(0)
    wq, wk = 1 + 0.1 * torch.randn(qw, generator=g), 1 + 0.1 * torch.randn(kw, generator=g)
    pos = torch.arange(3, 3 + T)
    q_ref, k_ref = row[:, :qw], row[:, qw:qw + kw]
    v_ref = k_ref.clone()
    if whole:
        q_ref, k_ref = P.rms_norm(q_ref, wq.double(), eps), P.rms_norm(k_ref, wk.double(), eps)
    q_ref, k_ref = q_ref.view(T, nh, hd), k_ref.view(T, nkv, hd)
    cos = sin = None
    if rd:
        rot = {"base": 100.0, "dims": rd}
        q_ref, k_ref = P.rotate_neighbours(q_ref, pos, rot), P.rotate_neighbours(k_ref, pos, rot)
        f = 100.0 ** (-2.0 * torch.arange(rd // 2, dtype=torch.float64) / rd)
        ang = torch.arange(128, dtype=torch.float64)[:, None] * f[None]
        cos, sin = torch.cos(ang).float().to(DEV), torch.sin(ang).float().to(DEV)
    kc = torch.zeros(4, nkv, 64, hd, dtype=dtype, device=DEV)
    vc = torch.zeros(4, nkv, 64, hd, dtype=dtype, device=DEV)
    table = torch.tensor([[2, 0, 3]], dtype=torch.int32, device=DEV)
    q = torch.empty(T, qw, dtype=dtype, device=DEV)
    gate = torch.empty(T, gw, device=DEV)
    ops.qkv_place_rows(x.to(DEV), 0, qw, qw, q, wq.to(DEV) if whole else None, wk.to(DEV) if whole else None, whole, cos, sin,
                       rd, True, pos.to(torch.int32).to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), kc, vc, table,
                       192, 64, nh, nkv, hd, hd, eps, qw + kw, gate)
    tol = 2e-6 if dtype == torch.float32 else 2 ** -7
    assert rel_err(q.view(T, nh, hd), q_ref) < tol
    assert rel_err(gate, row[:, qw + kw:qw + kw + gw]) < 1e-6
    pages = [2, 0, 3]
    for t in (0, 1, 60, 61, 69):
        p = int(pos[t])
        assert rel_err(kc[pages[p // 64], :, p % 64], k_ref[t]) < tol, t
        assert rel_err(vc[pages[p // 64], :, p % 64], v_ref[t].view(nkv, hd)) < tol, t


def _plain_attention(q, k, v, p, nh, nkv, scale, window, keep, slopes, sink):
    """One query (all heads) at position p over keys 0 .. p: float64."""
    out = []
    for h in range(nh):
        kv = h // (nh // nkv)
        j = torch.arange(p + 1)
        s = (k[:p + 1, kv].double() @ q.double().view(nh, -1)[h]) * scale
        if slopes is not None:
            s = s - slopes[h].double() * (p - j).double()
        if window:
            s = s.masked_fill(~((p - j < window) | (j < keep)), float("-inf"))
        if sink:
            m = max(float(s.max()), 0.0)
            e = torch.exp(s - m)
            w = e / (e.sum() + np.exp(-m))
        else:
            w = torch.softmax(s, 0)
        out.append(w @ v[:p + 1, kv].double())
    return torch.stack(out)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48, hdv=16, window=50, keep=3, slope=8.0, sink=False),
                                 dict(nh=2, nkv=2, hd=16, hdv=16, window=0, keep=0, slope=None, sink=True),
                                 dict(nh=4, nkv=1, hd=64, hdv=64, window=64, keep=70, slope=8.0, sink=False),
                                 dict(nh=3, nkv=3, hd=20, hdv=24, window=7, keep=0, slope=2.0, sink=True),
                                 dict(nh=4, nkv=2, hd=128, hdv=128, window=0, keep=0, slope=None, sink=True)])
def test_attention_with_window_kept_first_positions_distance_bias_sink_and_wide_gate(cfg, dtype):
    ops = _ops()
    nh, nkv, hd, hdv = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["hdv"]
    n = 300
    g = torch.Generator().manual_seed(hd)
    k = torch.randn(n, nkv, hd, generator=g).to(dtype)
    v = torch.randn(n, nkv, hdv, generator=g).to(dtype)
    kc, vc, table = _paged(k, v, 5, seed=1)
    places = sorted({0, 1, 2, 3, 6, 7, 49, 50, 52, 53, 63, 64, 65, 69, 70, 71, 99, 127, 128, 133, 134, 199, 255, 256, 299})
    q = torch.randn(len(places), nh * hd, generator=g).to(dtype).to(DEV)
    gate = torch.randn(len(places), nh * hdv + 3, generator=g).to(DEV)[:, 1:1 + nh * hdv]
    slopes = None
    if cfg["slope"] is not None:
        slopes = (2.0 ** (-cfg["slope"] * torch.arange(1, nh + 1, dtype=torch.float64) / nh)).float().to(DEV)
    out = torch.empty(len(places), nh * hdv, dtype=dtype, device=DEV)
    pos = torch.tensor(places, dtype=torch.int32, device=DEV)
    seq = torch.zeros(len(places), dtype=torch.int32, device=DEV)
    ops.attn_simple(q, kc, vc, out, pos, seq, table, 5 * 64, 64, nh, nkv, hd, cfg["window"], 0.3, v_head_dim=hdv, gate=gate,
                    keep_first=cfg["keep"], slopes=slopes, sink=cfg["sink"], out_scale=1.3)
    for i, p in enumerate(places):
        ref = _plain_attention(q[i].cpu(), k, v, p, nh, nkv, 0.3, cfg["window"], cfg["keep"],
                               slopes.cpu() if slopes is not None else None, cfg["sink"])
        ref = ref * 1.3 * torch.sigmoid(gate[i].double().cpu()).view(nh, hdv)
        err = rel_err(out[i].view(nh, hdv), ref)
        assert err <= (2e-5 if dtype == torch.float32 else 2 ** -6), (p, err)


def test_keys_at_the_edges_of_the_window_and_of_the_kept_positions_and_far_away():
    """One key is made to stand out (a score far above all others) and carries a value no other has: a query sees
    it exactly when the mask says so.  Window 96 with 4 kept positions, and window 64 with 70 kept ones (edges on
    and off a page's border); queries in a prompt portion and alone."""
    ops = _ops()
    nh = nkv = 1
    hd = 32
    for window, keep in ((96, 4), (64, 70), (10, 0)):
        n = 400
        g = torch.Generator().manual_seed(window)
        for marked in (0, keep - 1, keep, 63, 64, 200):
            if marked < 0:
                continue
            k = torch.randn(n, nkv, hd, generator=g) * 0.1
            v = torch.randn(n, nkv, hd, generator=g) * 0.1
            q = torch.randn(1, hd, generator=g)
            k[marked, 0] = q[0] * 4                              # score ~ 4 |q|^2 * scale against ~0.1 |q|
            v[marked, 0] = 50.0
            kc, vc, table = _paged(k, v, 7, seed=2)
            places = [p for p in (marked, marked + 1, marked + window - 1, marked + window, marked + window + 1, 399) if marked <= p < n]
            pos = torch.tensor(places, dtype=torch.int32, device=DEV)
            out = torch.empty(len(places), hd, device=DEV)
            ops.attn_simple(q.repeat(len(places), 1).to(DEV), kc, vc, out, pos, torch.zeros(len(places), dtype=torch.int32, device=DEV),
                            table, 7 * 64, 64, nh, nkv, hd, window, 1.0, keep_first=keep)
            for i, p in enumerate(places):
                seen = (p - marked < window) or marked < keep
                assert (float(out[i].mean()) > 45.0) == seen, (window, keep, marked, p, float(out[i].mean()))


class _KV:
    def __init__(self, k, v, table, ring, window):
        self.k, self.v, self.table, self.ring, self.page, self.window = k, v, table, ring, 64, window


class _B:
    pass


@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48, window=50, keep=3, slope=8.0, sink=False, gate=False),
                                 dict(nh=4, nkv=2, hd=64, window=0, keep=0, slope=None, sink=True, gate=True),
                                 dict(nh=4, nkv=1, hd=64, window=64, keep=70, slope=8.0, sink=False, gate=False),
                                 dict(nh=3, nkv=3, hd=16, window=7, keep=0, slope=2.0, sink=True, gate=True),
                                 dict(nh=16, nkv=1, hd=128, window=0, keep=0, slope=None, sink=True, gate=True),
                                 dict(nh=2, nkv=2, hd=32, window=96, keep=4, slope=8.0, sink=False, gate=False)])
def test_tensor_core_attention_with_the_further_options_prompts_and_single_tokens(cfg):
    """The mma.sync kernels against the float64 restatement: whole prompts of unequal lengths, continued prompts,
    and one token a sequence with the key range in one slice and in several."""
    from ultima_b200.engine import Runtime
    from ultima_b200.kernels import attn_tc
    nh, nkv, hd = cfg["nh"], cfg["nkv"], cfg["hd"]
    rt = Runtime(DEV, torch.bfloat16)
    slopes = sl2 = None
    if cfg["slope"] is not None:
        sl = 2.0 ** (-cfg["slope"] * torch.arange(1, nh + 1, dtype=torch.float64) / nh)
        slopes, sl2 = sl.float(), (sl * np.log2(np.e)).float().to(DEV)
    # (head sizes 64 and 128 without window and bias: the prompts run on the tcgen05 kernels, 128 rows a CTA; the
    # last case, a long prompt, on the one with 256 rows)
    cases = [([0, 0, 0, 0], [1, 17, 64, 200], None, 0), ([5, 64, 130, 0], [70, 1, 33, 129], None, 0),
             ([299, 0, 63, 130], [1, 1, 1, 1], 1, 0), ([299, 150, 64, 7], [1, 1, 1, 1], 4, 0)]
    if hd in (64, 128) and not cfg["window"] and cfg["slope"] is None:
        cases += [([0, 20], [320, 300], None, 2), ([5, 64, 130, 0], [70, 1, 33, 129], None, 2)]      # 256 rows a CTA
    for befores, news, slices, wide in cases:
        attn_tc.set_wide(wide)
        lens = [b + n for b, n in zip(befores, news)]
        g = torch.Generator().manual_seed(hd + len(lens) + befores[0])
        pages = 5
        perm = torch.randperm(len(lens) * pages + 3, generator=g)
        kc = torch.full((len(lens) * pages + 3, nkv, 64, hd), float("nan"), dtype=torch.bfloat16)
        vc = kc.clone()
        table = perm[:len(lens) * pages].view(len(lens), pages).to(torch.int32)
        dense = []
        for s_, n in enumerate(lens):
            k = torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16)
            v = torch.randn(n, nkv, hd, generator=g).to(torch.bfloat16)
            dense.append((k, v))
            for p_ in range(n):
                kc[table[s_, p_ // 64], :, p_ % 64], vc[table[s_, p_ // 64], :, p_ % 64] = k[p_], v[p_]
        T = sum(news)
        q = torch.randn(T, nh * hd, generator=g).to(torch.bfloat16).to(DEV)
        gate = torch.randn(T, nh * hd, generator=g).to(DEV) if cfg["gate"] else None
        out = torch.full((T, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
        b = _B()
        start = [0]
        for n in news:
            start.append(start[-1] + n)
        b.seq_start = torch.tensor(start, dtype=torch.int32, device=DEV)
        b.seq_before = torch.tensor(befores, dtype=torch.int32, device=DEV)
        b.n_seqs, b.max_new, b.max_after = len(lens), max(news), max(lens)
        kv = _KV(kc.to(DEV), vc.to(DEV), table.to(DEV), pages * 64, None)
        attn_tc.attention_ext(q, kv, out, b, nh, nkv, hd, 0.3, rt, window=cfg["window"] or None, keep_first=cfg["keep"],
                              sink=cfg["sink"], slopes_log2=sl2, out_scale=1.3, gate=gate, slices=slices)
        torch.cuda.synchronize()
        for s_, (bf, n) in enumerate(zip(befores, news)):
            k, v = dense[s_]
            for t in range(n):
                row = start[s_] + t
                ref = _plain_attention(q[row].cpu(), k, v, bf + t, nh, nkv, 0.3, cfg["window"], cfg["keep"], slopes, cfg["sink"]) * 1.3
                if gate is not None:
                    ref = ref * torch.sigmoid(gate[row].double().cpu()).view(nh, hd)
                got = out[row].view(nh, hd)
                assert torch.isfinite(got).all(), (cfg, s_, t)
                err = rel_err(got, ref)
                assert err <= 2 ** -6, (cfg, befores, news, s_, t, err)
    attn_tc.set_wide(1)


def test_the_sink_takes_weight_when_no_key_fits():
    """All scores far below zero: the sink's exp(0) dominates the sum and the output goes to zero; a score far above
    zero: the sink does not matter."""
    ops = _ops()
    hd, n = 16, 70
    g = torch.Generator().manual_seed(1)
    q = torch.randn(1, hd, generator=g)
    k = -q.repeat(n, 1).view(n, 1, hd) * 3
    v = torch.ones(n, 1, hd)
    kc, vc, table = _paged(k, v, 2, seed=3)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    seq = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.empty(1, hd, device=DEV)
    ops.attn_simple(q.to(DEV), kc, vc, out, pos, seq, table, 128, 64, 1, 1, hd, 0, 1.0, sink=True)
    assert float(out.abs().max()) < 1e-6
    ops.attn_simple(q.to(DEV), kc, vc, out, pos, seq, table, 128, 64, 1, 1, hd, 0, 1.0, sink=False)
    assert abs(float(out.mean()) - 1.0) < 1e-5
    ops.attn_simple(-q.to(DEV), kc, vc, out, pos, seq, table, 128, 64, 1, 1, hd, 0, 1.0, sink=True)
    assert abs(float(out.mean()) - 1.0) < 1e-5


def _ssm_inputs(T, H, P, N, G, taps, seed):
    g = torch.Generator().manual_seed(seed)
    inner = H * P
    rows = 2 * inner + 2 * G * N + H
    p = torch.randn(T, rows, generator=g)
    conv_w = torch.randn(inner + 2 * G * N, taps, generator=g) * 0.5
    conv_b = torch.randn(inner + 2 * G * N, generator=g) * 0.2
    dt_bias, a_log = torch.randn(H, generator=g) * 0.5, torch.randn(H, generator=g) * 0.5
    d_skip, norm_w = 1 + 0.2 * torch.randn(H, generator=g), 1 + 0.1 * torch.randn(inner, generator=g)
    return p, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w


def _plain_ssm(p, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w, H, P_, N, G, groups, eps):
    """The state-space mixer between its two projections, float64, from the plain implementation's pieces."""
    import plain_tinuzen as P
    T, inner = p.shape[0], H * P_
    p = p.double()
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = P.silu(P.causal_conv(xbc, conv_w.double(), conv_b.double()))
    x = xbc[:, :inner].view(T, H, P_)
    B = xbc[:, inner:inner + G * N].view(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].view(T, G, N).repeat_interleave(H // G, dim=1)
    y = P.state_space_scan(x, B, C, P.softplus(dt + dt_bias.double()), a_log.double(), d_skip.double()).reshape(T, inner)
    y = (y * P.silu(z)).view(T, groups, inner // groups)
    return (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, inner) * norm_w.double()


@pytest.mark.parametrize("shape", [(4, 16, 16, 2, 3, 2), (3, 10, 5, 3, 1, 1), (2, 33, 20, 1, 5, 2), (2, 64, 128, 1, 4, 4),
                                   (6, 8, 12, 3, 2, 3), (1, 1, 256, 1, 16, 1)])
def test_state_space_kernels_in_one_piece_in_portions_and_in_a_batch(shape):
    ops = _ops()
    H, P_, N, G, taps, groups = shape
    T, eps = 150, 1e-5
    inner, C = H * P_, H * P_ + 2 * G * N
    ins = _ssm_inputs(T, H, P_, N, G, taps, seed=N + P_)
    p, conv_w, conv_b, dt_bias, a_log, d_skip, norm_w = ins
    ref = _plain_ssm(*ins, H, P_, N, G, groups, eps) * 0.8
    dev = [t.contiguous().to(DEV) for t in ins]
    shp = ops.ssm_shape(H, P_, N, G, taps, (0, inner, 2 * inner, 2 * inner + G * N, 2 * inner + 2 * G * N))

    def run(rows, starts, slots, S, cs):
        """rows of p, packed; starts / slots of the step's sequences."""
        pp = dev[0][rows].contiguous()
        n = pp.shape[0]
        b = _Seqs(starts, slots)
        one = b.max_new == 1
        xbc, dtv, dec = torch.empty(n, C, device=DEV), torch.empty(n, H, device=DEV), torch.empty(n, H, device=DEV)
        y, out = torch.empty(n, inner, device=DEV), torch.empty(n, inner, device=DEV)
        ops.ssm_prepare(pp, shp, dev[1], dev[2], cs, dev[3], dev[4], b, xbc, dtv, dec, update_state=one)
        if not one:
            ops.ssm_conv_state_update(pp, shp, cs, b)
        ops.ssm_scan(xbc, dtv, dec, dev[5], y, S, b, H, P_, N, G)
        ops.ssm_finish(y, pp, shp, dev[6], out, groups, eps, 0.8)
        return out
    K = max(taps - 1, 1)
    S, cs = torch.zeros(3, H, N, P_, device=DEV), torch.zeros(3, K, C, device=DEV)
    whole = run(torch.arange(T), [0, T], [1], S, cs)
    assert rel_err(whole, ref) < 3e-5
    assert float(S[0].abs().max()) == 0.0 and float(S[2].abs().max()) == 0.0              # other slots untouched
    S2, cs2 = torch.zeros(3, H, N, P_, device=DEV), torch.zeros(3, K, C, device=DEV)
    cuts = [0, 1, 2, 4, 8, 9, 10, 17, 80, 81, 149, T]
    parts = [run(torch.arange(a, b), [0, b - a], [2], S2, cs2) for a, b in zip(cuts[:-1], cuts[1:])]
    assert torch.equal(torch.cat(parts), whole) and torch.equal(S2[2], S[1]) and torch.equal(cs2[2], cs[1])    # the same bits
    # two sequences in one launch, the second the first 60 tokens of the same data, in other slots
    S3, cs3 = torch.zeros(3, H, N, P_, device=DEV), torch.zeros(3, K, C, device=DEV)
    both = run(torch.cat([torch.arange(T), torch.arange(60)]), [0, T, T + 60], [2, 0], S3, cs3)
    assert torch.equal(both[:T], whole) and torch.equal(both[T:], whole[:60]) and torch.equal(S3[2], S[1])
    # and token by token, two sequences a step, one of them later in its data than the other
    S4, cs4 = torch.zeros(3, H, N, P_, device=DEV), torch.zeros(3, K, C, device=DEV)
    for t in range(20):
        if t < 3:
            o = run(torch.tensor([t]), [0, 1], [0], S4, cs4)
        else:
            o = run(torch.tensor([t, t - 3]), [0, 1, 2], [0, 1], S4, cs4)
            assert torch.equal(o[1], whole[t - 3])
        assert torch.equal(o[0], whole[t])


def test_scan_gives_the_same_bits_with_one_and_with_two_columns_a_thread():
    """A launch with many blocks lets a thread hold two columns of the state (they share the reads of B and C); the
    sums of a column keep their order, so forty sequences in one launch give each the bits of one sequence alone."""
    ops = _ops()
    H, P_, N, G, T, n = 6, 8, 16, 3, 21, 40
    C = H * P_ + 2 * G * N
    g = torch.Generator().manual_seed(3)
    xbc, dtv, dec = torch.randn(T, C, generator=g), torch.rand(T, H, generator=g), torch.rand(T, H, generator=g)
    d = torch.randn(H, generator=g).to(DEV)
    y1, S1 = torch.empty(T, H * P_, device=DEV), torch.zeros(1, H, N, P_, device=DEV)
    ops.ssm_scan(xbc.to(DEV), dtv.to(DEV), dec.to(DEV), d, y1, S1, _Seqs([0, T], [0]), H, P_, N, G)
    yn, Sn = torch.empty(n * T, H * P_, device=DEV), torch.zeros(n, H, N, P_, device=DEV)
    ops.ssm_scan(xbc.repeat(n, 1).to(DEV), dtv.repeat(n, 1).to(DEV), dec.repeat(n, 1).to(DEV), d, yn, Sn,
                 _Seqs([i * T for i in range(n + 1)], list(range(n))), H, P_, N, G)
    for i in (0, 17, n - 1):
        assert torch.equal(yn[i * T:(i + 1) * T], y1) and torch.equal(Sn[i], S1[0])


def test_the_state_keeps_an_early_input_for_hundreds_of_tokens():
    """A decay next to 1 and inputs of zero afterwards: what token 0 wrote is read out unchanged 400 tokens later."""
    ops = _ops()
    H, P_, N, G, T = 1, 8, 16, 1, 401
    C = P_ + 2 * N
    xbc = torch.zeros(T, C)
    xbc[0, :P_] = 3.0                                           # x_0
    xbc[0, P_] = 1.0                                            # B_0 = e_0
    xbc[T - 1, P_ + N] = 1.0                                    # C_last = e_0
    dtv = torch.ones(T, H)
    dec = torch.ones(T, H)
    y = torch.empty(T, P_, device=DEV)
    ops.ssm_scan(xbc.to(DEV), dtv.to(DEV), dec.to(DEV), torch.zeros(H, device=DEV), y, torch.zeros(1, H, N, P_, device=DEV),
                 _Seqs([0, T], [0]), H, P_, N, G)
    assert float((y[T - 1] - 3.0).abs().max()) < 1e-6 and float(y[1:T - 1].abs().max()) == 0.0


# ---------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """Random models whose projections are scaled up after drawing, so that attention weights are far from uniform,
    gates far from one half and the table of pairs as large as the token rows."""
    import plain_tinuzen as P
    import ultima_b200 as u
    from ultima_b200.weights.safetensors_io import write_safetensors
    base = tmp_path_factory.mktemp("tinuzen")
    made = {}

    def get(name):
        if name not in made:
            d = str(base / name)
            u.write_random_model(d, u.config_from_dict(CONFIGS[name]), seed=len(name), dtype="bfloat16")
            _, W = P.read_folder(d)
            scaled = {}
            for n, t in W.items():
                amp = 2.0 if name == "wide" else 3.0           # (nine runs of layers: less, or bfloat16 rounding grows past any bound)
                f = amp if (t.dim() == 2 and n not in ("embed", "loop.step") and not n.endswith(".conv")) else 1.0
                if n.endswith((".left.q", ".left.k")):
                    f = 2 * amp
                scaled[n] = (t * f).to(torch.bfloat16)
            write_safetensors(os.path.join(d, "model.safetensors"), scaled)
            made[name] = (d,) + P.read_folder(d)
        return made[name]
    return get


_engines = {}


def _engine(folder, dtype, **kw):
    from ultima_b200.engine import Engine
    key = (folder, dtype, tuple(sorted(kw.items())))
    if key not in _engines:
        _engines[key] = Engine.from_dir(folder, dtype=dtype, with_sampler=False, **{"max_tokens": 2048, "max_seqs": 6, **kw})
    return _engines[key]


def _ids(seed, n, vocab):
    return np.random.default_rng(seed).integers(0, vocab, size=n).tolist()


def _all(n):
    return list(range(n))


def _runs(cfg):
    import plain_tinuzen as P
    return len(P.layer_order(cfg))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_prompt_in_one_step_every_position_and_every_layer(folders, name, dtype):
    import plain_tinuzen as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype, poison_cache=True)
    for seed, n in ((1, 1), (2, 2), (3, 277)):                 # 277: past window and page borders of every configuration
        ids = _ids(seed, n, cfg["vocab"])
        taps, layers = [], []
        eng.model.tap = lambda i, x: taps.append(x.detach().double().cpu())
        s = eng.open(1)
        got = eng.step(s, [ids], [_all(n)]).cpu().numpy()
        eng.close(s)
        eng.model.tap = None
        eng.check_errors()
        with torch.no_grad():
            ref = P.forward(cfg, W, ids, torch.float64, layers).numpy()
        assert len(taps) == len(layers) == _runs(cfg)
        if dtype == "float32":
            for i, (a, b) in enumerate(zip(taps, layers)):     # the residual stream behind every run of a layer
                assert rel_err(a, b) < 2e-5, (name, n, i)
        err, bound = close_enough(got, ref, dtype, 2 * _runs(cfg))
        assert err <= bound, (name, dtype, n, err, bound)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_against_token_by_token_and_portions(folders, name):
    """float32: a sequence run whole, token by token, and in portions of several sizes gives the same logits
    up to rounding, and all of them the plain implementation's."""
    import plain_tinuzen as P
    d, cfg, W = folders(name)
    eng = _engine(d, "float32", poison_cache=True)
    n = 150
    ids = _ids(11, n, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    for sizes in ([1] * n, [2] * 75, [3, 2, 64, 1, 65, 2, 13], [149, 1], [5] + [1] * 145):
        assert sum(sizes) == n
        s = eng.open(1)
        rows, at = [], 0
        for m in sizes:
            rows.append(eng.step(s, [ids[at:at + m]], [_all(m)]).cpu().numpy())
            at += m
        eng.close(s)
        eng.check_errors()
        err, bound = close_enough(np.concatenate(rows), ref, "float32")
        assert err <= bound, (name, sizes[:4], err, bound)
    # the same through passes inside one step (a step cut at 16 tokens)
    small = _engine(d, "float32", max_step_tokens=16)
    s = small.open(1)
    got = small.step(s, [ids], [_all(n)]).cpu().numpy()
    small.close(s)
    err, bound = close_enough(got, ref, "float32")
    assert err <= bound, (name, "passes", err, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_unequal_requests_together_then_decoded_with_slots_used_again(folders, name, dtype):
    import plain_tinuzen as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype, poison_cache=True)
    for round_ in range(2):                                    # the second time on slots and pages just given back
        lens, tail = [1, 130, 66, 23], [3, 20, 9, 20]
        seqs = [_ids(20 + 10 * round_ + i, a + b, cfg["vocab"]) for i, (a, b) in enumerate(zip(lens, tail))]
        refs = [P.logits(cfg, W, s) for s in seqs]
        slots = eng.open(4)
        got = [dict() for _ in seqs]
        out = eng.step(slots, [s[:a] for s, a in zip(seqs, lens)], [_all(a) for a in lens]).cpu().numpy()
        o = 0
        for i, a in enumerate(lens):
            for p in range(a):
                got[i][p] = out[o]
                o += 1
        live = list(range(4))
        for t in range(max(tail)):
            live = [i for i in live if t < tail[i]]            # the shorter requests end earlier
            out = eng.step([slots[i] for i in live], [[seqs[i][lens[i] + t]] for i in live]).cpu().numpy()
            for r, i in enumerate(live):
                got[i][lens[i] + t] = out[r]
            for i in list(live):
                if t + 1 == tail[i]:
                    eng.close([slots[i]])
        eng.check_errors()
        for i, s in enumerate(seqs):
            g = np.stack([got[i][p] for p in range(len(s))])
            err, bound = close_enough(g, refs[i], dtype, 2 * _runs(cfg))
            assert err <= bound, (name, dtype, round_, i, err, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["mixed", "wide"])
def test_long_decoding_over_window_and_page_borders(folders, name, dtype):
    import plain_tinuzen as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype)
    ids = _ids(5, 210, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    s = eng.open(1)
    rows = [eng.step(s, [ids[:4]], [_all(4)]).cpu().numpy()]
    for t in range(4, 210):
        rows.append(eng.step(s, [[ids[t]]]).cpu().numpy())
    eng.close(s)
    eng.check_errors()
    err, bound = close_enough(np.concatenate(rows), ref, dtype, 2 * _runs(cfg))
    assert err <= bound, (dtype, err, bound)


def test_greedy_generation_through_the_loop(folders):
    import plain_tinuzen as P
    import ultima_b200 as u
    d, cfg, W = folders("mixed")
    llm = u.LLM(d, dtype="float32", n_ctx=128, max_batch=2)
    prompts = [_ids(1, 9, cfg["vocab"]), _ids(2, 30, cfg["vocab"])]
    outs = llm.generate(prompts, n_predict=8, temp=0.0)
    for p, g in zip(prompts, outs):
        ids = list(p)
        for _ in range(8):
            ids.append(int(np.argmax(P.logits(cfg, W, ids)[-1])))
        assert g.tokens == ids[len(p):], (g.tokens, ids[len(p):])


def test_trace_replay_and_the_command_line(folders, tmp_path):
    import plain_tinuzen as P
    d, cfg, W = folders("odd")
    listed = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ultima"), "archinfo", d], capture_output=True,
                            text=True, timeout=300)
    assert listed.returncode == 0 and "l0.mix.right.A_log" in listed.stdout and "all " in listed.stdout, listed.stderr[-1500:]
    a, b = _ids(3, 70, cfg["vocab"]), _ids(4, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + t]], "want": [0]}],
                      "end": ["a", "b"] if t == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})      # a slot used again
    for dtype in ("float32", "bfloat16"):
        out_dir = str(tmp_path / ("out_" + dtype))
        p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype,
                            "--out", out_dir, "--max-tokens", "192"], input="".join(json.dumps(s) + "\n" for s in steps),
                           capture_output=True, text=True, timeout=900)
        assert p.returncode == 0 and "done 5" in p.stdout, p.stderr[-2000:]
        ra, rb = P.logits(cfg, W, a), P.logits(cfg, W, b)
        got = [np.fromfile(os.path.join(out_dir, "0.f32"), dtype="<f4").reshape(3, cfg["vocab"])]
        want = [ra[0], ra[65], rb[4]]
        for t in range(4):
            got.append(np.fromfile(os.path.join(out_dir, f"{t + 1}.f32"), dtype="<f4").reshape(2, cfg["vocab"]))
            want += [ra[66 + t], rb[5 + t]]
        got.append(np.fromfile(os.path.join(out_dir, "5.f32"), dtype="<f4").reshape(1, cfg["vocab"]))
        want.append(rb[8])
        err, bound = close_enough(np.concatenate(got), np.stack(want), dtype, 8)
        assert err <= bound, (dtype, err, bound)
