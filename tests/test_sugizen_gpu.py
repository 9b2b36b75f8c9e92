"""Sugizen on the GPU against the plain implementation (tests/plain_sugizen.py): each mechanism's kernels
alone, then whole models from small configurations with random weights: prompts, token-by-token decoding,
portions, batches of unequal requests, slots used again, long decoding, greedy generation, trace replay."""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from conftest import ROOT, close_enough, has_gpu
from sugizen_configs import CONFIGS

pytestmark = [pytest.mark.gpu, pytest.mark.skipif(not has_gpu(), reason="needs a CUDA device")]
DEV = "cuda:0"


def _ops():
    from ultima_b200.kernels import ops
    return ops


def rel_err(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max() / max(1e-30, float(ref.abs().max())))


# ---------------------------------------------------------------------------------------
# mechanisms alone
# ---------------------------------------------------------------------------------------
@pytest.mark.parametrize("width", [64, 100, 2048])
def test_norm_on_a_sublayers_output(width):
    import plain_sugizen as P
    ops = _ops()
    g = torch.Generator().manual_seed(width)
    x, y, w = torch.randn(5, width, generator=g), torch.randn(5, width, generator=g) * 3, 1 + 0.1 * torch.randn(width, generator=g)
    ref = x.double() + P.rms_norm(y.double(), w.double(), 1e-5)
    xd, yd = x.to(DEV), y.to(DEV)
    h = torch.empty(5, width, dtype=torch.bfloat16, device=DEV)
    ops.rmsnorm_add(yd, w.to(DEV), xd, 1e-5, h=h, clear_y=True)
    assert rel_err(xd, ref) < 1e-6 and rel_err(h, ref) < 2 ** -7 and float(yd.abs().max()) == 0.0
    xd, yd = x.to(DEV), y.to(DEV)
    ops.rmsnorm_add(yd, w.to(DEV), xd, 1e-5)
    assert rel_err(xd, ref) < 1e-6 and torch.equal(yd.cpu(), y)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_gate_product_and_head_gate(dtype):
    ops = _ops()
    g = torch.Generator().manual_seed(2)
    T, F = 7, 37
    gu = (torch.randn(T, 2 * F, generator=g) * 2).to(DEV)
    for limit, alpha, shift in ((1.5, 1.702, 1.0), (0.4, 1.0, 0.0)):
        gate = torch.clamp(gu[:, :F].double(), max=limit)
        up = torch.clamp(gu[:, F:].double(), -limit, limit)
        ref = gate * torch.sigmoid(alpha * gate) * (up + shift)
        out = torch.empty(T, F, dtype=dtype, device=DEV)
        ops.glu_clamped(gu, out, limit, alpha, shift)
        assert rel_err(out, ref) < (1e-6 if dtype == torch.float32 else 2 ** -7)
    nh, hd = 3, 10
    o = torch.randn(T, nh * hd, generator=g).to(dtype).to(DEV)
    wide = torch.randn(T, nh + 5, generator=g).to(DEV)
    ref = (o.double().view(T, nh, hd) * torch.sigmoid(wide[:, 2:2 + nh].double())[:, :, None]).view(T, nh * hd)
    ops.head_gate(o, wide[:, 2:2 + nh], nh, hd)
    assert rel_err(o, ref) < (1e-6 if dtype == torch.float32 else 2 ** -7)


@pytest.mark.parametrize("T", [5, 300, 1500])
def test_clamped_gate_product_as_the_tensor_core_products_epilogue(T):
    """Sums large enough that both clamps are active; few tokens, many, and enough for the two-CTA kernel."""
    from ultima_b200.engine.runtime import Runtime
    ops = _ops()
    rt = Runtime(DEV, torch.bfloat16)
    g = torch.Generator().manual_seed(T)
    F, K = 192, 128
    a = torch.randn(T, K, generator=g).to(torch.bfloat16).to(DEV)
    wg = (torch.randn(F, K, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    wu = (torch.randn(F, K, generator=g) * 0.2).to(torch.bfloat16).to(DEV)
    wgu = torch.stack([wg.view(F // 64, 64, K), wu.view(F // 64, 64, K)], dim=1).reshape(2 * F, K).contiguous()
    for limit, alpha, shift in ((1.5, 1.702, 1.0), (0.5, 1.0, 0.0)):
        gate = torch.clamp(a.double() @ wg.double().T, max=limit)
        up = torch.clamp(a.double() @ wu.double().T, -limit, limit)
        assert float((gate == limit).double().mean()) > 0.1 and float((up.abs() == limit).double().mean()) > 0.2
        ref = gate * torch.sigmoid(alpha * gate) * (up + shift)
        out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
        rt.matmul(a, wgu, out, ops.EPI_SWIGLU_IL, gate=(limit, alpha, shift))
        rt.check_status()
        assert rel_err(out, ref) < 2 ** -6, (T, limit)
    # without the constants the epilogue is the plain silu(g) * u
    out = torch.empty(T, F, dtype=torch.bfloat16, device=DEV)
    rt.matmul(a, wgu, out, ops.EPI_SWIGLU_IL)
    gsum, usum = a.double() @ wg.double().T, a.double() @ wu.double().T
    assert rel_err(out, gsum * torch.sigmoid(gsum) * usum) < 2 ** -6


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
@pytest.mark.parametrize("cfg", [dict(nh=6, nkv=2, hd=48, hdv=16, block=50), dict(nh=2, nkv=2, hd=16, hdv=200, block=64),
                                 dict(nh=4, nkv=1, hd=96, hdv=96, block=7), dict(nh=3, nkv=3, hd=20, hdv=24, block=0)])
def test_attention_with_blocks_value_size_and_gate(cfg, dtype):
    ops = _ops()
    nh, nkv, hd, hdv, block = cfg["nh"], cfg["nkv"], cfg["hd"], cfg["hdv"], cfg["block"]
    n = 300
    g = torch.Generator().manual_seed(hd)
    k = torch.randn(n, nkv, hd, generator=g).to(dtype)
    v = torch.randn(n, nkv, hdv, generator=g).to(dtype)
    kc, vc, table = _paged(k, v, 5, seed=1)
    places = sorted({0, 1, 6, 7, 49, 50, 63, 64, 65, 99, 100, 127, 128, 199, 200, 255, 256, 299})
    q = torch.randn(len(places), nh * hd, generator=g).to(dtype).to(DEV)
    gate = torch.randn(len(places), nh + 3, generator=g).to(DEV)[:, 1:1 + nh]
    out = torch.empty(len(places), nh * hdv, dtype=dtype, device=DEV)
    pos = torch.tensor(places, dtype=torch.int32, device=DEV)
    seq = torch.zeros(len(places), dtype=torch.int32, device=DEV)
    ops.attn_simple(q, kc, vc, out, pos, seq, table, 5 * 64, 64, nh, nkv, hd, 0, 0.3, v_head_dim=hdv, block=block, gate=gate)
    for i, p in enumerate(places):
        lo = p - p % block if block else 0
        for h in range(nh):
            kv = h // (nh // nkv)
            s = (k[lo:p + 1, kv].double() @ q[i].double().cpu().view(nh, hd)[h]) * 0.3
            ref = (torch.softmax(s, 0) @ v[lo:p + 1, kv].double()) * torch.sigmoid(gate[i, h].double().cpu())
            err = rel_err(out[i].view(nh, hdv)[h], ref)
            assert err <= (2e-5 if dtype == torch.float32 else 2 ** -6), (p, h, err)


def test_a_key_just_outside_a_block_is_not_seen_and_one_just_inside_is():
    """One key is made to stand out; a query of the same block must return its value, a query of the next
    block must not know it.  The block's edge is put on a page's border and off it."""
    ops = _ops()
    nh, nkv, hd, n = 2, 1, 32, 640
    for block, marked in ((64, 128), (64, 191), (100, 300), (100, 399), (250, 250), (640, 3)):
        g = torch.Generator().manual_seed(block + marked)
        k = torch.randn(n, nkv, hd, generator=g) * 0.1
        v = torch.randn(n, nkv, hd, generator=g) * 0.1
        qdir = torch.randn(hd, generator=g)
        k[marked, 0] = qdir * 40.0
        v[marked, 0] = 5.0
        kc, vc, table = _paged(k, v, 10, seed=block)
        first, last = marked - marked % block, min(n, marked - marked % block + block) - 1
        places = [p for p in (marked, marked + 1, last, last + 1, first - 1, n - 1) if 0 <= p < n]
        q = (qdir * 0.5).repeat(len(places), nh).to(DEV)
        out = torch.empty(len(places), nh * hd, device=DEV)
        pos = torch.tensor(places, dtype=torch.int32, device=DEV)
        ops.attn_simple(q, kc, vc, out, pos, torch.zeros_like(pos), table, 640, 64, nh, nkv, hd, 0, 1.0, block=block)
        for i, p in enumerate(places):
            inside = first <= marked <= p <= last
            got = float(out[i, :hd].mean())
            assert (got > 4.9) if inside else (abs(got) < 1.0), (block, marked, p, got)


class _View:
    def __init__(self, k, v, table, ring):
        self.k, self.v, self.table, self.ring, self.page, self.window, self.owner = k, v, table, ring, 64, None, True


class _Step:
    def __init__(self, befores, news):
        start = [0]
        for n in news:
            start.append(start[-1] + n)
        self.seq_start = torch.tensor(start, dtype=torch.int32, device=DEV)
        self.seq_before = torch.tensor(befores, dtype=torch.int32, device=DEV)
        self.n_seqs, self.max_new, self.max_after = len(news), max(news), max(b + n for b, n in zip(befores, news))


@pytest.mark.parametrize("hd,kernel", [(64, None), (128, None), (96, None), (48, None), (64, "mma"), (128, "tc")])
def test_the_tensor_core_attention_kernels_keep_to_the_block(hd, kernel):
    """The same marked key for the kernels that prompts and single tokens of the bfloat16 path use (tcgen05 and
    mma.sync for prompts; TMA-fed, cp.async and tcgen05 for single tokens): every row of a prompt, and single
    tokens at the places around the block's edges, must see the marked key exactly when it lies in their block
    and not after them."""
    from ultima_b200.engine.runtime import Runtime
    from ultima_b200.kernels import attn_tc
    rt = Runtime(DEV, torch.bfloat16)
    nh, nkv, n = 4, 2, 640
    for block, marked in ((64, 128), (64, 191), (100, 300), (100, 399), (250, 250), (37, 36)):
        g = torch.Generator().manual_seed(block + marked + hd)
        k = (torch.randn(n, nkv, hd, generator=g) * 0.1)
        v = (torch.randn(n, nkv, hd, generator=g) * 0.1)
        qdir = torch.randn(hd, generator=g)
        k[marked] = qdir * 40.0
        v[marked] = 5.0
        kc, vc, table = _paged(k.to(torch.bfloat16), v.to(torch.bfloat16), 10, seed=block)
        kv = _View(kc, vc, table, 640)
        first, last = marked - marked % block, min(n, marked - marked % block + block) - 1
        q_all = (qdir * 0.5).repeat(n, nh).to(torch.bfloat16).to(DEV)
        if kernel != "tc":                                      # a prompt of all 640 positions
            out = torch.full((n, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            attn_tc.attention(q_all, kv, out, _Step([0], [n]), nh, nkv, hd, 1.0, rt, kernel=kernel, block=block)
            rt.check_status()
            got = out.float().view(n, nh, hd).mean(-1).cpu()
            for p in range(n):
                inside = first <= marked <= p <= last
                assert bool((got[p] > 4.8).all()) if inside else bool((got[p].abs() < 1.0).all()), (hd, block, marked, p, got[p])
        for p in {marked, marked + 1, last, last + 1, first - 1, n - 1}:          # single tokens
            if not 0 <= p < n:
                continue
            out = torch.full((1, nh * hd), float("nan"), dtype=torch.bfloat16, device=DEV)
            attn_tc.attention(q_all[:1], kv, out, _Step([p], [1]), nh, nkv, hd, 1.0, rt, kernel=kernel, block=block)
            rt.check_status()
            got = out.float().view(nh, hd).mean(-1).cpu()
            inside = first <= marked <= p <= last
            assert bool((got > 4.8).all()) if inside else bool((got.abs() < 1.0).all()), (hd, block, marked, p, got)


def _scan_inputs(T, H, G, D, E, seed, slow_decay=False):
    g = torch.Generator().manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(T, G, D, generator=g), dim=-1) * D ** -0.5
    k = torch.nn.functional.normalize(torch.randn(T, G, D, generator=g), dim=-1)
    v = torch.randn(T, H, E, generator=g)
    beta = torch.sigmoid(torch.randn(T, H, generator=g))
    dec = torch.exp(-torch.rand(T, H, D, generator=g) * (0.001 if slow_decay else 0.5))
    return q, k, v, beta, dec


class _Seqs:
    """The few fields of a step's batch that the delta kernels read."""

    def __init__(self, starts, slots):
        self.seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
        self.seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
        self.n_seqs = len(slots)
        seq = []
        for i in range(len(slots)):
            seq += [i] * (starts[i + 1] - starts[i])
        self.tok_seq = torch.tensor(seq, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("shape", [(4, 2, 24, 40), (3, 3, 64, 64), (2, 1, 72, 33), (2, 2, 130, 8), (1, 1, 8, 1), (6, 3, 256, 16)])
def test_delta_rule_scan_in_one_piece_in_portions_and_in_a_batch(shape):
    import plain_sugizen as P
    ops = _ops()
    H, G, D, E = shape
    T = 150
    q, k, v, beta, dec = _scan_inputs(T, H, G, D, E, seed=D + E)
    rep = H // G
    ref = P.delta_rule_scan(q.double().repeat_interleave(rep, 1), k.double().repeat_interleave(rep, 1), v.double(),
                            beta.double(), dec.double())
    dev = [t.contiguous().to(DEV) for t in (q.view(T, -1), k.view(T, -1), v.view(T, -1), beta, dec.view(T, -1))]

    def run(cuts, slot, state):
        out = torch.empty(T, H * E, device=DEV)
        for a, b in zip(cuts[:-1], cuts[1:]):
            part = [t[a:b].contiguous() for t in dev]
            o = torch.empty(b - a, H * E, device=DEV)
            ops.delta_scan(*part, o, state, _Seqs([0, b - a], [slot]), H, G, D, E)
            out[a:b] = o
        return out
    state = torch.zeros(3, H, D, E, device=DEV)
    whole = run([0, T], 1, state)
    assert rel_err(whole.view(T, H, E), ref) < 3e-5
    assert float(state[0].abs().max()) == 0.0 and float(state[2].abs().max()) == 0.0       # other slots untouched
    state2 = torch.zeros(3, H, D, E, device=DEV)
    cut = run([0, 1, 3, 8, 9, 17, 80, 81, 149, T], 2, state2)
    assert torch.equal(cut, whole) and torch.equal(state2[2], state[1])                     # portions: the same bits
    # two sequences in one launch, the second the first 60 tokens of the same data, in other slots
    both = [torch.cat([t, t[:60]]).contiguous() for t in dev]
    o = torch.empty(T + 60, H * E, device=DEV)
    state3 = torch.zeros(3, H, D, E, device=DEV)
    ops.delta_scan(*both, o, state3, _Seqs([0, T, T + 60], [2, 0]), H, G, D, E)
    assert torch.equal(o[:T], whole) and torch.equal(o[T:], whole[:60]) and torch.equal(state3[2], state[1])


def test_the_delta_state_keeps_an_early_write_for_hundreds_of_tokens():
    """With decays next to 1 and keys orthogonal to the first one, what token 0 wrote is read out unchanged by
    a query along its key 400 tokens later."""
    ops = _ops()
    H, G, D, E, T = 1, 1, 32, 16, 401
    q, k, v, beta, dec = _scan_inputs(T, H, G, D, E, seed=9, slow_decay=True)
    dec[:] = 1.0
    k[:, 0, 0] = 0.0
    k = torch.nn.functional.normalize(k, dim=-1)
    k[0, 0] = 0.0
    k[0, 0, 0] = 1.0
    beta[0] = 1.0
    v[0, 0] = 3.0
    q[T - 1, 0] = k[0, 0]
    dev = [t.contiguous().to(DEV) for t in (q.view(T, -1), k.view(T, -1), v.view(T, -1), beta, dec.view(T, -1))]
    out = torch.empty(T, H * E, device=DEV)
    ops.delta_scan(*dev, out, torch.zeros(1, H, D, E, device=DEV), _Seqs([0, T], [0]), H, G, D, E)
    assert float((out[T - 1] - 3.0).abs().max()) < 1e-4


# ---------------------------------------------------------------------------------------
# whole models
# ---------------------------------------------------------------------------------------
@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    import plain_sugizen as P
    import ultima_b200 as u
    base = tmp_path_factory.mktemp("sugizen")
    made = {}

    def get(name):
        if name not in made:
            d = str(base / name)
            u.write_random_model(d, u.config_from_dict(CONFIGS[name]), seed=len(name), dtype="bfloat16")
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


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_a_prompt_in_one_step_every_position(folders, name, dtype):
    import plain_sugizen as P
    d, cfg, W = folders(name)
    eng = _engine(d, dtype, poison_cache=True)
    for seed, n in ((1, 1), (2, 2), (3, 277)):                 # 277: past block and page borders of every configuration
        ids = _ids(seed, n, cfg["vocab"])
        s = eng.open(1)
        got = eng.step(s, [ids], [_all(n)]).cpu().numpy()
        eng.close(s)
        eng.check_errors()
        err, bound = close_enough(got, P.logits(cfg, W, ids), dtype, 2 * len(cfg["layers"]))
        assert err <= bound, (name, dtype, n, err, bound)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_prompt_against_token_by_token_and_portions(folders, name):
    """float32: a sequence run whole, token by token, and in portions of several sizes gives the same logits
    up to rounding, and all of them the plain implementation's."""
    import plain_sugizen as P
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
    import plain_sugizen as P
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
            err, bound = close_enough(g, refs[i], dtype, 2 * len(cfg["layers"]))
            assert err <= bound, (name, dtype, round_, i, err, bound)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_over_block_and_page_borders(folders, dtype):
    import plain_sugizen as P
    d, cfg, W = folders("mixed")
    eng = _engine(d, dtype)
    ids = _ids(5, 210, cfg["vocab"])
    ref = P.logits(cfg, W, ids)
    s = eng.open(1)
    rows = [eng.step(s, [ids[:4]], [_all(4)]).cpu().numpy()]
    for t in range(4, 210):
        rows.append(eng.step(s, [[ids[t]]]).cpu().numpy())
    eng.close(s)
    eng.check_errors()
    err, bound = close_enough(np.concatenate(rows), ref, dtype, 2 * len(cfg["layers"]))
    assert err <= bound, (dtype, err, bound)


def test_greedy_generation_through_the_loop(folders):
    import plain_sugizen as P
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
    import plain_sugizen as P
    d, cfg, W = folders("odd")
    listed = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "ultima"), "archinfo", d], capture_output=True,
                            text=True, timeout=300)
    assert listed.returncode == 0 and "l0.mix.a2" in listed.stdout and "all " in listed.stdout, listed.stderr[-1500:]
    a, b = _ids(3, 70, cfg["vocab"]), _ids(4, 9, cfg["vocab"])
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:66], "want": [0, 65]}, {"id": "b", "tokens": b[:5], "want": [4]}], "end": []}]
    for t in range(4):
        steps.append({"step": t + 1, "entries": [{"id": "a", "tokens": [a[66 + t]], "want": [0]},
                                                 {"id": "b", "tokens": [b[5 + t]], "want": [0]}],
                      "end": ["a", "b"] if t == 3 else []})
    steps.append({"step": 5, "entries": [{"id": "c", "tokens": b, "want": [8]}], "end": ["c"]})      # a slot used again
    out_dir = str(tmp_path / "out")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", "float32",
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
    err, bound = close_enough(np.concatenate(got), np.stack(want), "float32")
    assert err <= bound, (err, bound)
