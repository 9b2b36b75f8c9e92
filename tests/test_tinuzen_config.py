"""Tinuzen without a GPU: reading and writing the configuration, the model as data (layers, run list, tensor
names, what each run asks of the cache), and the plain implementation's own pieces against one another."""
import copy

import numpy as np
import pytest
import torch

import ultima_b200 as u
from tinuzen_configs import CONFIGS, MIXED, ODD, WIDE
from ultima_b200.config.base import ConfigError
from ultima_b200.parts.base import KVNeed, StateNeed


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_configuration_reads_writes_and_names_its_tensors(name):
    cfg = u.config_from_dict(CONFIGS[name])
    assert cfg.architecture == "Tinuzen" and u.config_from_dict(cfg.to_dict()) == cfg
    spec = u.model_spec_for(cfg)
    names = {s.name: s.shape for s in spec.weight_specs()}
    c = CONFIGS[name]
    assert names["embed"] == (c["vocab"], c["width"]) and names["bigram"] == (c["embedding"]["bigram"]["buckets"] + 1, c["width"])
    assert names["final.norm"] == (c["width"],) and names["head"] == (c["vocab"], c["width"])
    if c.get("loop"):
        assert names["loop.step"] == (c["loop"]["times"], c["width"])
    else:
        assert "loop.step" not in names
    for i, L in enumerate(c["layers"]):
        m = L["mixer"]
        assert names[f"l{i}.rg1"] == (c["width"], c["width"]) and names[f"l{i}.rg1.b"] == (c["width"],)
        assert (f"l{i}.rg2" in names) == (L["mlp"] is not None) == (f"l{i}.mlp.down" in names)
        if L["type"] == "attention":
            assert names[f"l{i}.mix.q.norm"] == (m["heads"] * m["dim"],) and names[f"l{i}.mix.k.norm"] == (m["kv_heads"] * m["dim"],)
            assert names[f"l{i}.mix.v"] == (m["kv_heads"] * m["vdim"], c["width"])
            assert names[f"l{i}.mix.o"] == (c["width"], m["heads"] * m["vdim"])
        else:
            a, r = m["left"], m["right"]
            inner = r["heads"] * r["vdim"]
            assert f"l{i}.mix.left.v" not in names and names[f"l{i}.mix.left.g"] == (a["heads"] * a["dim"], c["width"])
            assert names[f"l{i}.mix.right.in"] == (2 * inner + 2 * r["groups"] * r["state"] + r["heads"], c["width"])
            assert names[f"l{i}.mix.right.conv"] == (inner + 2 * r["groups"] * r["state"], r["conv"])
            assert names[f"l{i}.mix.right.norm"] == (inner,) and names[f"l{i}.mix.right.D"] == (r["heads"],)


def test_run_list_repeats_a_group_of_layers_with_a_marker_at_each_pass():
    spec = u.model_spec_for(u.config_from_dict(MIXED))          # loop 1 .. 2, twice
    assert [r.layer for r in spec.runs] == [0, 1, 2, 1, 2, 3]
    assert [r.entry for r in spec.runs] == [None, 0, None, 1, None, None]
    assert [e[0].get("index") for e in spec.entries] == [0, 1] and all(e[1] == "loop." for e in spec.entries)
    spec = u.model_spec_for(u.config_from_dict(WIDE))           # all three layers, three times
    assert [r.layer for r in spec.runs] == [0, 1, 2] * 3 and [r.entry for r in spec.runs] == [0, None, None, 1, None, None, 2, None, None]
    spec = u.model_spec_for(u.config_from_dict(ODD))
    assert [r.layer for r in spec.runs] == [0, 1, 2, 3] and spec.entries == ()


def test_what_the_runs_ask_of_the_cache():
    from ultima_b200.cache import Cache
    from ultima_b200.parts.base import build_part
    spec = u.model_spec_for(u.config_from_dict(MIXED))
    needs = [build_part("mixer", spec.layers[r.layer].part("mixer")).cache_need() for r in spec.runs]
    # a window with kept first positions holds every position; one without them is a ring
    assert needs[0] == KVNeed(2, 32, None, 16) and needs[2] == KVNeed(2, 16, 10, 24)
    side = needs[1]
    assert side[0] == KVNeed(2, 32, None, None) and side[1] == StateNeed((4, 16, 16), "float32") and side[2] == StateNeed((2, 64 + 64), "float32")
    emb = build_part("embedding", spec.embedding).cache_need()
    assert emb == StateNeed((1,), "int32")
    cache = Cache(needs + [emb], [None] * (len(needs) + 1), max_tokens=512, max_context=256, n_slots=3, step_chunk=64)
    # every run of a repeated layer has a cache of its own
    a, b = cache.run_cache(1, [None] * len(cache.kv_groups)), cache.run_cache(3, [None] * len(cache.kv_groups))
    assert a.states[0].data_ptr() != b.states[0].data_ptr() and a.kv.k.data_ptr() != b.kv.k.data_ptr()
    s = cache.acquire()
    last = cache.run_cache(len(needs), []).state
    assert last.dtype == torch.int32 and tuple(last.shape) == (3, 1)
    last[s] = 17
    a.states[0][s] += 1.0
    cache.release(s)
    assert cache.acquire() == s and int(last[s]) == 0 and float(a.states[0][s].abs().sum()) == 0.0


@pytest.mark.parametrize("edit, what", [
    (lambda c: c["layers"][0].__setitem__("type", "convolution"), "type must be"),
    (lambda c: c["layers"][1]["mixer"]["left"].__setitem__("vdim", 8), "vdim must equal dim"),
    (lambda c: c["layers"][1]["mixer"]["left"]["rot"].__setitem__("dims", 7), "rot.dims must be even"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("groups", 3), "multiple of groups"),
    (lambda c: c["layers"][1]["mixer"]["right"].__setitem__("norm_groups", 5), "multiple of norm_groups"),
    (lambda c: c["layers"][0]["mixer"].__setitem__("heads", 3), "multiple of kv_heads"),
    (lambda c: c["loop"].__setitem__("stop", 9), "loop.start < loop.stop"),
    (lambda c: c["embedding"].pop("bigram"), "'embedding' must be"),
    (lambda c: c["layers"][0]["mlp"].__setitem__("kind", "routed"), "mlp.kind must be"),
])
def test_bad_configurations_are_refused_with_the_key_named(edit, what):
    c = copy.deepcopy(MIXED)
    edit(c)
    with pytest.raises(ConfigError, match=what):
        u.config_from_dict(c)


def test_plain_pieces_agree_with_one_another():
    """The plain implementation run whole equals itself run on a prefix (causality), the sink only lowers the weights'
    sum, and the distance bias with slope 0 heads is the plain softmax."""
    import plain_tinuzen as P
    import tempfile
    d = tempfile.mkdtemp()
    u.write_random_model(d, u.config_from_dict(MIXED), seed=2, dtype="float32")
    cfg, W = P.read_folder(d)
    ids = np.random.default_rng(0).integers(0, cfg["vocab"], size=60).tolist()
    whole = P.logits(cfg, W, ids)
    assert np.abs(P.logits(cfg, W, ids[:37]) - whole[:37]).max() < 1e-12
    s = torch.randn(2, 5, 5, dtype=torch.float64)
    seen = torch.tril(torch.ones(5, 5, dtype=torch.bool))
    v = torch.ones(5, 1, 3, dtype=torch.float64)
    with_sink = P.weigh_and_sum(s, seen, v, 2, sink=True)
    assert float(with_sink.max()) < 1.0 and float(P.weigh_and_sum(s, seen, v, 2, sink=False).min()) > 1 - 1e-12
    assert P.layer_order({"layers": [0, 1, 2, 3], "loop": {"start": 1, "stop": 3, "times": 2}}) == \
        [(0, None), (1, 0), (2, None), (1, 1), (2, None), (3, None)]
