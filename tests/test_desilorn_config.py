"""Desilorn's configuration reader and its model written down as data (no GPU): tensor names and shapes, the order in
which layers run when a span is looped, a cache of its own for every run, what the two mixers ask of the attention part,
refusals, the page bookkeeping of a mask of chunks, and the plain implementation checked against itself (token by token
against whole prompts, the masks' edges, the sink's share)."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_desilorn as plain
from cuinfer_b200.cache import CacheManager, group_runs
from cuinfer_b200.config.model_config import ConfigError
from cuinfer_b200.config.registry import architecture_of
from cuinfer_b200.parts import DecoderModel


def sliding(heads=4, kv_heads=2, dim=12, vdim=8, window=10, temp=(0.5, 4), ff=40):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.3}
    if window:
        m["mask"] = {"size": window}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def chunks(heads=3, kv_heads=3, dim=16, vdim=20, chunk=8, rot=(1000.0, 8), ff=24):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": 0.25}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention_2", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


CFG = {"architecture": "Desilorn", "vocab": 61, "width": 48, "norm": {"eps": 1e-5}, "streams": 3,
       "loop": {"start": 1, "stop": 3, "times": 3},
       "layers": [chunks(), sliding(), chunks(chunk=None, rot=None, ff=None), sliding(window=None, temp=None), chunks(chunk=12)]}


def _build(cfg):
    arch = architecture_of(cfg)
    typed = arch.parse(cfg)
    return typed, arch.spec(typed), DecoderModel(arch.spec(typed), torch.float32)


def test_tensor_names_and_shapes_are_those_of_the_plain_model():
    for cfg in (CFG, {k: v for k, v in CFG.items() if k not in ("streams", "loop")}):
        _typed, _spec, model = _build(cfg)
        want = {k: tuple(v.shape) for k, v in plain.random_model(cfg, 0).items()}
        got = {t.name: tuple(t.shape) for t in model.tensors()}
        assert got == want


def test_looped_layers_run_in_a_row_and_every_run_has_a_cache_of_its_own():
    typed, spec, model = _build(CFG)
    assert list(spec.order) == plain.run_order(CFG) == [0, 1, 2, 1, 2, 1, 2, 3, 4]
    needs = model.cache_needs()
    assert sorted(needs) == list(range(9)), "one cache per layer run"
    for run, layer in enumerate(spec.order):
        m = CFG["layers"][layer]["mixer"]
        need = needs[run]
        assert (need.num_kv_heads, need.head_dim, need.planes) == (m["kv_heads"], m["dim"] + m["vdim"], 1)
        assert need.window == (m["mask"]["size"] if m.get("mask") else None)
        assert bool(need.chunked) == (CFG["layers"][layer]["type"] == "attention_2" and bool(m.get("mask")))
    assert architecture_of(typed.to_dict()).parse(typed.to_dict()) == typed
    assert model.capturable
    for loop, want in (({"start": 0, "stop": 5, "times": 2}, [0, 1, 2, 3, 4] * 2), ({"start": 2, "stop": 2, "times": 4}, [0, 1, 2, 3, 4]),
                       ({"start": 4, "stop": 5, "times": 1}, [0, 1, 2, 3, 4]), (None, [0, 1, 2, 3, 4])):
        cfg = dict(CFG, loop=loop) if loop else {k: v for k, v in CFG.items() if k != "loop"}
        assert list(_build(cfg)[1].order) == plain.run_order(cfg) == want


def test_what_the_two_mixers_ask_of_the_attention_part():
    _typed, spec, _model = _build(CFG)
    first, second = spec.layers[1].mixer, spec.layers[0].mixer
    assert first.kind == second.kind == "window_attention" and first.bias and second.bias
    assert (first.sink, first.distance_bias, first.q_temp, first.get("chunked", False), first.qk_norm) == ("learned", 8.0, (0.5, 4), False, "none")
    assert first.position.kind == "none"
    assert (second.sink, second.get("distance_bias"), second.get("q_temp"), second.chunked, second.qk_norm, second.norm_first) == \
        ("zero", None, None, True, "gain", True)
    assert (second.position.kind, second.position.theta, second.position.rotary_dim) == ("rope_half", 1000.0, 8)
    assert spec.layers[2].mixer.position.kind == "none" and spec.layers[2].feed_forward.kind == "none"
    assert spec.layers[3].mixer.get("q_temp") is None and not spec.layers[3].mixer.get("window")
    assert spec.residual_streams == 3 and spec.layers[0].block.kind == "hyper_prenorm"
    plain_sum = _build({k: v for k, v in CFG.items() if k != "streams"})[1]
    assert plain_sum.residual_streams == 0 and plain_sum.layers[0].block.kind == "prenorm"


@pytest.mark.parametrize("path,value,message", [
    (("layers", 0, "type"), "attention_3", "type"),
    (("layers", 1, "mixer", "heads"), 3, "multiple of kv_heads"),
    (("layers", 0, "mixer", "rot", "dims"), 7, "even"),
    (("layers", 0, "mixer", "rot", "dims"), 18, "at most dim"),
    (("layers", 0, "mixer", "q_temp"), {"coef": 1.0, "every": 2}, "no query temperature"),
    (("layers", 1, "mixer", "rot"), {"base": 10.0, "dims": 4}, "no rotation"),
    (("layers", 1, "mixer", "q_temp", "every"), 0, "positive"),
    (("layers", 1, "mixer", "mask", "size"), 0, "positive"),
    (("layers", 0, "mlp", "kind"), "moe", "dense"),
    (("norm", "eps"), 0.0, "positive"),
    (("streams",), 17, "at most"),
    (("loop", "stop"), 6, "does not fit"),
    (("loop", "times"), 0, "does not fit"),
])
def test_refusals(path, value, message):
    cfg = copy.deepcopy(CFG)
    node = cfg
    for key in path[:-1]:
        node = node[key]
    node[path[-1]] = value
    with pytest.raises(ConfigError, match=message):
        architecture_of(cfg).parse(cfg)


def test_pages_before_a_chunk_and_behind_a_window_are_given_back():
    needs = _build(CFG)[2].cache_needs()
    groups = group_runs(needs)
    page = 4
    mgr = CacheManager(groups, page, 128, 2)
    kinds = {}
    for i, g in enumerate(groups):
        kinds[(g.window, bool(getattr(g, "chunked", False)))] = i
    assert set(kinds) == {(8, True), (12, True), (10, False), (None, False)}
    mgr.admit("a")
    total = 0
    for n in (5, 2, 30, 1, 1, 9, 3, 1):
        assert mgr.allocate("a", n)
        mgr.commit("a", n)
        total += n
        for (size, chunked), g in kinds.items():
            for idx, p in enumerate(mgr.block_table("a", g)):
                first, last = idx * page, idx * page + page - 1
                if size is None:
                    needed = True
                elif chunked:                       # the next query, at ``total``, sees its own chunk only
                    needed = last >= total // size * size
                else:
                    needed = last >= total - size + 1
                if first > total:
                    continue
                assert (p >= 0) == needed, f"mask {size} (chunks: {chunked}): page {idx} after {total} tokens"
        mgr.check()
    mgr.release("a")
    assert all(pool.num_free == 128 for pool in mgr.pools)


# ---- the plain implementation against itself ------------------------------------------------------------------------------
def test_masks_at_their_edges():
    i = torch.tensor(20)
    assert [bool(plain.sees_sliding(i, torch.tensor(j), 5)) for j in (15, 16, 20, 21)] == [False, True, True, False]
    assert [bool(plain.sees_chunk(i, torch.tensor(j), 5)) for j in (19, 20, 21)] == [False, True, False]
    assert [bool(plain.sees_chunk(torch.tensor(24), torch.tensor(j), 5)) for j in (19, 20, 24)] == [False, True, True]
    assert bool(plain.sees_sliding(i, torch.tensor(0), None)) and bool(plain.sees_chunk(i, torch.tensor(0), None))
    assert plain.query_temperature(2, 0.5, 4) == 1.0 and plain.query_temperature(3, 0.5, 4) == 1.0 + 0.5 * math.log(2)
    assert plain.distance_slopes(4) == [0.25, 0.0625, 0.015625, 0.00390625]


def test_a_sink_takes_its_share_of_the_plain_softmax():
    T, H, d, dv = 6, 2, 4, 3
    g = torch.Generator().manual_seed(0)
    k, v = torch.randn(T, 1, d, generator=g).double(), torch.randn(T, 1, dv, generator=g).double()
    q = torch.zeros(T, H, d, dtype=torch.float64)
    sinks = torch.tensor([1.5, -2.0], dtype=torch.float64)
    out = plain.attend(q, k, v, 0.7, plain.sees_sliding, None, sinks=sinks).view(T, H, dv)
    for t in range(T):
        for h in range(H):
            want = v[:t + 1, 0].sum(0) / (t + 1 + math.exp(float(sinks[h])))
            assert torch.allclose(out[t, h], want, atol=1e-12)
    none = plain.attend(q, k, v, 0.7, plain.sees_sliding, None).view(T, H, dv)
    assert torch.allclose(none[3, 0], v[:4, 0].mean(0), atol=1e-12)


def test_the_plain_model_token_by_token():
    """A prefix's logits do not change when tokens follow (the design is causal), so greedy decoding by recomputation is
    decoding; and the residual after every run comes back once per run."""
    cfg = CFG
    w = {k: v.double() for k, v in plain.random_model(cfg, 3).items()}
    toks = [int(t) for t in torch.randint(0, cfg["vocab"], (30,), generator=torch.Generator().manual_seed(1))]
    taps = []
    whole = plain.forward(cfg, w, toks, taps=taps)
    assert len(taps) == 9 and taps[0].shape == (30, cfg["width"])
    for n in (1, 2, 9, 17):
        assert torch.allclose(plain.forward(cfg, w, toks[:n]), whole[:n], atol=1e-9)
    out = plain.greedy(cfg, w, toks[:5], 3)
    assert len(out) == 3 and out[0] == int(torch.argmax(plain.forward(cfg, w, toks[:5])[-1]))
