"""Zinunex without a GPU: configuration, tensor names, rotation laws, which cache each layer keeps or reads, and the
plain implementation against itself."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_zinunex as plain
from cuinfer_b200.cache.manager import CacheManager, group_runs
from cuinfer_b200.config import ConfigError
from cuinfer_b200.config.registry import get_architecture
from cuinfer_b200.parts.model import DecoderModel
from cuinfer_b200.parts.position import RotaryHalf, RotaryInterleaved
from cuinfer_b200.parts.spec import PartSpec

RAMP = {"base": 500.0, "dims": 6, "scaling": {"factor": 4.0, "original": 64, "fast": 8.0, "slow": 1.0}}


def _moe(experts, top, ff, scale=1.0, groups=1, keep=1, shared=0):
    f = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
         "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


CONFIG = {"architecture": "Zinunex", "vocab": 97, "width": 72, "norm": {"eps": 1e-5}, "token_side": {"dim": 10}, "layers": [
    {"type": "latent_attention", "mixer": {"heads": 3, "dim": 12, "rot_dim": 6, "vdim": 10, "kv_rank": 20, "scale": 0.3,
                                           "mask": {"size": 9}, "rot": RAMP}, "mlp": _moe(6, 2, 36, 1.5, 3, 2, shared=24)},
    {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 12, "vdim": 12, "scale": 0.4,
                                    "rot": {"base": 100.0, "dims": 8, "scaling": {"factor": 2.0}}}, "mlp": _moe(5, 2, 20)},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 6, "vdim": 14, "kv_rank": 20, "scale": 0.35,
                                           "mask": {"size": 17}, "rot": RAMP, "kv_from": 0}, "mlp": None},
    {"type": "latent_attention", "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 6, "kv_rank": 12, "scale": 0.35,
                                           "mask": {"size": 5}, "rot": {"base": 50.0, "dims": 4}}, "mlp": _moe(4, 4, 28, 0.5, 2, 2, shared=16)},
]}


def _build(cfg):
    arch = get_architecture("Zinunex")
    typed = arch.parse(cfg)
    return typed, DecoderModel(arch.spec(typed), torch.float32)


def test_tensor_names_and_shapes_are_the_plain_models():
    typed, model = _build(CONFIG)
    want = {k: tuple(v.shape) for k, v in plain.random_model(CONFIG, 0).items()}
    got = {t.name: tuple(t.shape) for t in model.tensors()}
    assert got == want
    assert "l2.mix.dkv" not in got and "l2.mix.dkv.norm" not in got, "a layer that reads another's cache has no down-projection"
    assert typed.to_dict() == CONFIG


def test_a_read_cache_keeps_what_its_widest_reader_sees():
    _, model = _build(CONFIG)
    needs = model.cache_needs()
    assert sorted(needs) == [0, 1, 3] and model.cache_source == {2: 0}
    assert needs[0].window == 17 and (needs[0].head_dim, needs[0].planes, needs[0].num_kv_heads) == (26, 1, 1)
    assert needs[1].window is None and (needs[1].head_dim, needs[1].num_kv_heads, needs[1].planes) == (24, 2, 1)
    assert needs[3].window == 5
    # a reader without a window keeps everything; a reader with a shorter window changes nothing
    for size, want in ((None, None), (4, 9)):
        cfg = copy.deepcopy(CONFIG)
        if size is None:
            del cfg["layers"][2]["mixer"]["mask"]
        else:
            cfg["layers"][2]["mixer"]["mask"]["size"] = size
        assert _build(cfg)[1].cache_needs()[0].window == want
    # pages behind the widened window are given back, those inside it are not
    groups = group_runs(needs)
    manager = CacheManager(groups, 4, 64, 2)
    g0 = [i for i, g in enumerate(groups) if 0 in g.runs][0]
    manager.admit("a")
    assert manager.allocate("a", 40)
    manager.commit("a", 40)
    table = manager.block_table("a", g0)
    assert table[:6] == [-1] * 6 and all(p >= 0 for p in table[6:]), "the next query at 40 sees keys from 24 on"


def test_rotation_laws():
    def part(cls, kind, **kw):
        return cls(PartSpec(kind, **kw), hidden_size=1, prefix="", dtype=torch.float32)

    for base, dims, factor, original, fast, slow in ((500.0, 6, 4.0, 64, 8.0, 1.0), (1e6, 32, 40.0, 4096, 32.0, 1.0), (50.0, 2, 2.0, 16, 4.0, 0.5),
                                                     (1e4, 64, 8.0, 128, 1.0, 1.0)):
        p = part(RotaryInterleaved, "rope_interleaved", theta=base, rotary_dim=dims,
                 scaling={"kind": "ramp", "factor": factor, "original": original, "fast": fast, "slow": slow})
        freqs, mag = plain.ramp_frequencies(base, dims, factor, original, fast, slow)
        assert torch.allclose(p.host_frequencies().double(), torch.tensor(freqs, dtype=torch.float64), rtol=1e-6, atol=0)
        assert abs(p.magnitude - mag) < 1e-12 and abs(mag - (0.1 * math.log(factor) + 1)) < 1e-12
    p = part(RotaryHalf, "rope_half", theta=100.0, rotary_dim=8, scaling={"kind": "linear", "factor": 2.0})
    assert torch.allclose(p.host_frequencies().double(), torch.tensor(plain.linear_frequencies(100.0, 8, 2.0), dtype=torch.float64), rtol=1e-6, atol=0)
    assert p.magnitude == 1.0 and p.layout == "half"
    # the ramp really blends: the fastest pair keeps its frequency, the slowest is divided by the factor
    freqs, _ = plain.ramp_frequencies(1e4, 64, 8.0, 128, 4.0, 0.25)
    plain_f = plain.plain_frequencies(1e4, 64)
    assert freqs[0] == plain_f[0] and abs(freqs[-1] - plain_f[-1] / 8.0) < 1e-15 and any(plain_f[i] / 8 < f < plain_f[i] for i, f in enumerate(freqs))
    with pytest.raises(ValueError):
        part(RotaryHalf, "rope_half", theta=100.0, rotary_dim=8, scaling={"kind": "other", "factor": 2.0})


def test_what_each_layer_asks_of_the_parts():
    typed, _ = _build(CONFIG)
    spec = get_architecture("Zinunex").spec(typed)
    first, second, third = (spec.layers[i].mixer for i in range(3))
    assert first.kind == "latent_attention" and first.own_cache and first.window == 9 and not first.q_rank and first.scale == 0.3
    assert first.position.kind == "rope_interleaved" and first.position.scaling["kind"] == "ramp"
    assert third.own_cache is False and third.window == 17
    assert second.kind == "window_attention" and second.value_from_key and second.sink == "learned" and second.qk_norm == "none"
    assert second.position.kind == "rope_half" and second.position.scaling == {"factor": 2.0, "kind": "linear"}
    ff = spec.layers[0].feed_forward
    assert (ff.kind, ff.score, ff.activation, ff.groups, ff.route_scale, ff.shared_size) == ("moe_routed", "sigmoid", "relu2", (3, 2), 1.5, 24)
    assert spec.layers[2].feed_forward.kind == "none" and spec.layers[1].feed_forward.shared_size == 0
    assert spec.layers[3].block.after.kind == "token_side" and spec.layers[3].block.after.index == 3


@pytest.mark.parametrize("change,message", [
    (lambda c: c["layers"][2]["mixer"].update(kv_from=1), "earlier latent_attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_from=2), "earlier latent_attention layer"),
    (lambda c: c["layers"][2]["mixer"].update(kv_rank=24), "must equal those of layer 0"),
    (lambda c: c["layers"][2]["mixer"].update(rot=dict(RAMP, base=501.0)), "must equal those of layer 0"),
    (lambda c: c["layers"][1]["mixer"].update(vdim=16), "the values are the keys"),
    (lambda c: c["layers"][1]["mixer"].update(kv_heads=3), "not a multiple"),
    (lambda c: c["layers"][0]["mlp"]["router"]["groups"].update(count=4), "groups"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=5), "cannot give"),
    (lambda c: c["layers"][0].update(type="mamba"), "unsupported option"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "unsupported option"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=8), "exceeds rot_dim"),
    (lambda c: c["layers"][0]["mixer"]["rot"]["scaling"].pop("slow"), "slow"),
    (lambda c: c.pop("norm"), "norm"),
])
def test_refusals(change, message):
    cfg = copy.deepcopy(CONFIG)
    change(cfg)
    with pytest.raises(ConfigError, match=message):
        _build(cfg)


def test_plain_model_token_by_token_equals_whole():
    """The plain implementation against itself: the logits of a prefix do not depend on what follows."""
    w = {k: v.double() for k, v in plain.random_model(CONFIG, 3).items()}
    toks = torch.randint(0, 97, (40,), generator=torch.Generator().manual_seed(1)).tolist()
    whole = plain.forward(CONFIG, w, toks)
    for n in (1, 9, 10, 18, 33):
        assert torch.allclose(plain.forward(CONFIG, w, toks[:n])[-1], whole[n - 1], atol=1e-9)
    assert plain.router_margin(CONFIG, w, toks) > 0.02


def test_plain_choice_of_experts():
    z = torch.tensor([2.0, -1.0, 0.5, 0.4, -3.0, 3.0], dtype=torch.float64)
    none = torch.zeros(6, dtype=torch.float64)
    # three groups of two; marks are the sums of both members: group 2 (experts 4, 5) loses to groups 0 and 1
    chosen, scores = plain.choose_experts(z, none, 2, 3, 2)
    assert chosen == [0, 2] and abs(float(scores[0]) - 1 / (1 + math.exp(-2.0))) < 1e-12
    # a correction changes the choice, not the weights; choice scores below zero still beat a masked expert
    corr = torch.tensor([-5.0, -5.0, -5.0, -5.0, -9.0, -9.0], dtype=torch.float64)
    chosen, scores = plain.choose_experts(z, corr, 2, 3, 1)
    assert chosen == [2, 3] and abs(float(scores[1]) - 1 / (1 + math.exp(-0.4))) < 1e-12
    margins = plain.choice_margins(z[None], none, 2, 3, 2)
    assert 0 < float(margins[0]) < 0.2
