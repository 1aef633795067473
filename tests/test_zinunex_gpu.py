"""Zinunex through the engine against the plain implementation (``plain_zinunex``), mechanism by mechanism and as a
whole: every way of cutting the work, pages and slots that are used again, keys far away, at page borders and just
inside and just outside the window, a latent cache read by a later layer with a longer or shorter window, the sink, the
router's groups and correction, sizes that are odd, equal to one or absent, and greedy generation through the entry point
and the scheduler.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import pytest
import torch

import plain_zinunex as plain
import traces
from conftest import note_error, random_tokens

pytestmark = pytest.mark.gpu


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, window=None, rot=None, kv_from=None, mlp=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = rot
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m, "mlp": mlp}


def _sink(heads, kv_heads, dim, scale, rot=None, mlp=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale}
    if rot:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp}


def _moe(experts, top, ff, scale=1.0, groups=1, keep=1, shared=0):
    f = {"kind": "moe", "router": {"experts": experts, "top": top, "scale": scale, "groups": {"count": groups, "keep": keep}},
         "expert": {"ff": ff}}
    if shared:
        f["shared"] = {"ff": shared}
    return f


def _config(vocab, width, layers, side=None, eps=1e-6):
    cfg = {"architecture": "Zinunex", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if side:
        cfg["token_side"] = {"dim": side}
    return cfg


def _ramp(base, dims, factor, original, fast, slow):
    return {"base": base, "dims": dims, "scaling": {"factor": factor, "original": original, "fast": fast, "slow": slow}}


# odd sizes everywhere; the third layer reads the first one's cached latent with a LONGER window than the first has (the
# cache must keep what the reader sees) and has no feed-forward; one key/value head; as many experts chosen as there are;
# part of a head rotated
ODD = _config(97, 72, [
    _latent(3, 12, 6, 10, 20, 0.3, window=9, rot=_ramp(500.0, 6, 4.0, 64, 8.0, 1.0), mlp=_moe(6, 2, 36, 1.5, 3, 2, shared=24)),
    _sink(4, 2, 12, 0.4, rot={"base": 100.0, "dims": 8, "scaling": {"factor": 2.0}}, mlp=_moe(5, 2, 20)),
    _latent(2, 8, 6, 14, 20, 0.35, window=17, rot=_ramp(500.0, 6, 4.0, 64, 8.0, 1.0), kv_from=0, mlp=None),
    _sink(3, 1, 20, 0.3, rot={"base": 3000.0, "dims": 20}, mlp=_moe(4, 4, 28, 0.5, 2, 2, shared=16)),
], side=10, eps=1e-5)
# the other mixer first; a latent layer without a window read by one with a window; groups of one expert; one expert
# per token; no per-layer token input; no scaling of the latent layers' rotation; part of the rotated key part rotated;
# pages of 32
LATE = _config(300, 128, [
    _sink(2, 2, 32, 0.25, rot={"base": 10000.0, "dims": 32, "scaling": {"factor": 16.0}}, mlp=_moe(6, 1, 64, 2.5, 6, 2)),
    _latent(4, 16, 8, 24, 40, 0.2, window=None, rot={"base": 10000.0, "dims": 4}, mlp=_moe(4, 2, 32, 1.0, 2, 1, shared=64)),
    _latent(1, 32, 8, 8, 40, 0.2, window=33, rot={"base": 10000.0, "dims": 4}, kv_from=1, mlp=_moe(3, 1, 48, 1.0, 1, 1, shared=8)),
])
# sizes in multiples of 16 and 64, for the tensor-core paths in bfloat16 (latent attention with a window, attention with
# a sink, grouped experts, tcgen05 projections); windows that start inside key tiles; a reader with a shorter window
WIDE = _config(768, 384, [
    _latent(6, 64, 32, 64, 96, 0.11, window=70, rot=_ramp(1e5, 32, 16.0, 256, 16.0, 2.0), mlp=_moe(6, 2, 128, 2.0, 3, 2, shared=192)),
    _sink(8, 2, 64, 0.14, rot={"base": 5e5, "dims": 32, "scaling": {"factor": 4.0}}, mlp=_moe(8, 3, 64, 1.5, 4, 2, shared=64)),
    _latent(12, 32, 32, 32, 96, 0.12, window=33, rot=_ramp(1e5, 32, 16.0, 256, 16.0, 2.0), kv_from=0, mlp=_moe(4, 2, 96, 1.0, 1, 1)),
    _sink(4, 4, 128, 0.1, rot={"base": 1e4, "dims": 128, "scaling": {"factor": 2.0}}, mlp=_moe(6, 2, 64, 1.0, 2, 1, shared=128)),
], side=16)
MODELS = {"odd": (ODD, 16, 31), "late": (LATE, 32, 32), "wide": (WIDE, 16, 33)}

# Largest error of a row of logits (see _row_error).  float32: only the order of sums differs.  bfloat16: the engine
# rounds where it stores (normed rows, projections, cached rows, mixer outputs, activations).
# float32 at a thousand tokens: the engine takes position times frequency in 32 bits, as the design says, the plain model
# in 64; at an angle of a thousand radians that is 3e-5 of a turn
TOLERANCE = {"float32": 2e-5, "bfloat16": 5e-2}
# Between two ways of cutting the same request the engine may differ only by which kernel a step's size selects.
CUT_TOLERANCE = {"float32": 2e-6, "bfloat16": 5e-2}
MARGIN = 0.02          # what the routers of the test models must leave (see plain.choice_margins)


def _write(folder, cfg, tensors, dtype):
    from cuinfer_b200.weights.safetensors_io import write_safetensors

    os.makedirs(folder, exist_ok=True)
    store = {k: v.to(torch.bfloat16 if dtype == "bfloat16" else torch.float32) for k, v in tensors.items()}
    write_safetensors(os.path.join(folder, "model.safetensors"), store)
    with open(os.path.join(folder, "config.json"), "w") as fh:
        json.dump(cfg, fh)
    return folder


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    """{name: (config, {dtype: folder}, tensors in float64, page size)}; the values are bfloat16 numbers, so that both
    engines and the plain implementation read the same weights."""
    out = {}
    for name, (cfg, block, seed) in MODELS.items():
        tensors = plain.random_model(cfg, seed)
        dirs = {d: _write(str(tmp_path_factory.mktemp(f"zinunex_{name}_{d}")), cfg, tensors, d) for d in TOLERANCE}
        out[name] = (cfg, dirs, {k: v.double() for k, v in tensors.items()}, block)
    return out


def _row_error(row, ref):
    """Root mean square of the difference over the vocabulary, the common offset taken off (it changes no probability),
    as a fraction of the root mean square of the plain logits about their mean."""
    d = row.astype(np.float64) - ref
    return float(np.sqrt(((d - d.mean()) ** 2).mean()) / np.sqrt(((ref - ref.mean()) ** 2).mean()))


def _requests(cfg, lengths, seed):
    return {f"r{i}": random_tokens(cfg["vocab"], n, seed * 100 + i) for i, n in enumerate(lengths)}


_WHOLE = {}


def _whole_rows(folders, name, dtype, rid, toks, tmp_path):
    """The engine's own logits of a request fed whole and alone."""
    key = (name, dtype, tuple(toks))
    if key not in _WHOLE:
        cfg, dirs, _tensors, block = folders[name]
        steps = traces.whole({rid: toks})
        out = str(tmp_path / f"whole_{name}_{dtype}_{rid}")
        traces.replay_in_process(dirs[dtype], dtype, steps, out, traces.live_token_peak(steps), block)
        _WHOLE[key] = traces.collect(steps, out, cfg["vocab"])[rid]
    return _WHOLE[key]


def _check(folders, name, dtype, steps, requests, tmp_path, max_tokens=None, **kw):
    """Every row against the plain implementation, and against the engine's own logits of the request fed whole."""
    cfg, dirs, tensors, block = folders[name]
    out = str(tmp_path / f"out_{name}_{dtype}")
    runner = traces.replay_in_process(dirs[dtype], dtype, steps, out, max_tokens or traces.live_token_peak(steps), block, **kw)
    got = traces.collect(steps, out, cfg["vocab"])
    worst = 0.0
    for rid, toks in requests.items():
        assert plain.router_margin(cfg, tensors, list(toks)) > MARGIN, "the test's routers must not rest on a close call"
        ref = plain.forward(cfg, tensors, list(toks)).numpy()
        assert got.get(rid), f"no logits came back for request {rid}"
        assert sorted(got[rid]) == list(range(len(toks)))
        whole = _whole_rows(folders, name, dtype, rid, list(toks), tmp_path)
        for pos, row in sorted(got[rid].items()):
            assert np.isfinite(row).all(), f"request {rid} position {pos}: logits are not finite"
            cut = _row_error(row, whole[pos].astype(np.float64))
            assert cut <= CUT_TOLERANCE[dtype], f"{name}/{dtype}: request {rid}: position {pos} of {len(toks)} depends on how the work was cut ({cut:.3e})"
            err = _row_error(row, ref[pos])
            assert err <= TOLERANCE[dtype], f"{name}/{dtype}: request {rid}: first wrong position {pos} of {len(toks)} (error {err:.3e})"
            worst = max(worst, err)
    note_error(dtype, f"model {name}", worst, family="Zinunex")
    return runner


NAMES, DTYPES = list(MODELS), list(TOLERANCE)


# ---- the whole model under every way of cutting the work ------------------------------------------------------------
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [1, 2, 17, 33, 150], seed=1)
    _check(folders, name, dtype, traces.whole(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prefill_then_token_by_token(folders, name, dtype, tmp_path):
    """The decoded tail is longer than every window, so windows pass over decoded tokens and pages are given back."""
    requests = _requests(folders[name][0], [40, 131], seed=2)
    _check(folders, name, dtype, traces.tail_decode(requests, 80), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_portions_down_to_two_tokens(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [64, 131, 90], seed=3)
    _check(folders, name, dtype, traces.portions(requests), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_mixed_batches_reuse_pages_and_slots(folders, name, dtype, tmp_path):
    requests = _requests(folders[name][0], [70, 33, 120, 58, 90, 45, 101], seed=4)
    steps = traces.mixed(requests, max_live=4)
    peak = traces.live_token_peak(steps)
    assert peak < sum((len(t) + 63) // 64 * 64 for t in requests.values()), "pages must be used again"
    runner = _check(folders, name, dtype, steps, requests, tmp_path, max_tokens=peak, max_live=4)
    assert runner.num_pages * runner.page_size == peak and runner.manager.slots.num_slots == 4


@pytest.mark.parametrize("dtype", DTYPES)
def test_long_decoding_from_the_first_token(folders, dtype, tmp_path):
    requests = _requests(folders["odd"][0], [260], seed=5)
    _check(folders, "odd", dtype, traces.tail_decode(requests, 259), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["odd", "wide"])
def test_a_long_prompt_then_decoding(folders, name, dtype, tmp_path):
    """More than a thousand tokens: keys far behind every window, many pages given back and many key tiles a query;
    most of it in one step, then 40 tokens one by one; and a second request cut into portions throughout."""
    cfg = folders[name][0]
    requests = _requests(cfg, [1100], seed=9)
    _check(folders, name, dtype, traces.tail_decode(requests, 40), requests, tmp_path)
    requests = _requests(cfg, [700], seed=10)
    _check(folders, name, dtype, traces.portions(requests, sizes=(130, 2, 64, 3, 257, 16)), requests, tmp_path)


@pytest.mark.parametrize("dtype", DTYPES)
def test_steps_through_cuda_graphs(folders, dtype, tmp_path):
    """The same logits when decode steps and repeated step shapes are replayed from graphs, as generation runs them:
    padding rows and the padding request own no slot and no page."""
    requests = _requests(folders["wide"][0], [70, 40, 90, 33], seed=6)
    steps = traces.mixed(requests, max_live=3, sizes=(32, 40, 35))
    runner = _check(folders, "wide", dtype, steps, requests, tmp_path, cuda_graph=True, passes=2, max_live=4)
    assert runner.model.capturable and runner.graph_steps + runner.step_graph_replays > 0


@pytest.mark.parametrize("graphs", [False, True])
def test_many_requests_decoding_together(folders, graphs, tmp_path):
    """Thirteen requests decode side by side: enough (request, key head) pairs for the layer with heads of 128 to take
    the tcgen05 kernel in steps of single tokens too, eagerly and from a decode graph whose bucket has padding rows."""
    cfg = folders["wide"][0]
    requests = _requests(cfg, [20 + 3 * i for i in range(13)], seed=8)
    heads = {rid: len(t) - 6 for rid, t in requests.items()}
    steps = [{"step": 0, "entries": [{"id": rid, "tokens": t[:heads[rid]], "want": list(range(heads[rid]))} for rid, t in requests.items()], "end": []}]
    for k in range(6):
        steps.append({"step": k + 1, "entries": [{"id": rid, "tokens": [t[heads[rid] + k]], "want": [0]} for rid, t in requests.items()],
                      "end": list(requests) if k == 5 else []})
    runner = _check(folders, "wide", "bfloat16", steps, requests, tmp_path, cuda_graph=graphs, passes=2 if graphs else 1, max_live=16)
    assert not graphs or runner.graph_steps > 0


def test_the_stream_after_every_layer(folders):
    """The residual stream after each layer of a short prompt, in 32 bits, against the plain model's."""
    from cuinfer_b200.engine import replay
    from cuinfer_b200.engine.runner import StepEntry

    for name in NAMES:
        cfg, dirs, tensors, block = folders[name]
        toks = random_tokens(cfg["vocab"], 29, 77)
        want = []
        plain.forward(cfg, tensors, toks, tap=lambda i, x: want.append(x.clone()))
        runner = replay.make_runner(dirs["float32"], "float32", 64, block)
        entries = [StepEntry("a", toks, [0])]
        assert runner.reserve("a", len(toks))
        runner.storage.zero_slots(runner.manager.take_newly_admitted())
        ctx, _ = runner.build_context(entries)
        got = []
        runner.model.forward(ctx, tap=lambda run, stream: got.append(stream.collapsed().double().cpu()))
        assert len(got) == len(want) == len(cfg["layers"])
        for i, (g, w) in enumerate(zip(got, want)):
            err = float((g - w).abs().max() / w.abs().max())
            assert err < 2e-5, f"{name}: the stream after layer {i} is off by {err:.3e}"


def test_greedy_generation_through_the_entry_point(folders):
    from cuinfer_b200 import LLM, SamplingParams

    for name in ("odd", "late"):
        cfg, dirs, tensors, block = folders[name]
        prompts = [random_tokens(cfg["vocab"], n, 70 + n) for n in (3, 19, 8)]
        llm = LLM(dirs["float32"], dtype="float32", block_size=block, num_blocks=24, max_num_seqs=3, max_num_scheduled_tokens=16)
        outs = llm.generate(prompts, SamplingParams(max_tokens=12, temperature=0.0, ignore_eos=True))
        for prompt, out in zip(prompts, outs):
            assert out.token_ids == plain.greedy(cfg, tensors, prompt, 12), f"{name}: prompt of {len(prompt)} tokens"


def test_command_line(folders):
    import subprocess
    import sys

    from conftest import ROOT

    cfg, dirs, tensors, block = folders["late"]
    prompt = random_tokens(cfg["vocab"], 9, 95)
    proc = subprocess.run([sys.executable, "-m", "cuinfer_b200", "generate", "--model", dirs["float32"], "--dtype", "float32",
                           "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--ignore-eos",
                           "--num-blocks", "16", "--max-num-seqs", "4", "--block-size", str(block)],
                          capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")][0]
    assert line["token_ids"] == plain.greedy(cfg, tensors, prompt, 5)


# ---- mechanisms alone -------------------------------------------------------------------------------------------------
def _dev(t, dtype):
    return t.to(device="cuda", dtype=dtype).contiguous()


def _close(got, want, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype == torch.float32 else 2e-2)
    err = float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-9))
    assert err <= tol, f"{what} in {dtype}: error {err:.3e} of the largest value"


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


def _angles32(position, freqs):
    """The design takes the angle in 32 bits: position times frequency, both float32.  The plain rotation gets those
    angles as "frequencies" at "position" one."""
    return (torch.tensor(float(position), dtype=torch.float32) * torch.tensor(freqs, dtype=torch.float32)).double().tolist()


def _rotated(x, positions, freqs, layout, magnitude=1.0):
    out = torch.empty_like(x)
    for t in range(x.shape[0]):
        out[t] = plain.rotate(x[t:t + 1], torch.ones(1), _angles32(positions[t], freqs), layout, magnitude)[0]
    return out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_norm_scaled_rotation_and_cache_write(dtype):
    """Rows [queries | latent | rotated key part] without a query latent: the latent's RMS norm and the key part's
    rotation under the ramp law (cosine and sine times its magnitude) land in the token's cache row; queries stay."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(3)
    T, qcols, rk, dr, dims, page = 9, 14, 12, 8, 6, 4
    proj = torch.randn(T, qcols + rk + dr + 3, generator=g).to(dtype).double()
    kg = (1 + 0.3 * torch.randn(rk, generator=g)).bfloat16().double()
    positions = [0, 1, 2, 3, 1000, 1001, 70000, 5, 6]
    slots = [7, 2, 3, -1, 0, 1, 11, 10, 5]
    freqs, mag = plain.ramp_frequencies(250.0, dims, 5.0, 48, 6.0, 0.5)
    assert mag > 1.1 and len({round(f * 250.0 ** (2 * i / dims), 6) for i, f in enumerate(freqs)}) > 1, "the ramp must do something"
    cache = torch.zeros(3, 1, 1, page, rk + dr, dtype=dtype, device="cuda")
    dev = _dev(proj, dtype)
    before = dev.clone()
    kernels.latent_prep(dev, 0, 0, qcols, rk, dr, None, _dev(kg, torch.float32), 1e-5, _ints(positions),
                        torch.tensor(freqs, dtype=torch.float32).cuda(), dims, _ints(slots), cache, None, rot_gain=mag)
    assert torch.equal(dev, before)
    c = plain.rms(proj[:, qcols:qcols + rk], 1e-5) * kg
    kr = _rotated(proj[:, qcols + rk:qcols + rk + dr].reshape(T, 1, dr), positions, freqs, "neighbours", mag).reshape(T, dr)
    flat = cache.view(-1, rk + dr)
    for t in range(T):
        if slots[t] < 0:
            continue
        _close(flat[slots[t], :rk], c[t], dtype, f"latent of token {t}")
        _close(flat[slots[t], rk:], kr[t], dtype, f"rotated key part of token {t} at position {positions[t]}")
    assert float(flat[[4, 6, 8, 9]].abs().max()) == 0.0, "a token without slot wrote somewhere"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("d,dims", [(10, 6), (64, 64), (24, 0), (128, 32)])
def test_rotation_in_halves_and_values_that_are_the_keys(dtype, d, dims):
    """Rows [q | k] only: queries and keys rotated in halves at frequencies divided by one factor; the cached value is
    the key as projected, before the rotation."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(d)
    T, H, G, page = 9, 4, 2, 4
    rows = torch.randn(T, (H + G) * d + 5, generator=g).to(dtype).double()
    positions = [0, 1, 2, 3, 1000, 1001, 70000, 5, 6]
    slots = [7, 2, 3, -1, 0, 1, 11, 10, 5]
    freqs = plain.linear_frequencies(250.0, dims, 3.0) if dims else []
    cache = torch.zeros(3, 1, G, page, 2 * d, dtype=dtype, device="cuda")
    dev = _dev(rows, dtype)
    kernels.window_attention_prep(dev, _ints(positions), _ints(slots), torch.tensor(freqs, dtype=torch.float32).cuda() if dims else None,
                                  dims, 1e-5, H, G, d, d, None, None, cache, norm=False, rot_half=True, value_from_key=True)
    q = _rotated(rows[:, :H * d].view(T, H, d), positions, freqs, "halves")
    k_plain = rows[:, H * d:(H + G) * d].view(T, G, d)
    k = _rotated(k_plain, positions, freqs, "halves")
    _close(dev[:, :H * d].view(T, H, d), q, dtype, "queries")
    assert torch.equal(dev[:, H * d:].double().cpu(), rows[:, H * d:]), "keys in the rows and the columns after them stay"
    for t in range(T):
        if slots[t] < 0:
            continue
        got = cache[slots[t] // page, 0, :, slots[t] % page]
        _close(got[:, :d], k[t], dtype, f"key of token {t} at position {positions[t]}")
        assert torch.equal(got[:, d:].double().cpu(), k_plain[t]), f"the value of token {t} is its key before the rotation"
    flat = cache.permute(0, 3, 1, 2, 4).reshape(-1, G, 2 * d)
    assert float(flat[[4, 6, 8, 9]].abs().max()) == 0.0, "a token without slot wrote somewhere"


def _paged(g, lengths, page, heads, width, dtype, spare=3):
    """A cache ``[pages, 1, heads, page, width]`` of random rows behind block tables in a shuffled order."""
    pages_per = [-(-n // page) for n in lengths]
    num_pages = sum(pages_per) + spare
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((len(lengths), max(pages_per)), -1, dtype=torch.int32)
    cache = (torch.randn(num_pages, 1, heads, page, width, generator=g) * 0.5).to(dtype)
    rows, at = {}, 0
    for r, n in enumerate(lengths):
        table[r, :pages_per[r]] = torch.tensor(perm[at:at + pages_per[r]], dtype=torch.int32)
        at += pages_per[r]
        rows[r] = torch.stack([cache[int(table[r, j // page]), 0, :, j % page] for j in range(n)]).double()     # [n, heads, width]
    return cache, table, rows


def _layout(lengths, new):
    pos, treq, qsl = [], [], [0]
    for r, (n, k) in enumerate(zip(lengths, new)):
        pos += list(range(n - k, n))
        treq += [r] * k
        qsl.append(qsl[-1] + k)
    return pos, treq, qsl


def _latent_case(dtype, H, dn, dr, rk, dims, lengths, new, page, seed, window, sharpen=None, tensor_cores=False, freed=False):
    """Requests of ``lengths`` tokens whose last ``new`` are this step's queries, over cached rows [latent | key part];
    returns the kernel's output and the plain result [T, H, rk].  ``freed``: the pages wholly behind the window of a
    request's first query are taken from its table, as the cache manager does."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    cache, table, rows = _paged(g, lengths, page, 1, rk + dr, dtype)
    pos, treq, qsl = _layout(lengths, new)
    T = len(pos)
    q_abs = torch.randn(T, H, rk, generator=g).double() * 0.3
    q = (torch.randn(T, H, dn + dr, generator=g) * 0.3).to(dtype).double()
    freqs, mag = plain.ramp_frequencies(1000.0, dims, 4.0, 64, 8.0, 1.0) if dims else ([], 1.0)
    if sharpen is not None:            # make query t's score with key j of its request stand out for every head
        for t, j in sharpen.items():
            key = rows[treq[t]][j, 0]
            q_abs[t] = 6.0 * key[:rk] / key[:rk].norm()
    if tensor_cores:                   # that kernel takes the absorbed queries in bfloat16: both sides get those values
        q_abs = q_abs.bfloat16().double()
    scale = 0.7
    want = torch.zeros(T, H, rk, dtype=torch.float64)
    for t in range(T):
        lo = max(0, pos[t] - window + 1) if window else 0
        keys = rows[treq[t]][lo: pos[t] + 1, 0]
        q_rot = plain.rotate(q[t:t + 1, :, dn:], torch.ones(1), _angles32(pos[t], freqs), "neighbours", mag)[0]      # [H, dr]
        scores = (q_abs[t] @ keys[:, :rk].T + q_rot @ keys[:, rk:].T) * scale
        want[t] = torch.softmax(scores, -1) @ keys[:, :rk]
    if freed and window:
        for r, (n, k) in enumerate(zip(lengths, new)):
            table[r, :max(0, n - k - window + 1) // page] = -1
    freq = torch.tensor(freqs, dtype=torch.float32).cuda() if dims else None
    out = torch.empty(T, H * rk, dtype=dtype, device="cuda")
    if tensor_cores:
        assert kernels.latent_attention_mma_supports(rk, dr, dn)
        kernels.latent_attention_mma(_dev(q_abs.reshape(T, H * rk), dtype), _dev(q.reshape(T, -1), dtype), out, cache.cuda(),
                                     table.cuda(), _ints(qsl), _ints(lengths), list(new), freq, dims, None, H, dn, rk, dr, scale,
                                     max(lengths), decode_only=all(k == 1 for k in new), window=window, rot_gain=mag)
    else:
        kernels.latent_attention_generic(_dev(q_abs.reshape(T, H * rk), torch.float32), _dev(q.reshape(T, -1), dtype), out, cache.cuda(),
                                         table.cuda(), _ints(qsl), _ints(lengths), _ints(treq), _ints(pos), freq, dims, None, H, dn, rk,
                                         dr, scale, window=window, rot_gain=mag)
    return out.view(T, H, rk), want


@pytest.mark.parametrize("tensor_cores,dtype", [(False, torch.float32), (False, torch.bfloat16), (True, torch.bfloat16)])
@pytest.mark.parametrize("decode", [False, True])
def test_latent_window_one_key_stands_out_at_every_edge(tensor_cores, dtype, decode):
    """A key whose score is made to dominate must be seen exactly when it lies in the window: the last key inside and
    the first outside, the first token, both sides of page borders and of key tiles, the query's own key; for a query
    inside a prompt's portion and for a single decoded token; with the pages behind the window given back."""
    page, window, n = 8, 45, 200
    pos = n - 1
    sizes = dict(H=4, dn=8, dr=16, rk=32, dims=16) if tensor_cores else dict(H=3, dn=8, dr=6, rk=20, dims=4)
    for j, seen in [(pos - window + 1, True), (pos - window, False), (pos, True), (pos - 7, True), (pos - 8, True), (160, True),
                    (159, True), (0, False), (7, False), (100, False), (pos - window - 1, False)]:
        assert (0 <= pos - j < window) == seen
        new, t = ([1, 1], 0) if decode else ([70, 3], 69)
        got, want = _latent_case(dtype, lengths=[n, 40], new=new, page=page, seed=7 + j, window=window, sharpen={t: j},
                                 tensor_cores=tensor_cores, freed=True, **sizes)
        _close(got, want, dtype, f"query {pos} with key {j} standing out")
        assert not seen or float(want[t].abs().max()) > 0.2, "the case does not single a key out"


@pytest.mark.parametrize("H, dn, dr, rk, dims, lengths, new, page, window", [
    (3, 8, 16, 32, 8, [37, 1, 64, 129], [37, 1, 1, 5], 8, 20),          # prompts beside single tokens, a window inside a tile
    (5, 16, 16, 160, 16, [50, 33, 200], [2, 33, 100], 16, 64),           # a window of whole tiles
    (16, 8, 64, 512, 64, [300, 90], [170, 1], 16, 97),                   # 512: eight warps, two halves of the value columns
    (1, 8, 16, 48, 16, [130], [130], 32, 1),                             # one head: 64 tokens to a tile; a window of the query alone
    (32, 8, 64, 256, 64, [700, 90, 33], [1, 1, 1], 16, 300),             # a decode step: keys split, a window longer than some contexts
    (6, 8, 16, 64, 16, [70, 1, 200], [1, 1, 1], 16, 33),                 # a decode step with few heads
    (4, 8, 0, 16, 0, [150, 20], [150, 3], 4, 0),                         # no window, nothing rotated
])
def test_latent_window_on_tensor_cores(H, dn, dr, rk, dims, lengths, new, page, window):
    got, want = _latent_case(torch.bfloat16, H, dn, dr, rk, dims, lengths, new, page, seed=H, window=window, tensor_cores=True, freed=True)
    _close(got, want, torch.bfloat16, "tensor-core latent attention with a window")
    got, want = _latent_case(torch.float32, H, dn, dr, rk, dims, lengths, new, page, seed=H, window=window, freed=True)
    _close(got, want, torch.float32, "latent attention with a window")


def _sink_case(dtype, H, G, d, lengths, new, page, seed, sharpen=None, sink=None, tensor_cores=False, splits=1, window=0):
    """Attention over cached rows [key | value] with every earlier key visible (or the last ``window``) and a sink per
    head.  ``tensor_cores``: False (the all-sizes kernel), True (``mma.sync``) or "tcgen05" (key and value size 128)."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    cache, table, rows = _paged(g, lengths, page, G, 2 * d, dtype)
    pos, treq, qsl = _layout(lengths, new)
    T = len(pos)
    q = (torch.randn(T, H, d, generator=g) * 0.4).to(dtype).double()
    if sharpen is not None:
        for t, j in sharpen.items():
            for h in range(H):
                key = rows[treq[t]][j, h // (H // G), :d]
                q[t, h] = (7.0 * key / key.norm()).to(dtype).double()
    sinks = sink if sink is not None else torch.randn(H, generator=g).double()
    scale = 0.8
    want = torch.zeros(T, H, d, dtype=torch.float64)
    for t in range(T):
        kv = rows[treq[t]][max(0, pos[t] - window + 1) if window else 0: pos[t] + 1]
        for h in range(H):
            s = (kv[:, h // (H // G), :d] @ q[t, h]) * scale
            m = torch.maximum(s.max(), sinks[h])
            e = torch.exp(s - m)
            want[t, h] = (e / (e.sum() + torch.exp(sinks[h] - m))) @ kv[:, h // (H // G), d:]
    out = torch.empty(T, H * d, dtype=dtype, device="cuda")
    if tensor_cores == "tcgen05":
        assert kernels.attention_tcgen05_supports(d, H, G, page)
        kernels.attention_tcgen05(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(qsl), _ints(lengths),
                                  list(new), H, G, d, scale, window, joined=True, sinks=_dev(sinks, torch.float32))
        kernels.check_error_flags(force=True)
    elif tensor_cores:
        assert kernels.window_attention_mma_supports(d, d, H, G)
        kernels.window_attention_mma(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(qsl), _ints(lengths),
                                     list(new), H, G, d, d, scale, 0.0, window, 0, splits=splits, sinks=_dev(sinks, torch.float32))
    else:
        kernels.window_attention_generic(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(pos), _ints(treq),
                                         H, G, d, d, scale, 0.0, window, 0, sinks=_dev(sinks, torch.float32))
    return out.view(T, H, d), want


KERNELS = [(False, torch.float32), (False, torch.bfloat16), (True, torch.bfloat16), ("tcgen05", torch.bfloat16)]


@pytest.mark.parametrize("tensor_cores,dtype", KERNELS)
def test_sink_attention_finds_one_far_key_among_hundreds(tensor_cores, dtype):
    """The last query of a long request looks at ONE key — the first of the sequence, the last of a page, the first of
    the next, one in the middle, itself — in a prompt's portion and decoded alone (with its keys split over CTAs)."""
    n, page = 700, 16
    d = 128 if tensor_cores == "tcgen05" else 64 if tensor_cores else 20
    for j in (0, 1, page - 1, page, 127, 128, 333, n - 2, n - 1):
        for new, t, splits in (([1, 1], 0, 3 if tensor_cores is True else 1), ([40, 2], 39, 1)):
            got, want = _sink_case(dtype, 4, 2, d, [n, 40], new, page, 10 + j, sharpen={t: j}, tensor_cores=tensor_cores, splits=splits)
            _close(got, want, dtype, f"query at {n - 1} looking at key {j}")
            assert float(want[t].abs().max()) > 0.2, "the case does not single a key out"


@pytest.mark.parametrize("tensor_cores,dtype", KERNELS)
def test_the_sink_takes_weight_and_gives_nothing(tensor_cores, dtype):
    big = torch.tensor([30.0, -30.0, 0.5, -1.0], dtype=torch.float64)
    d = 128 if tensor_cores == "tcgen05" else 64 if tensor_cores else 12
    for lengths, new in (([21], [21]), ([300, 5], [1, 1])):
        got, want = _sink_case(dtype, 4, 1, d, lengths, new, 4 if not tensor_cores else 16, 5, sink=big, tensor_cores=tensor_cores)
        _close(got, want, dtype, "sinks of +30, -30 and small ones")
        assert float(got[:, 0].float().abs().max()) < 1e-6, "a sink far above every score leaves no weight for the keys"
        assert float(got[:, 1].float().abs().max()) > 1e-2


@pytest.mark.parametrize("H,G", [(4, 2), (3, 3), (8, 1), (16, 2)])
def test_joined_rows_and_sinks_on_tcgen05(H, G):
    """The tcgen05 kernel over rows [key | value] of one plane with a sink per head: prompts beside single tokens, several
    query tiles a request, pages out of order, and a window whose pages behind it are kept or not."""
    dtype = torch.bfloat16
    for window in (0, 200, 33):
        got, want = _sink_case(dtype, H, G, 128, [300, 1, 97, 410], [300, 1, 40, 3], 16, 3 * H + window, tensor_cores="tcgen05", window=window)
        _close(got, want, dtype, f"tcgen05 attention over joined rows, window {window}")
    n, window = 260, 70
    for j in (n - window, n - window - 1, 0, 127, 128, n - 1):
        got, want = _sink_case(dtype, H, G, 128, [n, 50], [100, 2], 16, j, sharpen={99: j}, tensor_cores="tcgen05", window=window)
        _close(got, want, dtype, f"query {n - 1} with key {j} standing out")


@pytest.mark.parametrize("E,top,groups,keep", [(8, 3, 2, 1), (6, 2, 3, 2), (5, 2, 1, 1), (4, 4, 2, 2), (6, 1, 6, 2), (130, 7, 10, 3),
                                               (12, 5, 4, 4), (1, 1, 1, 1), (1000, 9, 8, 2)])
def test_scored_router(E, top, groups, keep):
    """Choice by score plus correction within the best groups, weights from the score alone: against the plain choice,
    with corrections that make choice scores negative (a masked expert counts as minus infinity, not as zero)."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(E * 7 + top)
    T = 67
    z = (torch.randn(T, E + 3, generator=g) * 2).float()
    corr = (torch.randn(E, generator=g) * 0.4 - (1.5 if E % 2 == 0 else 0.0)).float()
    choice = torch.empty(T, top, dtype=torch.int32, device="cuda")
    weight = torch.empty(T, top, dtype=torch.float32, device="cuda")
    kernels.router_scored_topk(z.cuda()[:, :E], top, choice, weight, correction=corr.cuda(), groups=groups, keep=keep, scale=2.5)
    margins = plain.choice_margins(z[:, :E].double(), corr.double(), top, groups, keep)
    checked = 0
    for t in range(T):
        if margins[t] < 1e-5:
            continue                                    # a close call in float32 may fall either way
        want, scores = plain.choose_experts(z[t, :E].double(), corr.double(), top, groups, keep)
        assert sorted(choice[t].tolist()) == sorted(want), f"token {t}: chose {choice[t].tolist()}, plain {want}"
        by_expert = dict(zip(choice[t].tolist(), weight[t].tolist()))
        for e, s in zip(want, scores):
            assert abs(by_expert[e] - 2.5 * float(s)) < 1e-5
        checked += 1
    assert checked > T // 2
    # without correction and with one group: the largest scores
    kernels.router_scored_topk(z.cuda()[:, :E], top, choice, weight)
    for t in range(0, T, 9):
        assert sorted(choice[t].tolist()) == sorted(torch.topk(z[t, :E], top).indices.tolist())


def test_scored_router_ties_go_to_the_lower_index():
    from cuinfer_b200 import kernels

    z = torch.zeros(3, 8, dtype=torch.float32, device="cuda")
    choice = torch.empty(3, 3, dtype=torch.int32, device="cuda")
    weight = torch.empty(3, 3, dtype=torch.float32, device="cuda")
    kernels.router_scored_topk(z, 3, choice, weight, groups=4, keep=2, scale=1.0)
    assert choice.tolist() == [[0, 1, 2]] * 3 and torch.allclose(weight, torch.full_like(weight, 0.5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("W,ff,E,top,T", [(72, 36, 5, 2, 9), (64, 32, 3, 3, 300), (128, 96, 9, 1, 700), (96, 160, 4, 2, 77), (40, 2600, 6, 5, 3)])
def test_experts_without_a_gate_and_a_gated_shared_expert(dtype, W, ff, E, top, T):
    """``sum_k w_k down_e(relu(up_e h)^2) + sigmoid(g) base``: rows by token and choice, and grouped by expert on the
    tensor cores (from 128 rows of bfloat16 on), with an expert that gets no row and a choice of -1."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(W + T)
    h = torch.randn(T, W, generator=g).to(dtype).double()
    up = (torch.randn(E, ff, W, generator=g) / math.sqrt(W)).to(dtype).double()
    down = (torch.randn(E, W, ff, generator=g) / math.sqrt(ff)).to(dtype).double()
    base = torch.randn(T, W, generator=g).to(dtype).double()
    gate = torch.randn(T, 3, generator=g).float()
    choice = torch.stack([torch.randperm(E, generator=g)[:top] for _ in range(T)]).to(torch.int32)
    choice[choice == E - 1] = 0 if top == 1 else -1                 # the last expert gets no row; some choices are void
    weights = torch.rand(T, top, generator=g).float()
    want = torch.sigmoid(gate[:, 1:2].double()) * base
    for t in range(T):
        for k in range(top):
            e = int(choice[t, k])
            if e >= 0:
                want[t] += float(weights[t, k]) * plain.expert(h[t], up[e], down[e])
    out = torch.empty(T, W, dtype=dtype, device="cuda")
    kernels.moe_table_feed_forward(_dev(h, dtype), None, choice.cuda(), _dev(up, dtype), _dev(down, dtype), _dev(base, dtype), out,
                                   weights=weights.cuda(), activation="relu2", base_gate=gate.cuda()[:, 1])
    _close(out, want, dtype, "experts without a gate", tol=3e-5 if dtype == torch.float32 else 3e-2)


# ---- other sizes, drawn at random ------------------------------------------------------------------------------------------
def _random_config(seed):
    """A small configuration whose every size, count, constant and order of layers is drawn: odd and even, ones, absent
    parts; from the sixth on every size is odd or no multiple of eight."""
    import random

    rnd = random.Random(seed)
    odd = seed >= 5
    width = rnd.choice([25, 41, 57, 99] if odd else [24, 40, 56, 64, 104])
    vocab = rnd.choice([33, 64, 131])
    layers, latents = [], []
    for i in range(rnd.randint(2, 5)):
        experts = rnd.choice([1, 2, 3, 4, 6, 8])
        groups = rnd.choice([g for g in (1, 2, 3, 4) if experts % g == 0])
        keep = rnd.randint(1, groups)
        top = rnd.randint(1, keep * (experts // groups))
        mlp = rnd.choice([None] + [_moe(experts, top, rnd.choice([9, 15, 21] if odd else [8, 16, 32]), rnd.choice([0.5, 1.0, 2.5]), groups, keep,
                                        shared=rnd.choice([0, 7 if odd else 8, 24]))] * 4)
        if rnd.random() < 0.55:
            rot_dim = rnd.choice([2, 4, 6, 16])
            dims = rnd.choice([rot_dim, rot_dim, rot_dim // 4 * 2])
            source = rnd.choice(latents) if latents and rnd.random() < 0.5 else None
            if source is not None:
                src = layers[source]["mixer"]
                rot_dim, rk, rot = src["rot_dim"], src["kv_rank"], src.get("rot")
            else:
                rk = rnd.choice([9, 20, 33] if odd else [8, 16, 24, 48])
                rot = None if dims == 0 else rnd.choice([
                    _ramp(rnd.choice([50.0, 1e4, 1e6]), dims, rnd.choice([2.0, 8.0, 40.0]), rnd.choice([16, 64, 1024]), rnd.choice([4.0, 32.0]), rnd.choice([0.5, 1.0])),
                    {"base": 300.0, "dims": dims}])
            layers.append(_latent(rnd.randint(1, 5), rnd.choice([5, 12, 20] if odd else [4, 8, 16]), rot_dim, rnd.choice([3, 10] if odd else [4, 8, 16]),
                                  rk, rnd.choice([0.1, 0.25, 0.5]), window=rnd.choice([None, 1, 2, 7, 16, 40]), rot=rot, kv_from=source, mlp=mlp))
            if source is None:
                latents.append(i)
        else:
            kv = rnd.randint(1, 3)
            d = rnd.choice([6, 10, 22] if odd else [8, 16, 32])
            dims = rnd.choice([d, d // 4 * 2, 0])
            rot = None if dims == 0 else {"base": rnd.choice([100.0, 5e4]), "dims": dims, **rnd.choice([{}, {"scaling": {"factor": rnd.choice([2.0, 8.0])}}])}
            layers.append(_sink(kv * rnd.randint(1, 3), kv, d, rnd.choice([0.15, 0.3]), rot=rot, mlp=mlp))
    return _config(vocab, width, layers, side=rnd.choice([None, 3, 8]), eps=rnd.choice([1e-6, 1e-5, 1e-3]))


@pytest.mark.parametrize("seed", range(12))
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg = _random_config(seed)
    tensors = plain.random_model(cfg, 100 + seed)
    t64 = {k: v.double() for k, v in tensors.items()}
    requests = _requests(cfg, [1, 23, 61, 9], seed=30 + seed)
    steps = traces.mixed(requests, max_live=3, sizes=(5, 2, 11, 3))
    for dtype in ("float32", "bfloat16"):
        folder = _write(str(tmp_path / dtype), cfg, tensors, dtype)
        out = str(tmp_path / f"out_{dtype}")
        traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), 16, max_live=4)
        got = traces.collect(steps, out, cfg["vocab"])
        whole_steps = traces.whole(requests)
        whole_out = str(tmp_path / f"whole_{dtype}")
        traces.replay_in_process(folder, dtype, whole_steps, whole_out, traces.live_token_peak(whole_steps), 16)
        whole = traces.collect(whole_steps, whole_out, cfg["vocab"])
        errors = []
        for rid, toks in requests.items():
            safe = plain.router_margin(cfg, t64, list(toks)) > MARGIN
            ref = plain.forward(cfg, t64, list(toks)).numpy()
            for pos, row in sorted(got[rid].items()):
                assert np.isfinite(row).all()
                if dtype == "float32":
                    cut = _row_error(row, whole[rid][pos].astype(np.float64))
                    assert cut <= CUT_TOLERANCE[dtype], f"configuration {seed}: request {rid} position {pos} depends on the cut ({cut:.3e}): {json.dumps(cfg)}"
                if safe or dtype == "float32":
                    errors.append((_row_error(row, ref[pos]), rid, pos))
        worst = max(errors)
        if dtype == "float32":
            assert worst[0] <= TOLERANCE[dtype], f"configuration {seed}: request {worst[1]} position {worst[2]} (error {worst[0]:.3e}): {json.dumps(cfg)}"
        else:
            # very narrow layers now and then give a token a sub-layer output that nearly cancels, which magnifies the
            # rounding of bfloat16; the bfloat16 run is held by its median row, which a wrong shape or kernel would move
            median = sorted(e for e, _, _ in errors)[len(errors) // 2]
            assert median <= 0.05, f"configuration {seed} in bfloat16: median row error {median:.3e}: {json.dumps(cfg)}"
