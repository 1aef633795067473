"""Desilorn through the engine against the plain implementation (``plain_desilorn``), mechanism by mechanism and as a
whole: every way of cutting the work, pages and slots that are used again, keys just inside and just outside a sliding
window and a chunk, sinks, the distance bias, the streams of the residual, sizes that are odd, equal to one or absent,
and greedy generation through the entry point and the scheduler.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np
import pytest
import torch

import plain_desilorn as plain
import traces
from conftest import note_error, random_tokens

pytestmark = pytest.mark.gpu


def _sliding(heads, kv_heads, dim, vdim, scale, window=None, temp=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window:
        m["mask"] = {"size": window}
    if temp:
        m["q_temp"] = {"coef": temp[0], "every": temp[1]}
    return {"type": "attention", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _chunks(heads, kv_heads, dim, vdim, scale, chunk=None, rot=None, ff=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if chunk:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"base": rot[0], "dims": rot[1]}
    return {"type": "attention_2", "mixer": m, "mlp": {"kind": "dense", "ff": ff} if ff else None}


def _config(vocab, width, layers, streams=None, loop=None, eps=1e-6):
    cfg = {"architecture": "Desilorn", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}
    if streams:
        cfg["streams"] = streams
    if loop:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# odd sizes everywhere; three streams; the two middle layers run three times; one key/value head; a layer without
# feed-forward; a window of 9, chunks of 7 and of a page (16); a layer without mask; rotation of a part and of all of a head
ODD = _config(89, 40, [
    _sliding(3, 1, 10, 6, 0.4, window=9, temp=(0.7, 5), ff=52),
    _chunks(4, 2, 12, 20, 0.5, chunk=7, rot=(50.0, 6)),
    _sliding(2, 2, 16, 8, 0.3, ff=24),
    _chunks(2, 1, 8, 8, 0.6, chunk=16, rot=(1000.0, 8), ff=30),
], streams=3, loop=(1, 3, 3), eps=1e-5)
# one residual row and a plain sum (no streams), no loop, pages of 32; chunks without rotation and a layer of chunks
# without mask; a query temperature that changes with every token; a window one longer than a page
PLAIN = _config(300, 64, [
    _chunks(4, 4, 16, 16, 0.4, chunk=33, ff=96),
    _sliding(4, 2, 24, 12, 0.3, window=33, temp=(0.4, 1), ff=80),
    _chunks(2, 1, 32, 24, 0.25, rot=(10000.0, 16)),
])
# one stream with its coefficients; the whole model runs twice
ONE = _config(120, 48, [
    _sliding(4, 1, 12, 12, 0.45, window=20, temp=(0.2, 64), ff=64),
    _chunks(3, 3, 16, 8, 0.5, chunk=24, rot=(200.0, 16), ff=64),
], streams=1, loop=(0, 2, 2))
# sizes that the tensor-core kernels take in bfloat16 (key sizes 64 and 128; value sizes 32, 64 and 128); two streams;
# windows and chunks that start inside key tiles
WIDE = _config(512, 256, [
    _sliding(8, 2, 64, 64, 0.2, window=48, temp=(0.5, 32), ff=512),
    _chunks(4, 4, 128, 64, 0.12, chunk=40, rot=(1e4, 64), ff=256),
    _sliding(2, 1, 128, 128, 0.1, window=100, ff=256),
    _chunks(6, 2, 64, 32, 0.2, chunk=64, rot=(5e5, 32)),
], streams=2, loop=(2, 4, 2))
MODELS = {"odd": (ODD, 16, 31), "plain": (PLAIN, 32, 32), "one": (ONE, 16, 33), "wide": (WIDE, 16, 34)}

# Largest error of a row of logits (see _row_error).  float32: only the order of sums differs.  bfloat16: the engine
# rounds where it stores (normed rows, projections, cached keys and values, mixer outputs, activations).
TOLERANCE = {"float32": 4e-5, "bfloat16": 8e-2}
# Between two ways of cutting the same request: float32 has one kernel per operation, so the logits agree to the last
# bits; in bfloat16 the kernels of a step of few rows and of many round at different places.
CUT_TOLERANCE = {"float32": 2e-6, "bfloat16": 8e-2}


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
        dirs = {d: _write(str(tmp_path_factory.mktemp(f"desilorn_{name}_{d}")), cfg, tensors, d) for d in TOLERANCE}
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
        ref = plain.forward(cfg, tensors, list(toks)).numpy()
        assert got.get(rid), f"no logits came back for request {rid}"
        assert sorted(got[rid]) == list(range(len(toks)))
        whole = _whole_rows(folders, name, dtype, rid, list(toks), tmp_path)
        over = []
        # float32 is held at every position.  In bfloat16 the narrow models round coarsely (rows of 40 values, queries
        # made sharp): one position in fifty of a request may reach twice the bound.
        slack = 1 if dtype == "float32" else 2
        for pos, row in sorted(got[rid].items()):
            assert np.isfinite(row).all(), f"request {rid} position {pos}: logits are not finite"
            cut = _row_error(row, whole[pos].astype(np.float64))
            err = _row_error(row, ref[pos])
            assert cut <= slack * CUT_TOLERANCE[dtype], f"{name}/{dtype}: request {rid}: position {pos} of {len(toks)} depends on how the work was cut ({cut:.3e})"
            assert err <= slack * TOLERANCE[dtype], f"{name}/{dtype}: request {rid}: first wrong position {pos} of {len(toks)} (error {err:.3e})"
            if err > TOLERANCE[dtype] or cut > CUT_TOLERANCE[dtype]:
                over.append(pos)
            else:
                worst = max(worst, err)
        assert len(over) <= max(1, len(toks) // 50), f"{name}/{dtype}: request {rid}: positions {over} of {len(toks)} are over the bound"
    note_error(dtype, f"model {name}", worst, family="Desilorn")
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
    """The decoded tail is longer than every window and chunk but one, so windows pass over decoded tokens, chunks
    begin among them and pages are given back."""
    requests = _requests(folders[name][0], [40, 131], seed=2)
    _check(folders, name, dtype, traces.tail_decode(requests, 70), requests, tmp_path)


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
def test_steps_through_cuda_graphs(folders, dtype, tmp_path):
    """The same logits when decode steps and repeated step shapes are replayed from graphs, as generation runs them."""
    requests = _requests(folders["wide"][0], [70, 40, 90, 33], seed=6)
    steps = traces.mixed(requests, max_live=3, sizes=(32, 40, 35))
    _check(folders, "wide", dtype, steps, requests, tmp_path, cuda_graph=True, passes=2, max_live=4)


def test_greedy_generation_through_the_entry_point(folders):
    from cuinfer_b200 import LLM, SamplingParams

    for name in ("odd", "plain", "one"):
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

    cfg, dirs, tensors, block = folders["one"]
    prompt = random_tokens(cfg["vocab"], 9, 95)
    proc = subprocess.run([sys.executable, "-m", "cuinfer_b200", "generate", "--model", dirs["float32"], "--dtype", "float32",
                           "--prompt-ids", ",".join(map(str, prompt)), "--max-tokens", "5", "--temperature", "0", "--ignore-eos",
                           "--num-blocks", "16", "--max-num-seqs", "4", "--block-size", str(block)],
                          capture_output=True, text=True, cwd=ROOT, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    line = [json.loads(l) for l in proc.stdout.splitlines() if l.startswith("{")][0]
    assert line["token_ids"] == plain.greedy(cfg, tensors, prompt, 5)


def test_residual_after_every_layer_run(folders):
    """The sum of the streams after every layer run (a looped layer counts each time) against the plain implementation."""
    from cuinfer_b200.engine import replay
    from cuinfer_b200.engine.runner import StepEntry

    for name in NAMES:
        cfg, dirs, tensors, block = folders[name]
        toks = random_tokens(cfg["vocab"], 37, 8)
        want = []
        plain.forward(cfg, tensors, toks, taps=want)
        runner = replay.make_runner(dirs["float32"], "float32", 64, block)
        entries = [StepEntry("a", toks, [0])]
        assert runner.reserve("a", len(toks))
        runner.storage.zero_slots(runner.manager.take_newly_admitted())
        ctx, _ = runner.build_context(entries)
        got = []
        runner.model.forward(ctx, tap=lambda run, stream: got.append(stream.collapsed().double().cpu()))
        assert len(got) == len(want) == len(plain.run_order(cfg))
        for run, (g, w) in enumerate(zip(got, want)):
            err = float((g - w).abs().max() / w.abs().max())
            assert err <= 2e-5, f"{name}: the residual after run {run} is off by {err:.3e} of its largest value"


# ---- mechanisms alone -------------------------------------------------------------------------------------------------
def _dev(t, dtype):
    return t.to(device="cuda", dtype=dtype).contiguous()


def _close(got, want, dtype, what, tol=None):
    tol = tol or (2e-5 if dtype == torch.float32 else 2e-2)
    err = float((got.double().cpu() - want).abs().max() / want.abs().max().clamp_min(1e-9))
    assert err <= tol, f"{what} in {dtype}: error {err:.3e} of the largest value"


def _ints(values):
    return torch.tensor(values, dtype=torch.int32, device="cuda")


class _Store:
    """The tensors of a test, handed to a part the way the loader does."""

    def __init__(self, tensors, dtype):
        self.tensors, self.dtype = tensors, dtype

    def get(self, spec):
        t = self.tensors[spec.name]
        assert tuple(t.shape) == tuple(spec.shape), spec.name
        return t.to(device="cuda", dtype=self.dtype).contiguous()

    def get_stacked(self, specs):
        return torch.cat([self.get(s) for s in specs]).contiguous()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("S,W", [(1, 40), (2, 64), (3, 37), (4, 256), (5, 1000), (8, 72), (4, 4096), (7, 2052), (12, 48), (16, 33)])
def test_streams_are_read_and_written_in_one_pass(dtype, S, W):
    """Write alone, read with its norm alone, both in one pass, and the read row itself; the streams stay 32-bit."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(S * 1000 + W)
    T = 11
    xs = torch.randn(S, T, W, generator=g).float().double() * 3
    y = torch.randn(T, W, generator=g).to(dtype).double()
    mix = (torch.eye(S) + 0.4 * torch.randn(S, S, generator=g)).float()
    out_w, in_w = torch.randn(S, generator=g).float(), torch.randn(S, generator=g).float()
    gain = (1 + 0.2 * torch.randn(W, generator=g)).float()
    eps = 1e-5
    written = plain.streams_write(xs, y, mix.double(), out_w.double())
    read = plain.streams_read(written, in_w.double())
    normed = plain.rms(read, eps) * gain.double()

    def device_streams():
        return xs.permute(1, 0, 2).float().contiguous().cuda()               # [T, S, W]

    # the write alone
    dev = device_streams()
    kernels.hyper_stream(dev, _dev(y, dtype), (mix.cuda(), out_w.cuda()), None, None, None)
    _close(dev.permute(1, 0, 2), written, torch.float32, "streams after the write")
    # the read and its norm alone, on the written streams
    out = torch.empty(T, W, dtype=dtype, device="cuda")
    row = torch.empty(T, W, dtype=torch.float32, device="cuda")
    before = dev.clone()
    kernels.hyper_stream(dev, None, None, in_w.cuda(), (gain.cuda(), eps), out, read_out=row)
    assert torch.equal(dev, before), "a read changed the streams"
    _close(out, normed, dtype, "normed read")
    _close(row, read, torch.float32, "the read row")
    # both in one pass
    dev = device_streams()
    out2 = torch.empty(T, W, dtype=dtype, device="cuda")
    kernels.hyper_stream(dev, _dev(y, dtype), (mix.cuda(), out_w.cuda()), in_w.cuda(), (gain.cuda(), eps), out2)
    _close(dev.permute(1, 0, 2), written, torch.float32, "streams after write and read in one pass")
    _close(out2, normed, dtype, "normed read in one pass")
    # the sum of the streams at a few tokens, with and without a write outstanding; an index outside gives zeros
    dev = device_streams()
    idx = [T - 1, 0, 4, T + 3]
    rows = torch.empty(len(idx), W, dtype=torch.float32, device="cuda")
    kernels.hyper_gather(dev, _dev(y, dtype), (mix.cuda(), out_w.cuda()), _ints(idx), rows)
    _close(rows[:3], written.sum(0)[idx[:3]], torch.float32, "sum of the streams after the outstanding write")
    assert float(rows[3].abs().max()) == 0.0
    assert torch.equal(dev, device_streams()), "the gather changed the streams"
    kernels.hyper_gather(dev, None, None, _ints(idx), rows)
    _close(rows[:3], xs.sum(0)[idx[:3]], torch.float32, "sum of the streams")


def test_every_stream_starts_as_the_embedding_row():
    from cuinfer_b200 import kernels

    table = torch.randn(20, 24).bfloat16().cuda()
    ids = _ints([3, 19, 0, 3])
    out = torch.empty(4, 5, 24, dtype=torch.float32, device="cuda")
    kernels.embedding_gather(ids, table, out)
    for s in range(5):
        assert torch.equal(out[:, s], table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_with_a_weight_stored_around_zero(dtype):
    from cuinfer_b200.parts import NORMS, PartSpec

    g = torch.Generator().manual_seed(4)
    W = 72
    w = (0.3 * torch.randn(W, generator=g)).bfloat16()
    norm = NORMS.get("rmsnorm")(PartSpec("rmsnorm", eps=1e-5, weight_suffix="", one_plus=True), hidden_size=W, prefix="n", dtype=dtype)
    norm.load(_Store({"n": w}, dtype))
    rows = torch.randn(6, W, generator=g).float() * 4
    got = norm.norm_rows(rows.cuda())
    _close(got, plain.norm_one_plus(rows.double(), w.double(), 1e-5), dtype, "one plus the weight")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,width,ff", [(1, 40, 24), (7, 64, 96), (200, 256, 512), (150, 72, 100)])
def test_feed_forward_gated_by_gelu(dtype, rows, width, ff):
    """Few rows (the projection's own epilogue) and many (the tensor-core product's) against the plain feed-forward."""
    from cuinfer_b200.parts import FEED_FORWARDS, PartSpec

    g = torch.Generator().manual_seed(rows)
    w = {"f.gate": torch.randn(ff, width, generator=g) / math.sqrt(width), "f.up": torch.randn(ff, width, generator=g) / math.sqrt(width),
         "f.down": torch.randn(width, ff, generator=g) / math.sqrt(ff)}
    w = {k: v.bfloat16() for k, v in w.items()}
    part = FEED_FORWARDS.get("gated")(PartSpec("gated", intermediate_size=ff, activation="gelu_tanh", names=("gate", "up", "down")),
                                      hidden_size=width, prefix="f", dtype=dtype)
    part.load(_Store(w, dtype))
    h = (torch.randn(rows, width, generator=g) * 2).to(dtype)
    want = plain.feed_forward(h.double(), {k[2:]: v.double() for k, v in w.items()})
    _close(part.forward(h.cuda(), None), want, dtype, "gelu(gate) * up through down", tol=None if dtype == torch.float32 else 3e-2)


# ---- the two attentions alone, over a paged cache ---------------------------------------------------------------------
def _attention_case(dtype, H, G, d, dv, lengths, new, page, seed, size, chunked, bias, sinks, sharpen=None, tensor_cores=False,
                    splits=1, strength=14.0):
    """Requests of ``lengths`` tokens whose last ``new`` are this step's queries, over a cache of random keys and values
    on shuffled pages; kernel output and the plain result from the same cached rows.  ``bias``: the distance bias of the
    sliding kind; ``sinks``: None, "zero" or a list of numbers per head.  ``sharpen[t] = j`` makes query t's score with
    key j of its request stand out."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(seed)
    R = len(lengths)
    pages_per = [-(-n // page) for n in lengths]
    num_pages = sum(pages_per) + 3
    perm = torch.randperm(num_pages, generator=g).tolist()
    table = torch.full((R, max(pages_per) + 1), -1, dtype=torch.int32)
    cache = torch.randn(num_pages, 1, G, page, d + dv, generator=g).to(dtype)
    rows = {}
    at = 0
    for r, n in enumerate(lengths):
        table[r, :pages_per[r]] = torch.tensor(perm[at:at + pages_per[r]], dtype=torch.int32)
        at += pages_per[r]
        rows[r] = torch.stack([cache[int(table[r, j // page]), 0, :, j % page] for j in range(n)]).double()      # [n, G, d + dv]
    T = sum(new)
    q = torch.randn(T, H, d, generator=g).to(dtype).double()
    pos, treq = [], []
    for r, (n, k) in enumerate(zip(lengths, new)):
        pos += list(range(n - k, n))
        treq += [r] * k
    scale = 0.35
    if sharpen:
        for t, j in sharpen.items():
            for h in range(H):
                key = rows[treq[t]][j, h // (H // G), :d]
                q[t, h] = (strength / scale) * key / (key @ key)
        q = q.to(dtype).double()
    sink_values = None if sinks is None else torch.zeros(H, dtype=torch.float64) if sinks == "zero" else torch.tensor(sinks, dtype=torch.float64)
    slopes = plain.distance_slopes(H) if bias else None
    want = torch.zeros(T, H, dv, dtype=torch.float64)
    at = 0
    for r, (n, k) in enumerate(zip(lengths, new)):
        full = torch.zeros(n, H, d, dtype=torch.float64)
        full[n - k:] = q[at:at + k]
        res = plain.attend(full, rows[r][:, :, :d], rows[r][:, :, d:], scale, plain.sees_chunk if chunked else plain.sees_sliding,
                           size or None, slopes=slopes, sinks=sink_values)
        want[at:at + k] = res.view(n, H, dv)[n - k:]
        at += k
    out = torch.empty(T, H * dv, dtype=dtype, device="cuda")
    kw = dict(chunked=chunked, slopes=torch.tensor(slopes, dtype=torch.float32).cuda() if slopes else None,
              sinks=sink_values.float().cuda() if sink_values is not None else None)
    if tensor_cores:
        assert kernels.window_attention_mma_supports(d, dv, H, G)
        qsl = [0]
        for k in new:
            qsl.append(qsl[-1] + k)
        kernels.window_attention_mma(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(qsl), _ints(lengths),
                                     [T + 64] + [1] * (len(new) - 1), H, G, d, dv, scale, 0.0, size, 0, splits=splits, **kw)
    else:
        kernels.window_attention_generic(_dev(q.reshape(T, H * d), dtype), out, cache.cuda(), table.cuda(), _ints(pos), _ints(treq),
                                         H, G, d, dv, scale, 0.0, size, 0, **kw)
    return out.view(T, H, dv), want


def _edge_cases(pos, size, chunked):
    """(key, whether the query at ``pos`` sees it): both sides of the window's or chunk's edge, the query's own key, the
    first token, keys far back and both sides of a page border of 8."""
    first = pos // size * size if chunked else pos - size + 1
    keys = {first, first - 1, first + 1, pos, pos - 1, 0, 1, 7, 8, first - 8, (first + pos) // 2}
    sees = plain.sees_chunk if chunked else plain.sees_sliding
    return [(j, bool(sees(torch.tensor(pos), torch.tensor(j), size))) for j in sorted(keys) if 0 <= j <= pos]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("decode", [False, True])
@pytest.mark.parametrize("chunked", [False, True])
def test_one_key_stands_out_at_every_edge(dtype, decode, chunked):
    """A key whose score is made to dominate is seen exactly when the mask says so, for a query inside a prompt's
    portion and for a single decoded token; the chunked kind also for a query that opens a chunk and sees itself only."""
    page, size = 8, 21
    for n in (96, 85 if chunked else 22, 106):
        pos = n - 1
        cases = _edge_cases(pos, size, chunked)
        assert any(e for _, e in cases) and any(not e for _, e in cases)
        for j, _expected in cases:
            new, t = ([1, 1], 0) if decode else ([min(30, n), 3], min(30, n) - 1)
            got, want = _attention_case(dtype, 4, 2, 24, 12, [n, 40], new, page, 7 + j, size, chunked, bias=not chunked,
                                        sinks="zero" if chunked else [0.5, -3.0, 2.0, 0.0], sharpen={t: j})
            _close(got, want, dtype, f"query {pos} with key {j} standing out")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_sink_takes_its_share_and_brings_nothing(dtype):
    """Queries of zero give every seen key the score 0; the output is then the sum of the seen values over their count
    plus exp(sink), which a sink that was left out, scaled, biased or counted twice would change."""
    from cuinfer_b200 import kernels

    H, G, d, dv, n, page = 4, 2, 16, 8, 13, 4
    g = torch.Generator().manual_seed(1)
    cache = torch.randn(5, 1, G, page, d + dv, generator=g).to(dtype)
    table = torch.tensor([[3, 0, 4, 1, -1]], dtype=torch.int32)
    sinks = torch.tensor([2.0, -1.0, 0.0, 4.0])
    values = torch.stack([cache[int(table[0, j // page]), 0, :, j % page, d:] for j in range(n)]).double()     # [n, G, dv]
    out = torch.empty(1, H * dv, dtype=dtype, device="cuda")
    q = torch.zeros(1, H * d, dtype=dtype, device="cuda")
    kernels.window_attention_generic(q, out, cache.cuda(), table.cuda(), _ints([n - 1]), _ints([0]), H, G, d, dv, 0.7, 0.0, 0, 0,
                                     sinks=sinks.cuda())
    want = torch.stack([values[:, h // 2].sum(0) / (n + math.exp(float(sinks[h]))) for h in range(H)])
    _close(out.view(H, dv), want, dtype, "equal weights beside a sink")
    # the distance bias alone: weights exp(-slope (i - j)) over their sum plus exp(sink)
    slopes = plain.distance_slopes(H)
    kernels.window_attention_generic(q, out, cache.cuda(), table.cuda(), _ints([n - 1]), _ints([0]), H, G, d, dv, 0.7, 0.0, 5, 0,
                                     slopes=torch.tensor(slopes).cuda(), sinks=sinks.cuda())
    want = []
    for h in range(H):
        w = torch.tensor([math.exp(-slopes[h] * (n - 1 - j)) if n - 1 - j < 5 else 0.0 for j in range(n)], dtype=torch.float64)
        want.append((w[:, None] * values[:, h // 2]).sum(0) / (w.sum() + math.exp(float(sinks[h]))))
    _close(out.view(H, dv), torch.stack(want), dtype, "the distance bias inside a window beside a sink")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,size,chunked,bias,sinks", [
    (3, 1, 20, 36, 0, False, True, [1.0, -2.0, 0.3]), (6, 3, 64, 16, 16, True, False, "zero"), (2, 2, 7, 5, 3, False, True, [0.0, 5.0]),
    (8, 2, 128, 128, 40, True, False, "zero"), (1, 1, 32, 160, 1, False, True, [-4.0]), (5, 5, 48, 48, 1, True, False, "zero"),
    (4, 1, 9, 3, 0, True, False, "zero"), (2, 1, 12, 12, 17, False, False, None), (7, 7, 3, 2, 64, True, True, [0.1] * 7)])
def test_attention_of_many_shapes(dtype, H, G, d, dv, size, chunked, bias, sinks):
    got, want = _attention_case(dtype, H, G, d, dv, [50, 1, 17, 70], [50, 1, 2, 1], 16, d + size, size, chunked, bias, sinks)
    _close(got, want, dtype, "attention output")


@pytest.mark.parametrize("d,dv,H,G", [(64, 32, 4, 2), (64, 64, 8, 2), (128, 128, 2, 2), (128, 64, 6, 1), (64, 128, 4, 4), (128, 32, 3, 1),
                                      (64, 64, 5, 1), (128, 128, 14, 2), (64, 32, 10, 2), (128, 64, 16, 1)])
def test_attention_on_the_tensor_cores(d, dv, H, G):
    """The tensor-core kernel against plain attention over the same cached rows: windows and chunks that start inside and
    between key tiles, requests of one token beside long portions, and a key made to stand out at every edge."""
    dtype = torch.bfloat16
    sink_list = [((-1) ** h) * 0.5 * h for h in range(H)]
    for size, chunked, bias, sinks in ((0, False, True, sink_list), (70, False, True, sink_list), (64, True, False, "zero"),
                                       (200, True, False, "zero"), (5, True, False, "zero"), (64, False, False, None), (1, False, True, sink_list)):
        got, want = _attention_case(dtype, H, G, d, dv, [300, 1, 97, 210], [300, 1, 40, 3], 16, d + dv + size, size, chunked, bias, sinks,
                                    tensor_cores=True)
        _close(got, want, dtype, f"attention output with a mask of {size} (chunks: {chunked})")
    n, size = 260, 70
    for chunked in (False, True):
        for j, _ in _edge_cases(n - 1, size, chunked) + [(63, None), (64, None)]:
            got, want = _attention_case(dtype, H, G, d, dv, [n, 50], [100, 2], 16, j, size, chunked, not chunked,
                                        "zero" if chunked else sink_list, sharpen={99: j}, tensor_cores=True)
            _close(got, want, dtype, f"query {n - 1} with key {j} standing out (chunks: {chunked})")


@pytest.mark.parametrize("splits", [2, 3, 8])
def test_decode_steps_share_a_mask_over_several_ctas(splits):
    """Single decoded tokens whose key tiles are split over CTAs and merged; the sink counts once, not once per split."""
    dtype = torch.bfloat16
    sink_list = [3.0, -1.0, 0.0, 1.5, 0.2, -0.3, 6.0, 0.7]
    for size, chunked, bias, sinks in ((0, False, True, sink_list), (300, False, True, sink_list), (256, True, False, "zero"), (40, True, False, "zero")):
        got, want = _attention_case(dtype, 8, 2, 64, 64, [700, 1, 97, 333], [1, 1, 1, 1], 16, 5 + size, size, chunked, bias, sinks,
                                    tensor_cores=True, splits=splits)
        _close(got, want, dtype, f"decode with a mask of {size} (chunks: {chunked}) over {splits} splits")
    n, size = 640, 300
    for chunked in (False, True):
        for j, _ in _edge_cases(n - 1, size, chunked) + [(n - 65, None)]:
            got, want = _attention_case(dtype, 4, 2, 128, 64, [n, 20], [1, 1], 16, j, size, chunked, not chunked,
                                        "zero" if chunked else sink_list[:4], sharpen={0: j}, tensor_cores=True, splits=splits)
            _close(got, want, dtype, f"query {n - 1} with key {j} standing out over {splits} splits (chunks: {chunked})")


@pytest.mark.parametrize("H,G,d,dv,new", [(3, 3, 64, 32, 1), (10, 2, 128, 128, 3), (16, 1, 64, 64, 1), (16, 2, 128, 64, 2), (12, 4, 64, 128, 5)])
@pytest.mark.parametrize("splits", [1, 4])
def test_steps_of_few_rows_share_the_keys_of_a_tile(H, G, d, dv, new, splits):
    """A step whose requests all bring at most sixteen rows (tokens x query heads of a key head) runs the form of the
    tensor-core kernel whose four warps take a quarter of every key tile each: one to sixteen rows, a key made to stand
    out in every quarter of a tile and at the window's and the chunk's edges, requests of a few keys and of many."""
    dtype = torch.bfloat16
    assert new * (H // G) <= 16
    sink_list = [0.5 * (h % 5) - 1.0 for h in range(H)]
    n, size = 700, 200
    lengths, news = [n, new, 97 + new, 333], [new, new, new, new]
    for chunked in (False, True):
        edges = [j for j, _ in _edge_cases(n - 1, size, chunked)]
        first = (n - 1) // size * size if chunked else n - size
        quarters = [first // 64 * 64 + 64 + 16 * w + 3 * w for w in range(4)]      # one key in each warp's share of a whole tile
        for j in edges + quarters:
            got, want = _attention_case(dtype, H, G, d, dv, lengths, news, 16, 11 + j, size, chunked, not chunked,
                                        "zero" if chunked else sink_list, sharpen={new - 1: j}, tensor_cores=True, splits=splits)
            _close(got, want, dtype, f"{new} tokens x {H // G} heads with key {j} standing out (chunks: {chunked}, {splits} splits)")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,G,d,dv,dims", [(4, 2, 10, 6, 6), (3, 1, 16, 16, 16), (2, 2, 64, 32, 2), (5, 5, 7, 9, 0)])
def test_bias_head_norm_rotation_in_halves_and_cache_write(dtype, H, G, d, dv, dims):
    """What the chunked kind does between projection and scores: biases, the norm of every query and key head with one
    gain for all heads, then the rotation of the first dimensions in halves; keys and values land in their slots."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(3 + d)
    T, page, eps, base = 9, 4, 1e-5, 250.0
    columns = (H + G) * d + G * dv
    rows = torch.randn(T, columns + 3, generator=g).to(dtype).double()
    bias = (0.5 * torch.randn(columns, generator=g)).float()
    q_gain, k_gain = (1 + 0.3 * torch.randn(d, generator=g)).float(), (1 + 0.3 * torch.randn(d, generator=g)).float()
    positions = [0, 1, 2, 3, 1000, 1001, 70000, 5, 6]
    slots = [7, 2, 3, -1, 0, 1, 11, 10, 5]
    freqs = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float32)
    cache = torch.zeros(3, 1, G, page, d + dv, dtype=dtype, device="cuda")
    dev = _dev(rows, dtype)
    kernels.window_attention_prep(dev, _ints(positions), _ints(slots), freqs.cuda() if dims else None, dims, eps, H, G, d, dv, None, None,
                                  cache, bias=bias.cuda(), norm=True, q_gain=q_gain.cuda(), k_gain=k_gain.cuda(), norm_first=True,
                                  rot_half=True)
    biased = rows[:, :columns] + bias.double()

    def rotated(x):
        """The design takes the angle in 32 bits, position times frequency; the plain rotation gets those very angles."""
        if not dims:
            return x
        out = x.clone()
        half = dims // 2
        for t in range(T):
            a = (torch.tensor(float(positions[t]), dtype=torch.float32) * freqs).double()
            u, v = x[t, :, :half], x[t, :, half:dims]
            out[t, :, :half] = u * torch.cos(a) - v * torch.sin(a)
            out[t, :, half:dims] = v * torch.cos(a) + u * torch.sin(a)
        return out

    q = rotated(plain.rms(biased[:, :H * d].view(T, H, d), eps) * q_gain.double())
    k = rotated(plain.rms(biased[:, H * d:(H + G) * d].view(T, G, d), eps) * k_gain.double())
    v = biased[:, (H + G) * d:].view(T, G, dv)
    if dims:        # the plain rotation by whole positions agrees where the 32-bit angle is exact
        small = plain.rotate_half(plain.rms(biased[:4, :H * d].view(4, H, d), eps) * q_gain.double(), torch.arange(4), base, dims)
        assert float((small - q[:4]).abs().max()) < 1e-5
    _close(dev[:, :H * d].view(T, H, d), q, dtype, "queries")
    for t in range(T):
        if slots[t] < 0:
            continue
        got = cache[slots[t] // page, 0, :, slots[t] % page]
        _close(got[:, :d], k[t], dtype, f"key of token {t} at position {positions[t]}")
        _close(got[:, d:], v[t], dtype, f"value of token {t}")
    flat = cache.permute(0, 3, 1, 2, 4).reshape(-1, G, d + dv)
    assert float(flat[[4, 6, 8, 9]].abs().max()) == 0.0, "a token without slot wrote somewhere"


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("coef,every", [(0.5, 4), (0.3, 1), (1.5, 1000), (0.0, 3)])
def test_bias_and_query_temperature(dtype, coef, every):
    """What the sliding kind does between projection and scores: biases, and the queries times
    1 + coef ln(floor((p + 1) / every) + 1); keys and values are not scaled."""
    from cuinfer_b200 import kernels

    g = torch.Generator().manual_seed(every)
    H, G, d, dv, page = 3, 1, 12, 5, 4
    positions = [0, 1, 2, 3, 4, 6, 7, 8, 998, 999, 1000, 70000]
    T = len(positions)
    columns = (H + G) * d + G * dv
    rows = torch.randn(T, columns, generator=g).to(dtype).double()
    bias = (0.5 * torch.randn(columns, generator=g)).float()
    cache = torch.zeros(3, 1, G, page, d + dv, dtype=dtype, device="cuda")
    dev = _dev(rows, dtype)
    kernels.window_attention_prep(dev, _ints(positions), _ints(list(range(T))), None, 0, 1e-6, H, G, d, dv, None, None, cache,
                                  bias=bias.cuda(), norm=False, q_temp=(coef, every))
    biased = rows + bias.double()
    factor = torch.tensor([plain.query_temperature(p, coef, every) for p in positions], dtype=torch.float64)
    if every == 4:
        assert factor[2] == 1.0 and factor[3] > 1.0 and factor[5] == factor[3] and factor[6] > factor[5]
    _close(dev[:, :H * d], biased[:, :H * d] * factor[:, None], dtype, "queries")
    for t in range(T):
        got = cache[t // page, 0, :, t % page]
        _close(got[:, :d], biased[t, H * d:(H + G) * d].view(G, d), dtype, f"key of token {t}")
        _close(got[:, d:], biased[t, (H + G) * d:].view(G, dv), dtype, f"value of token {t}")


# ---- other sizes, drawn at random ---------------------------------------------------------------------------------------
def _random_config(seed):
    """A small configuration whose every size, count, constant, the order of its layers and the looped span are drawn:
    ones, absent parts (no mask, no rotation, no temperature, no feed-forward, no streams, no loop); from seed 10 on every
    size is odd or at least no multiple of eight; seeds 6 to 9 draw the sizes that the tensor-core kernels take."""
    import random

    rnd = random.Random(1000 + seed)
    odd, wide = seed >= 10, 6 <= seed < 10
    pick = lambda even_sizes, odd_sizes: rnd.choice(odd_sizes if odd else even_sizes)      # noqa: E731
    width = rnd.choice([128, 192, 256]) if wide else pick([24, 40, 56, 64, 104], [37, 50, 66, 98, 131])
    vocab = pick([33, 64, 136], [31, 77, 257])
    layers = []
    for _ in range(rnd.randint(1, 5)):
        kv = pick([1, 2, 4], [1, 3, 5])
        heads = kv * pick([1, 2, 4], [1, 2, 3])
        dim = rnd.choice([64, 128]) if wide else pick([8, 12, 16, 20, 32, 48], [6, 7, 9, 14, 22, 50])
        vdim = rnd.choice([32, 64, 128]) if wide else pick([4, 8, 16, 20, 32, 48], [5, 9, 17, 40])
        scale = rnd.choice([0.5, 1.0, 2.0]) / math.sqrt(dim)
        size = pick([None, 1, 2, 8, 16, 32, 64, 96], [None, 1, 3, 7, 15, 31, 65, 100])
        ff = rnd.choice([None, pick([16, 40, 96], [15, 41, 99])]) if rnd.random() < 0.8 else None
        if rnd.random() < 0.5:
            temp = (rnd.choice([0.1, 0.5, 2.0]), rnd.choice([1, 2, 7, 16, 128])) if rnd.random() < 0.8 else None
            layers.append(_sliding(heads, kv, dim, vdim, scale, window=size, temp=temp, ff=ff))
        else:
            rot = (rnd.choice([50.0, 1e4, 1e6]), rnd.choice([2, 4, dim // 4 * 2, dim // 2 * 2])) if rnd.random() < 0.8 else None
            layers.append(_chunks(heads, kv, dim, vdim, scale, chunk=size, rot=rot, ff=ff))
    n = len(layers)
    loop = None
    if rnd.random() < 0.7:
        start = rnd.randint(0, n - 1)
        loop = (start, rnd.randint(start, n), rnd.randint(1, 3))
    return (_config(vocab, width, layers, streams=rnd.choice([None, 1, 2, 3, 4, 5, 8]), loop=loop, eps=rnd.choice([1e-6, 1e-5, 1e-3])),
            pick([16, 32], [16, 32, 64]))


@pytest.mark.parametrize("seed", range(16))
def test_configurations_drawn_at_random(seed, tmp_path):
    cfg, page = _random_config(seed)
    tensors = plain.random_model(cfg, 100 + seed)
    t64 = {k: v.double() for k, v in tensors.items()}
    requests = _requests(cfg, [1, 23, 150, 9], seed=30 + seed)
    steps = traces.mixed(requests, max_live=3, sizes=(5, 2, 11, 3))
    refs = {rid: plain.forward(cfg, t64, list(toks)).numpy() for rid, toks in requests.items()}
    for dtype in ("float32", "bfloat16"):
        folder = _write(str(tmp_path / dtype), cfg, tensors, dtype)
        out = str(tmp_path / f"out_{dtype}")
        traces.replay_in_process(folder, dtype, steps, out, traces.live_token_peak(steps), page, max_live=4)
        got = traces.collect(steps, out, cfg["vocab"])
        whole_steps = traces.whole(requests)
        whole_out = str(tmp_path / f"whole_{dtype}")
        traces.replay_in_process(folder, dtype, whole_steps, whole_out, traces.live_token_peak(whole_steps), page)
        whole = traces.collect(whole_steps, whole_out, cfg["vocab"])
        errors = []
        for rid, toks in requests.items():
            assert sorted(got[rid]) == list(range(len(toks)))
            for pos, row in sorted(got[rid].items()):
                assert np.isfinite(row).all()
                errors.append((_row_error(row, refs[rid][pos]), rid, pos))
                if dtype == "float32":
                    cut = _row_error(row, whole[rid][pos].astype(np.float64))
                    assert cut <= CUT_TOLERANCE[dtype], f"configuration {seed}: request {rid} position {pos} depends on the cut ({cut:.3e}): {json.dumps(cfg)}"
        # float32 is held row by row, but for the few positions that a drawn design conditions badly (a temperature that
        # multiplies sharp queries by ten and more makes scores of hundreds, whose rounding the softmax magnifies); the
        # bfloat16 run of these very narrow layers is held by its median row, which a wrong shape or kernel choice would move
        ranked = sorted(errors)
        if dtype == "float32":
            assert ranked[int(0.97 * len(ranked))][0] <= TOLERANCE[dtype] and ranked[-1][0] <= 10 * TOLERANCE[dtype], \
                f"configuration {seed}: request {ranked[-1][1]} position {ranked[-1][2]} (error {ranked[-1][0]:.3e}): {json.dumps(cfg)}"
        else:
            assert ranked[len(ranked) // 2][0] <= 0.05, f"configuration {seed} in bfloat16: median row error {ranked[len(ranked) // 2][0]:.3e}: {json.dumps(cfg)}"
