"""Bilolorn, Kusolorn, Desilorn and Zinunex beside the Qwen3 dense decoder at equal layer sizes: prefill and decode throughput
through the model runner, and the time of every kernel of a step with the share of its roofline that it reaches.

``bench.py --designs`` runs this (``--design-names kusolorn,qwen3`` chooses the designs; ``kusolorn_attention`` is
Kusolorn with windowed attention and a dense feed-forward in every layer, the closest model to Desilorn);
``python -m cuinfer_b200.bench_designs [--sizes small,large] [--designs kusolorn,qwen3]`` does the same.
Weights are random, drawn on the device; the models have a few layers only (the figures are per step of that model;
what is compared is one design against the other at the same sizes, and every kernel against its own roofline).

Kernel times are taken in place: while one eager step runs, every call through ``cuinfer_b200.kernels`` is made once
for its result and then repeated between two CUDA events on the same arguments (the repeats change nothing that later
kernels read differently: a norm that adds into the residual is repeated on a copy).  The roofline of a call is the larger
of its algorithmic bytes over the measured copy bandwidth and its FLOPs over the measured bfloat16 peak
(``MEASURED_PEAKS.json``, else the fallback figures).
"""
from __future__ import annotations

import argparse
import dataclasses
import json
import os
import statistics
import sys
import tempfile
from typing import Callable, Dict, List

import torch

from . import kernels

# Layer sizes that resemble real models.  Bilolorn: H heads of (dim + rot_dim) query/key and vdim value dimensions,
# latents of q_rank / kv_rank, a dense squared-ReLU layer first and table-routed experts after it.  Qwen3: the dense
# decoder with the same width, head count and feed-forward size.
SIZES = {
    "small": dict(width=1024, heads=16, dim=64, rot_dim=32, vdim=64, q_rank=512, kv_rank=256, ff=3072, experts=16, top=2,
                  expert_ff=768, shared_ff=768, vocab=32768, layers=4, kv_heads=8, head_dim=128,
                  window=512, keep_first=4, side_dim=64, delta_heads=16, delta_kv_heads=8, delta_dim=64, delta_vdim=64,
                  memory_heads=4, memory_dim=128, memory_vdim=256),
    "medium": dict(width=2048, heads=16, dim=128, rot_dim=64, vdim=128, q_rank=1024, kv_rank=384, ff=6144, experts=16, top=2,
                   expert_ff=1024, shared_ff=1536, vocab=32768, layers=4, kv_heads=8, head_dim=128,
                   window=1024, keep_first=4, side_dim=128, delta_heads=16, delta_kv_heads=8, delta_dim=128, delta_vdim=128,
                   memory_heads=4, memory_dim=256, memory_vdim=512),
    "large": dict(width=4096, heads=32, dim=128, rot_dim=64, vdim=128, q_rank=1536, kv_rank=512, ff=12288, experts=32, top=2,
                  expert_ff=1536, shared_ff=3072, vocab=32768, layers=4, kv_heads=8, head_dim=128,
                  window=1024, keep_first=4, side_dim=256, delta_heads=32, delta_kv_heads=16, delta_dim=128, delta_vdim=128,
                  memory_heads=8, memory_dim=256, memory_vdim=512),
}


def bilolorn_config(s: dict) -> dict:
    mixer = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "q_rank": s["q_rank"],
             "kv_rank": s["kv_rank"], "scale": (s["dim"] + s["rot_dim"]) ** -0.5, "rot": {"base": 10000.0, "dims": s["rot_dim"]}}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"]},
           "shared": {"ff": s["shared_ff"]}}
    layers = [{"type": "latent_attention", "mixer": mixer, "mlp": dense if i == 0 else moe} for i in range(s["layers"])]
    return {"architecture": "Bilolorn", "architectures": ["Bilolorn"], "vocab": s["vocab"], "width": s["width"],
            "embedding": {"scale": 1.0}, "norm": {"eps": 1e-5}, "layers": layers, "loop": {"start": 0, "stop": 0, "times": 1}}


def kusolorn_config(s: dict) -> dict:
    """Four layers, one of each kind and a second attention layer that mixes the first one's values in: windowed
    attention with the Qwen3 arm's head counts and head size, the gated delta rule, the matrix memory; a dense
    feed-forward first and routed experts after it; the per-layer token input."""
    attention = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["head_dim"], "vdim": s["head_dim"], "scale": s["head_dim"] ** -0.5,
                 "softcap": 30.0, "v_mix": True, "mask": {"size": s["window"], "keep_first": s["keep_first"]},
                 "rot": {"base": 1000000.0, "dims": s["head_dim"] // 2, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 8192}}}
    delta = {"heads": s["delta_heads"], "kv_heads": s["delta_kv_heads"], "dim": s["delta_dim"], "vdim": s["delta_vdim"], "conv": 4}
    memory = {"heads": s["memory_heads"], "dim": s["memory_dim"], "vdim": s["memory_vdim"], "gate_cap": 15.0}
    dense = {"kind": "dense", "ff": s["ff"]}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"]}, "expert": {"ff": s["expert_ff"], "limit": 7.0}}
    kinds = [("attention", attention, dense), ("delta", delta, moe), ("attention", attention, moe), ("mlstm", memory, moe)]
    layers = [{"type": t, "mixer": m, "mlp": f} for t, m, f in (kinds * ((s["layers"] + 3) // 4))[:s["layers"]]]
    return {"architecture": "Kusolorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "token_side": {"dim": s["side_dim"]}, "layers": layers}


def kusolorn_attention_config(s: dict) -> dict:
    """Kusolorn with windowed attention and a dense feed-forward in every layer and no per-layer token input: the model
    whose kernels are closest to Desilorn's, at the same sizes."""
    attention = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["head_dim"], "vdim": s["head_dim"], "scale": s["head_dim"] ** -0.5,
                 "softcap": 30.0, "v_mix": False, "mask": {"size": s["window"], "keep_first": s["keep_first"]},
                 "rot": {"base": 1000000.0, "dims": s["head_dim"] // 2}}
    layers = [{"type": "attention", "mixer": attention, "mlp": {"kind": "dense", "ff": s["ff"]}} for _ in range(s["layers"])]
    return {"architecture": "Kusolorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "layers": layers}


def desilorn_config(s: dict) -> dict:
    """Both kinds of attention in turn (the sliding window with its temperature, distance bias and learned sinks; chunks
    with head norm and rotation in halves), the Qwen3 arm's head counts and head size, a dense feed-forward in every
    layer, four residual streams, no looped span (every arm runs the same number of layers)."""
    common = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["head_dim"], "vdim": s["head_dim"], "scale": s["head_dim"] ** -0.5,
              "mask": {"size": s["window"]}}
    sliding = dict(common, q_temp={"coef": 0.1, "every": 256})
    chunks = dict(common, rot={"base": 1000000.0, "dims": s["head_dim"] // 2})
    layers = [{"type": "attention" if i % 2 == 0 else "attention_2", "mixer": sliding if i % 2 == 0 else chunks,
               "mlp": {"kind": "dense", "ff": s["ff"]}} for i in range(s["layers"])]
    return {"architecture": "Desilorn", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6}, "streams": s.get("streams", 4),
            "layers": layers}


def zinunex_config(s: dict) -> dict:
    """Four layers: attention over a cached latent with a sliding window (Bilolorn's head sizes and latent size), two
    layers of grouped-query attention with a sink whose values are its keys (the Qwen3 arm's head counts and head size),
    and a second latent layer that reads the first one's cache; a mixture of ungated experts under a scored router with
    a gated shared expert in every layer (Bilolorn's expert sizes); the per-layer token input."""
    rot = {"base": 1000000.0, "dims": s["rot_dim"], "scaling": {"factor": 8.0, "original": 4096, "fast": 32.0, "slow": 1.0}}
    latent = {"heads": s["heads"], "dim": s["dim"], "rot_dim": s["rot_dim"], "vdim": s["vdim"], "kv_rank": s["kv_rank"],
              "scale": (s["dim"] + s["rot_dim"]) ** -0.5, "mask": {"size": s["window"]}, "rot": rot}
    sink = {"heads": s["heads"], "kv_heads": s["kv_heads"], "dim": s["head_dim"], "vdim": s["head_dim"], "scale": s["head_dim"] ** -0.5,
            "rot": {"base": 50000.0, "dims": s["head_dim"], "scaling": {"factor": 8.0}}}
    moe = {"kind": "moe", "router": {"experts": s["experts"], "top": s["top"], "scale": 2.0, "groups": {"count": 4, "keep": 2}},
           "expert": {"ff": s["expert_ff"]}, "shared": {"ff": s["shared_ff"]}}
    kinds = [("latent_attention", latent), ("attention", sink), ("attention", sink), ("latent_attention", dict(latent, kv_from=0))]
    layers = [{"type": t, "mixer": dict(m, kv_from=i // 4 * 4) if "kv_from" in m else m, "mlp": moe}
              for i, (t, m) in enumerate((kinds * ((s["layers"] + 3) // 4))[:s["layers"]])]
    return {"architecture": "Zinunex", "vocab": s["vocab"], "width": s["width"], "norm": {"eps": 1e-6},
            "token_side": {"dim": s["side_dim"]}, "layers": layers}


def qwen3_config(s: dict) -> dict:
    return dict(architectures=["Qwen3ForCausalLM"], num_hidden_layers=s["layers"], hidden_size=s["width"],
                num_attention_heads=s["heads"], num_key_value_heads=s["kv_heads"], head_dim=s["head_dim"],
                intermediate_size=s["ff"], vocab_size=s["vocab"], rope_theta=1000000.0, rms_norm_eps=1e-6,
                tie_word_embeddings=False, max_position_embeddings=8192, torch_dtype="bfloat16")


def load_peaks() -> dict:
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            return dict(json.load(fh), source="measured")
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def make_runner(config: dict, pages: int, max_seqs: int, graphs: bool):
    from .config import EngineConfig
    from .engine.runner import ModelRunner
    from .weights import write_random_model

    folder = tempfile.mkdtemp(prefix="cuinfer_b200_designs_")
    write_random_model(folder, config, 7, std=0.02, gain_std=0.02, dtype="bfloat16", generator="counter", materialize=False)
    cfg = EngineConfig(model_path=folder, block_size=16, dtype="bfloat16", num_blocks=pages, max_num_seqs=max_seqs,
                       max_num_scheduled_tokens=1 << 20, enable_cuda_graph=graphs)
    return ModelRunner(folder, cfg)


# ---- bytes and FLOPs of a call, from its arguments ----------------------------------------------------------------------
def _nbytes(*tensors) -> int:
    return sum(t.numel() * t.element_size() for t in tensors if isinstance(t, torch.Tensor))


def _attention_cost(q_rows: int, heads: int, qk: int, v: int, kv_row_bytes: int, lens_q: List[int], lens_k: List[int]):
    """Causal attention of requests with lens_q new tokens at the end of lens_k keys: FLOPs of both products over the
    visible pairs; bytes of the keys/values read once per request plus the queries and outputs."""
    pairs = sum(n * (k - n) + n * (n + 1) // 2 for n, k in zip(lens_q, lens_k))
    flops = 2.0 * pairs * heads * (qk + v)
    return flops, sum(lens_k) * kv_row_bytes + q_rows * heads * (qk + v) * 2


class KernelTimes:
    """Patches ``kernels.<name>`` for the duration of one step (see the module's head)."""

    def __init__(self, step_lens: Dict[str, List[int]], reps: int = 5) -> None:
        self.reps = reps
        self.lens = step_lens
        self.rows: List[dict] = []
        self._saved: Dict[str, Callable] = {}

    def _timed(self, name: str, fn: Callable, cost: Callable):
        def wrapper(*args, **kw):
            fn(*args, **kw)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            rep_args = args
            if name in ("sandwich_layernorm", "add_rmsnorm", "rms_stream"):           # they add into their first argument
                rep_args = (args[0].clone(),) + tuple(args[1:])
            # the repeats are recorded into a CUDA graph and the graph is timed: the device's time, not Python's
            torch.cuda.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(self.reps):
                    fn(*rep_args, **kw)
            graph.replay()
            torch.cuda.synchronize()
            a.record()
            graph.replay()
            b.record()
            torch.cuda.synchronize()
            del graph
            flops, nbytes = cost(*args, **kw)
            self.rows.append({"kernel": name, "ms": a.elapsed_time(b) / self.reps, "flops": float(flops), "bytes": float(nbytes)})
        return wrapper

    def __enter__(self):
        lq, lk = self.lens["q"], self.lens["k"]

        def rowwise(*a, **kw):
            return 0.0, _nbytes(*a, *kw.values())

        def windowed(q, heads, qk, v, window, keep, chunked=False):
            """Attention in which a query sees at most ``window`` keys and ``keep`` kept ones (with ``chunked`` the keys of
            its own chunk of ``window`` positions): FLOPs over the visible pairs, bytes of the visible rows of the cache
            read once per request."""
            pairs, rows = 0, 0
            for n, k in zip(lq, lk):
                for p in range(k - n, k):
                    pairs += (p % window + 1) if chunked and window else min(p + 1, (window + keep) if window else p + 1)
                rows += min(k, k - (k - n) // window * window) if chunked and window else min(k, (window + keep + n) if window else k)
            return 2.0 * pairs * heads * (qk + v), rows * (qk + v) * 2 + q.shape[0] * heads * (qk + v) * 2

        def latent(q, heads, rk, dr, window):
            """Attention over cached latent rows of rk + dr values that every head reads: all earlier keys, or the last
            ``window``."""
            if not window:
                return _attention_cost(q.shape[0], heads, rk + dr, rk, (rk + dr) * 2, lq, lk)
            flops, _ = windowed(q, heads, rk + dr, rk, window, 0)
            rows = sum(min(k, window + n) for n, k in zip(lq, lk))
            return flops, rows * (rk + dr) * 2 + q.shape[0] * heads * (2 * rk + dr) * 2

        def hyper(streams, y, write, read, norm, out, read_out=None):
            """One pass over the streams: read once, written once when a sub-layer's output is outstanding."""
            return 0.0, _nbytes(streams) * (2 if y is not None else 1) + _nbytes(y, out, read_out)

        def scan(tokens, heads, d, dv, per_pair, state):
            """A recurrence over a matrix per head: ``per_pair`` operations per token and matrix element; the state is read
            and written once, the inputs read once."""
            return float(per_pair) * tokens * heads * d * dv, 2 * _nbytes(state) * len(lq) / max(1, state.shape[0]) + tokens * heads * (2 * d + 2 * dv) * 4

        costs = {
            "rms_stream": rowwise, "hyper_stream": hyper, "hyper_gather": lambda st, y, w, idx, out: (0.0, (st.shape[1] + 1) * _nbytes(out)),
            "gelu_tanh": rowwise, "router_topk": rowwise, "head_rms_gate": rowwise,
            "window_attention_prep": lambda qkv, *a, **k: (0.0, 2 * _nbytes(qkv)),
            "window_attention_generic": lambda q, out, cache, bt, pos, tr, H, G, d, dv, scale, cap, window, keep, **kw:
                windowed(q, H, d, dv, window, keep, kw.get("chunked", False)),
            "window_attention_mma": lambda q, out, cache, bt, qsl, sl, ql, H, G, d, dv, scale, cap, window, keep, **kw:
                windowed(q, H, d, dv, window, keep, kw.get("chunked", False)),
            "mlstm_scan": lambda q, k, v, gates, ib, fb, cap, qs, state, qsl, slots, out, H, d, dv, **kw: scan(out.shape[0], H, d, dv, 4, state),
            "delta_scan": lambda qkv, gates, al, db, state, qsl, slots, out, G, H, d, dv: scan(out.shape[0], H, d, dv, 6, state),
            "delta_prep": lambda x, taps, cs, qsl, tr, slots, G, H, d, dv, ue, qs, out: (0.0, _nbytes(out) + out.numel() * x.element_size()),
            "sandwich_layernorm": rowwise, "add_rmsnorm": rowwise, "relu_squared": rowwise, "sigmoid_gate": rowwise,
            "silu_mul": rowwise, "embedding_gather": lambda ids, table, out, *a, **k: (0.0, 2 * _nbytes(out)),
            "gather_rows": lambda res, delta, idx, out: (0.0, 2 * _nbytes(out)),
            "latent_prep": lambda proj, q_off, rq, kv_off, rk, dr, *a, **k: (0.0, proj.shape[0] * (2 * rq + 2 * (rk + dr)) * 2),
            "qk_norm_rope_kv_write": lambda qkv, *a, **k: (0.0, 2 * _nbytes(qkv)),
            "latent_attention_mma": lambda q_abs, q, out, cache, bt, qsl, sl, ql, freq, rd, sinks, H, dn, rk, dr, *a, **k:
                latent(q, H, rk, dr, k.get("window", 0)),
            "latent_attention_generic": lambda q_abs, q, out, cache, bt, qsl, sl, tr, pos, freq, rd, sinks, H, dn, rk, dr, *a, **k:
                latent(q, H, rk, dr, k.get("window", 0)),
            "router_scored_topk": rowwise,
            "attention_tcgen05": lambda qkv, out, cache, bt, qsl, sl, lens, nq, nkv, d, *a, **k:
                _attention_cost(qkv.shape[0], nq, d, d, 2 * nkv * d * 2, lq, lk),
            "paged_attention_prefill": lambda qkv, out, cache, bt, qsl, sl, lens, nq, nkv, d, *a, **k:
                _attention_cost(qkv.shape[0], nq, d, d, 2 * nkv * d * 2, lq, lk),
            "paged_attention_decode": lambda qkv, out, cache, bt, sl, nq, nkv, d, *a, **k:
                _attention_cost(qkv.shape[0], nq, d, d, 2 * nkv * d * 2, lq, lk),
            "moe_table_feed_forward": lambda h, ids, table, gate_up, down, base, out, **kw:
                (2.0 * h.shape[0] * table.shape[1] * (gate_up.shape[1] + down.shape[2]) * h.shape[1],
                 min(h.shape[0] * table.shape[1], gate_up.shape[0]) * (gate_up.shape[1] + down.shape[2]) * h.shape[1] * 2 + 3 * _nbytes(h)),
            "gemm_generic_batched": lambda a, w, out: (2.0 * a.shape[0] * a.shape[1] * a.shape[2] * w.shape[1], _nbytes(a, w, out)),
            "gemm_tcgen05": lambda a, w, out, **k: (2.0 * a.shape[0] * a.shape[1] * w.shape[0], _nbytes(a, w, out)),
            "gemm_skinny": lambda w, out, **k: (2.0 * out.shape[0] * w.shape[0] * w.shape[1], _nbytes(w, out)),
            "gemm_wstream": lambda a, w, out, **k: (2.0 * a.shape[0] * a.shape[1] * w.shape[0], _nbytes(a, w, out)),
        }
        for name, cost in costs.items():
            self._saved[name] = getattr(kernels, name)
            setattr(kernels, name, self._timed(name, self._saved[name], cost))
        return self

    def __exit__(self, *exc):
        for name, fn in self._saved.items():
            setattr(kernels, name, fn)

    def summary(self, peaks: dict) -> List[dict]:
        by: Dict[str, dict] = {}
        for r in self.rows:
            roof_ms = max(r["bytes"] / (peaks["hbm_gbs"] * 1e9), r["flops"] / (peaks["bf16_tflops"] * 1e12)) * 1e3
            e = by.setdefault(r["kernel"], {"kernel": r["kernel"], "calls": 0, "ms": 0.0, "roofline_ms": 0.0})
            e["calls"] += 1
            e["ms"] += r["ms"]
            e["roofline_ms"] += roof_ms
        out = []
        for e in sorted(by.values(), key=lambda e: -e["ms"]):
            e["of_roofline"] = round(e["roofline_ms"] / e["ms"], 4) if e["ms"] > 0 else None
            e["ms"], e["roofline_ms"] = round(e["ms"], 4), round(e["roofline_ms"], 4)
            out.append(e)
        return out


# ---- one design at one size -----------------------------------------------------------------------------------------------
def measure(design: str, size: str, prefill_tokens: int, batch: int, context: int, steps: int, peaks: dict) -> dict:
    from .engine.runner import StepEntry

    s = SIZES[size]
    config = {"bilolorn": bilolorn_config, "kusolorn": kusolorn_config, "kusolorn_attention": kusolorn_attention_config,
              "desilorn": desilorn_config, "zinunex": zinunex_config, "qwen3": qwen3_config}[design](s)
    pages = (batch * (context + steps + 64) + prefill_tokens) // 16 + 64
    runner = make_runner(config, pages, max_seqs=max(batch, 8), graphs=True)
    gen = torch.Generator().manual_seed(5)
    prompt = torch.randint(0, s["vocab"], (prefill_tokens,), generator=gen).tolist()

    def prefill_once() -> float:
        assert runner.reserve("p", prefill_tokens)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        runner.step([StepEntry("p", prompt, [prefill_tokens - 1])])
        b.record()
        torch.cuda.synchronize()
        runner.release("p")
        return a.elapsed_time(b)

    times = [prefill_once() for _ in range(8)][3:]
    prefill_ms = statistics.median(times)
    with_graphs = runner.config
    runner.config = dataclasses.replace(with_graphs, enable_cuda_graph=False)
    with KernelTimes({"q": [prefill_tokens], "k": [prefill_tokens]}) as kt:
        prefill_once()
    prefill_kernels = kt.summary(peaks)
    runner.config = with_graphs

    # decode: `batch` requests of `context` tokens, then `steps` timed steps through the decode graphs
    ids = [f"d{i}" for i in range(batch)]
    for rid in ids:
        toks = torch.randint(0, s["vocab"], (context,), generator=gen).tolist()
        assert runner.reserve(rid, context)
        runner.step([StepEntry(rid, toks, [])])

    def decode_steps(n: int, eager: bool = False) -> None:
        for _ in range(n):
            entries = [StepEntry(rid, [1], [0]) for rid in ids]
            for rid in ids:
                assert runner.reserve(rid, 1)
            runner.step(entries) if eager else runner.decode_step(entries)

    decode_steps(4)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    decode_steps(steps)
    b.record()
    torch.cuda.synchronize()
    decode_ms = a.elapsed_time(b) / steps
    held = context + 4 + steps
    with KernelTimes({"q": [1] * batch, "k": [held + 1] * batch}) as kt:
        decode_steps(1, eager=True)
    decode_kernels = kt.summary(peaks)
    params = sum(t.numel() for t in _weights(runner))
    out = {"design": design, "size": size, "layers": s["layers"], "parameters": params,
           "prefill": {"tokens": prefill_tokens, "ms": round(prefill_ms, 3), "tokens_per_s": round(prefill_tokens / prefill_ms * 1e3)},
           "decode": {"batch": batch, "context": held, "ms_per_step": round(decode_ms, 4), "tokens_per_s": round(batch / decode_ms * 1e3)},
           "prefill_kernels": prefill_kernels, "decode_kernels": decode_kernels, "peaks": peaks.get("source")}
    del runner
    torch.cuda.empty_cache()
    return out


def _weights(runner) -> List[torch.Tensor]:
    seen, out = set(), []

    def walk(obj, depth=0):
        if isinstance(obj, torch.Tensor):
            if obj.data_ptr() not in seen and obj.dtype in (torch.bfloat16, torch.float32) and obj.numel() > 1:
                seen.add(obj.data_ptr())
                out.append(obj)
        elif depth < 4 and hasattr(obj, "__dict__"):
            for v in vars(obj).values():
                walk(v, depth + 1)
        elif depth < 4 and isinstance(obj, (list, tuple)):
            for v in obj:
                walk(v, depth + 1)

    walk(runner.model.embedding)
    walk(runner.model.lm_head)
    for part in runner.model.parts():
        walk(part)
    return out


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m cuinfer_b200.bench_designs", description=__doc__.split("\n\n")[0])
    ap.add_argument("--sizes", default="small,large")
    ap.add_argument("--designs", default="bilolorn,qwen3")
    ap.add_argument("--prefill-tokens", type=int, default=2048)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=32)
    args = ap.parse_args(argv)
    peaks = load_peaks()
    for size in args.sizes.split(","):
        for design in args.designs.split(","):
            print(json.dumps(measure(design, size, args.prefill_tokens, args.batch, args.context, args.steps, peaks)), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
