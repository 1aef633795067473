"""Grouped-query attention with sizes of its own for keys and values and a choice of what happens around the scores:
a norm of queries and keys, a query temperature, a capped score, a distance bias, a sliding window that keeps the first
tokens of a sequence visible or a mask of chunks, and a sink in the softmax's denominator.

For the mixer's input h, H query heads and G key/value heads (query head i uses key/value head ``i // (H / G)``), query
and key size ``dim``, value size ``vdim``:

* ``q = Wq h``, ``k = Wk h``, ``v = Wv h``; with ``bias`` each has a bias (the tensor's name plus ``bias_suffix``),
  added in 32 bits; with ``value_from_key`` there is no ``Wv``: a token's value is its key as projected, before norm and
  rotation (``vdim == dim``);
* ``qk_norm``: ``"unit"`` divides each head of q and k by its root mean square over ``dim`` (``eps`` inside the root),
  ``"gain"`` also multiplies by a gain of ``dim`` values shared by all heads (one for q, one for k), ``"none"`` leaves
  them; the norm comes after the position encoding or, with ``norm_first``, before it;
* the position encoding (rotary, on the first ``rotary_dim`` values of each head; ``rope_interleaved`` pairs
  neighbours, ``rope_half`` pairs i with ``i + rotary_dim / 2``) on q and k;
* ``q_temp = (coef, every)``: the query at position p is multiplied by ``1 + coef * ln(floor((p + 1) / every) + 1)``;
* value mixing (``value_mix``): the ``"source"`` layer publishes its values of the step's tokens; a ``"mixed"`` layer
  caches ``(1 - m) v + m v_source`` with its own learned number ``m``;
* ``score = scale * q . k``, then ``softcap * tanh(score / softcap)`` when a cap is given, then, with
  ``distance_bias = c``, minus ``2 ** (-c (h + 1) / H) * (i - j)`` for head h;
* the query at position i sees key j when ``j <= i`` and (no window, or ``i - j < window``, or ``j < keep_first``);
  with ``chunked`` the window is a chunk counted from position 0: ``j // window == i // window``;
* softmax; ``sink="learned"`` adds ``exp(sink_h)``, a learned number per head, to the denominator and ``sink="zero"``
  adds one (a sink has no key and no value, is not scaled and gets no bias); output projection ``Wo`` on the
  concatenated heads.

The cache holds a token's key and (mixed) value side by side: ``PagedCacheNeed(G, dim + vdim, window, planes=1,
keep_first, chunked)``; pages behind the window (before the chunk) are given back, except those of the kept tokens.

Spec: ``PartSpec("window_attention", num_heads, num_kv_heads, dim, vdim, scale, softcap, window, keep_first, chunked,
qk_norm, norm_first, eps, bias, bias_suffix, q_temp, distance_bias, sink, value_mix, value_from_key, position=PartSpec(...),
names=(q, k, v, o, mix, q_norm, k_norm, sink))``.  ``qk_unit_norm`` (True / False) is the older spelling of ``qk_norm``
``"unit"`` / ``"none"``.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .. import kernels
from . import attention_dispatch
from .base import Mixer
from .context import StepContext
from .linear import Linear
from .registry import MIXERS, POSITION_ENCODINGS
from .spec import PagedCacheNeed, PartSpec, TensorSpec

VALUE_MIX_KEY = "window_attention.values"


@MIXERS.register("window_attention")
class WindowAttention(Mixer):
    accepts_lazy_norm = True       # the q/k/v projection can compute the norm of its input itself

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads = int(spec.num_heads)
        self.num_kv_heads = int(spec.num_kv_heads)
        self.dim = int(spec.dim)
        self.vdim = int(spec.vdim)
        if self.num_heads <= 0 or self.num_kv_heads <= 0 or self.num_heads % self.num_kv_heads:
            raise ValueError("window_attention: num_heads must be a positive multiple of num_kv_heads")
        if not (0 < self.dim <= 512 and 0 < self.vdim <= 512):
            raise ValueError(f"window_attention: key size {self.dim} / value size {self.vdim} are beyond what the kernels take (512)")
        self.scale = float(spec.scale)
        self.softcap = float(spec.get("softcap") or 0.0)
        self.window = int(spec.get("window") or 0)
        self.keep_first = int(spec.get("keep_first") or 0) if self.window else 0
        self.chunked = bool(spec.get("chunked", False)) and bool(self.window)
        if self.chunked and self.keep_first:
            raise ValueError("window_attention: a mask of chunks keeps no first tokens")
        self.eps = float(spec.get("eps", 1e-6))
        self.qk_norm = spec.get("qk_norm") or ("unit" if spec.get("qk_unit_norm", True) else "none")
        if self.qk_norm not in ("unit", "gain", "none"):
            raise ValueError(f"window_attention: qk_norm must be 'unit', 'gain' or 'none', got {self.qk_norm!r}")
        self.norm_first = bool(spec.get("norm_first", False))
        self.has_bias = bool(spec.get("bias", False))
        temp = spec.get("q_temp")
        self.q_temp = (float(temp[0]), int(temp[1])) if temp else None
        if self.q_temp and self.q_temp[1] <= 0:
            raise ValueError("window_attention: the query temperature's period must be positive")
        bias = spec.get("distance_bias")
        self.distance_bias = float(bias) if bias else 0.0
        self.sink = spec.get("sink")
        if self.sink not in (None, "learned", "zero"):
            raise ValueError(f"window_attention: sink must be None, 'learned' or 'zero', got {self.sink!r}")
        self.value_mix = spec.get("value_mix")
        if self.value_mix not in (None, "source", "mixed"):
            raise ValueError(f"window_attention: value_mix must be None, 'source' or 'mixed', got {self.value_mix!r}")
        self.value_from_key = bool(spec.get("value_from_key", False))
        if self.value_from_key and (self.vdim != self.dim or self.value_mix):
            raise ValueError("window_attention: values taken from the keys have the keys' size and are not mixed")
        pos_spec: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        if self.position.rotary_dim > self.dim:
            raise ValueError("window_attention: rotary_dim exceeds dim")
        if self.position.rotary_dim and not hasattr(self.position, "frequencies"):
            raise ValueError("window_attention: the position encoding must hand out frequencies (rope_interleaved)")
        names = tuple(spec.get("names", ("q", "k", "v", "o", "vmix")))
        q, k, v, o, mix, q_norm, k_norm, sink = names + ("q.norm", "k.norm", "sink")[len(names) - 5:]
        p = prefix
        self.q_size, self.k_size, self.v_size = self.num_heads * self.dim, self.num_kv_heads * self.dim, self.num_kv_heads * self.vdim
        if self.value_from_key:
            self.qkv = Linear([f"{p}.{q}", f"{p}.{k}"], [self.q_size, self.k_size], hidden_size, dtype)
        else:
            self.qkv = Linear([f"{p}.{q}", f"{p}.{k}", f"{p}.{v}"], [self.q_size, self.k_size, self.v_size], hidden_size, dtype)
        self.rot_gain = float(getattr(self.position, "magnitude", 1.0))
        self.o = Linear([f"{p}.{o}"], [hidden_size], self.num_heads * self.vdim, dtype)
        self._mix_spec = TensorSpec(f"{p}.{mix}", (), init="zeros") if self.value_mix else None
        self.mix: Optional[torch.Tensor] = None
        suffix = spec.get("bias_suffix", ".b")
        self._bias_specs = [TensorSpec(f"{p}.{n}{suffix}", (size,), init="zeros")
                            for n, size in ((q, self.q_size), (k, self.k_size), (v, self.v_size))[:2 if self.value_from_key else 3]] if self.has_bias else []
        self._gain_specs = [TensorSpec(f"{p}.{n}", (self.dim,), keep_stored_precision=True, init="ones")
                            for n in (q_norm, k_norm)] if self.qk_norm == "gain" else []
        self._sink_spec = TensorSpec(f"{p}.{sink}", (self.num_heads,), keep_stored_precision=True, init="zeros") if self.sink == "learned" else None
        self.bias: Optional[torch.Tensor] = None          # 32-bit [q | k | v] biases
        self.q_gain: Optional[torch.Tensor] = None
        self.k_gain: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None         # 32-bit [H]: the learned numbers, or zeros
        self.slopes: Optional[torch.Tensor] = None        # 32-bit [H]

    def tensors(self) -> List[TensorSpec]:
        return (self.qkv.tensors() + self._bias_specs + self._gain_specs + self.o.tensors()
                + ([self._mix_spec] if self._mix_spec else []) + ([self._sink_spec] if self._sink_spec else [])
                + self.position.tensors())

    def load(self, store) -> None:
        self.qkv.load(store)
        self.o.load(store)
        device = self.o.weight.device
        if self._mix_spec is not None:
            self.mix = store.get(self._mix_spec).reshape(1).contiguous()
        if self._bias_specs:
            self.bias = torch.cat([store.get(b).float().reshape(-1) for b in self._bias_specs]).contiguous()
        if self._gain_specs:
            self.q_gain, self.k_gain = (store.get(g).float().contiguous() for g in self._gain_specs)
        if self._sink_spec is not None:
            self.sinks = store.get(self._sink_spec).float().contiguous()
        elif self.sink == "zero":
            self.sinks = torch.zeros(self.num_heads, dtype=torch.float32, device=device)
        if self.distance_bias:
            H = self.num_heads
            self.slopes = torch.tensor([2.0 ** (-self.distance_bias * (h + 1) / H) for h in range(H)],
                                       dtype=torch.float64).to(torch.float32).to(device)
        self.position.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.qkv.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    def cache_need(self) -> Optional[PagedCacheNeed]:
        return PagedCacheNeed(self.num_kv_heads, self.dim + self.vdim, self.window or None, planes=1,
                              keep_first=self.keep_first, chunked=self.chunked)

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        return self.qkv.workspace_bytes(tokens) + tokens * self.num_heads * self.vdim * width + self.o.workspace_bytes(tokens)

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        kv = ctx.paged_kv(run)
        qkv = self.qkv.forward(x)
        v_first = None
        if self.value_mix == "source":
            ctx.shared[VALUE_MIX_KEY] = qkv[:, self.q_size + self.k_size:]        # stays unmixed: only the cache gets values
        elif self.value_mix == "mixed":
            v_first = ctx.shared.get(VALUE_MIX_KEY)
            if v_first is None or v_first.shape != (qkv.shape[0], self.v_size):
                raise RuntimeError("window_attention: no earlier layer of this step published values of this shape to mix in")
        freq = self.position.frequencies() if self.position.rotary_dim else None
        kernels.window_attention_prep(qkv, ctx.positions, kv.group.slot_mapping if kv.writes else None, freq,
                                      self.position.rotary_dim, self.eps, self.num_heads, self.num_kv_heads, self.dim, self.vdim,
                                      v_first, self.mix if v_first is not None else None, kv.cache if kv.writes else None,
                                      bias=self.bias, norm=self.qk_norm != "none", q_gain=self.q_gain, k_gain=self.k_gain,
                                      norm_first=self.norm_first, rot_half=getattr(self.position, "layout", "") == "half",
                                      q_temp=self.q_temp, value_from_key=self.value_from_key, rot_gain=self.rot_gain)
        out = torch.empty((qkv.shape[0], self.num_heads * self.vdim), dtype=qkv.dtype, device=qkv.device)
        attention_dispatch.window_attention(qkv, out, kv, ctx, self.num_heads, self.num_kv_heads, self.dim, self.vdim,
                                            self.scale, self.softcap, self.window, self.keep_first, chunked=self.chunked,
                                            slopes=self.slopes, sinks=self.sinks)
        return self.o.forward(out)
