"""Causal attention through latents: queries, keys and values are low-rank, and only the key/value latent is cached.

For the mixer's input h (one row per token), with H heads, per head ``dim`` unrotated and ``rot_dim`` rotated
query/key dimensions and ``vdim`` value dimensions:

* queries: ``c_q = rmsnorm(Dq h)`` (rank ``q_rank``), ``q = Uq c_q``, laid out head by head as [dim | rot_dim];
* keys and values: ``Dkv h`` has ``kv_rank + rot_dim`` rows; the first ``kv_rank``, RMS-normed, are the latent ``c``,
  the rest is ONE rotary key part shared by all heads.  Head h's keys are ``[Uk_h c | rot(k_r)]``, its values ``Uv_h c``;
* score = ``(q_plain . Uk_h c + rot(q_rot) . rot(k_r)) * scale``, causal, softmax in 32 bits whose denominator may also
  hold ``exp(sink_h)`` for a learned per-head number (no key, no value);
* the concatenated heads are multiplied by ``sigmoid(G h)`` (optional) and projected by ``O``.

The cache holds one row ``[c | rot(k_r)]`` per token and layer run (``PagedCacheNeed(1, kv_rank + rot_dim, planes=1)``).
The up-projections are applied on the query and output side, so that nothing per head is ever expanded for the keys a
step reads: ``q_abs_h = Uk_h^T q_plain_h`` (a batch of H small products), attention over the cached rows with values =
their first ``kv_rank`` columns, then ``Uv_h`` on the result (again a batch).  Steps of a forward:

  one stacked projection [Dq; Dkv; G] -> norms + rotary + cache write (one kernel) -> Uq -> q_abs (batched) ->
  attention -> Uv (batched) -> gate -> O.

Variants, each a parameter of the spec:

* ``q_rank`` absent or 0: the queries have no latent, ``q = Q h`` with one matrix (role ``q``);
* ``window`` w: the query at position i sees key j only when ``0 <= i - j < w`` (pages behind the window are given back);
* ``own_cache=False``: the layer has no ``Dkv`` (and no norm for it): it reads the rows ``[c | rot(k_r)]`` that an earlier
  layer cached (``ModelSpec.cache_source`` names it), with its own ``Uk``, ``Uv``, queries, window and everything else;
  ``kv_rank``, ``rot_dim`` and the rotation must be the earlier layer's;
* a position encoding with a ``magnitude`` multiplies cosine and sine by it, on queries and on the cached key part.

Spec: ``PartSpec("latent_attention", num_heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, eps, sink, gate, window,
own_cache, position=PartSpec(...), names={...})``; ``names`` maps the roles (dq, dq_norm, uq, q, dkv, dkv_norm, uk, uv, sink,
g, o) to tensor names relative to the mixer's prefix.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import kernels
from . import attention_dispatch
from . import gemm_dispatch  # noqa: F401  (sets the library products to 32-bit accumulation before the first one runs)
from .base import Mixer
from .context import StepContext
from .linear import Linear
from .registry import MIXERS, POSITION_ENCODINGS
from .spec import PagedCacheNeed, PartSpec, TensorSpec

_DEFAULT_NAMES = {"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                  "uv": "uv", "sink": "sink", "g": "g", "o": "o"}


def per_head_products(a: torch.Tensor, w: torch.Tensor, out: torch.Tensor) -> None:
    """``out[h] = a[h] @ w[h]^T`` for every head h; ``a [H, T, K]`` and ``out [H, T, N]`` are views of rows in which
    the heads lie side by side, ``w [H, N, K]`` is dense.  bfloat16 with sizes in multiples of 8: the library's
    strided batched product (as for the plain projections); else the FMA kernel, which is also the 32-bit path."""
    H, T, K = a.shape
    N = w.shape[1]
    if (a.dtype == torch.bfloat16 and out.dtype == torch.bfloat16 and K % 8 == 0 and N % 8 == 0
            and a.stride(1) % 8 == 0 and a.stride(0) % 8 == 0 and out.stride(1) % 8 == 0 and out.stride(0) % 8 == 0 and T > 0):
        torch.bmm(a, w.transpose(1, 2), out=out)
        kernels.launch_count += 1
        return
    kernels.gemm_generic_batched(a, w, out)


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.num_heads = int(spec.num_heads)
        self.dim = int(spec.dim)
        self.rot_dim = int(spec.rot_dim)
        self.vdim = int(spec.vdim)
        self.q_rank = int(spec.get("q_rank") or 0)           # 0: queries projected directly
        self.own_cache = bool(spec.get("own_cache", True))
        self.kv_rank = int(spec.kv_rank)
        self.eps = float(spec.eps)
        scale = spec.get("scale")
        self.scale = float(scale) if scale is not None else (self.dim + self.rot_dim) ** -0.5
        self.has_sink = bool(spec.get("sink", False))
        self.has_gate = bool(spec.get("gate", False))
        window = spec.get("window")
        self.window = int(window) if window else 0
        for name in ("num_heads", "dim", "vdim", "kv_rank"):
            if getattr(self, name) <= 0:
                raise ValueError(f"latent_attention: {name} must be positive")
        if self.rot_dim < 0 or self.q_rank < 0:
            raise ValueError("latent_attention: rot_dim and q_rank must not be negative")
        pos_spec: PartSpec = spec.get("position") or PartSpec("none")
        self.position = POSITION_ENCODINGS.get(pos_spec.kind)(pos_spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        if self.position.rotary_dim > self.rot_dim:
            raise ValueError("latent_attention: the encoding rotates more dimensions than the rotary part has")
        if self.position.rotary_dim and not hasattr(self.position, "frequencies"):
            raise ValueError("latent_attention: the position encoding must give its frequencies (no table is read)")
        names: Dict[str, str] = dict(_DEFAULT_NAMES)
        names.update(spec.get("names") or {})
        self.names = {role: f"{prefix}.{n}" for role, n in names.items()}
        H = self.num_heads
        self.q_size = H * (self.dim + self.rot_dim)
        self.v_size = H * self.vdim
        self.row = self.kv_rank + self.rot_dim                     # what a token keeps in the cache
        # one stacked projection of the mixer's input: [query latent, or the queries themselves | Dkv | G]
        self.q_cols = self.q_rank or self.q_size
        down_names = [self.names["dq"] if self.q_rank else self.names["q"]]
        down_sizes = [self.q_cols]
        if self.own_cache:
            down_names.append(self.names["dkv"])
            down_sizes.append(self.row)
        if self.has_gate:
            down_names.append(self.names["g"])
            down_sizes.append(self.v_size)
        self.down = Linear(down_names, down_sizes, hidden_size, dtype)
        self.uq = Linear([self.names["uq"]], [self.q_size], self.q_rank, dtype) if self.q_rank else None
        self.rot_gain = float(getattr(self.position, "magnitude", 1.0))
        self.o = Linear([self.names["o"]], [hidden_size], self.v_size, dtype)
        self.uk_t: Optional[torch.Tensor] = None     # [H, kv_rank, dim]: Uk per head, transposed for the query side
        self.uv: Optional[torch.Tensor] = None       # [H, vdim, kv_rank]
        self.q_gain: Optional[torch.Tensor] = None
        self.kv_gain: Optional[torch.Tensor] = None
        self.sinks: Optional[torch.Tensor] = None

    # ---- weights -------------------------------------------------------------------------------------------
    def _own_specs(self) -> Dict[str, TensorSpec]:
        n, H = self.names, self.num_heads
        out = {
            "uk": TensorSpec(n["uk"], (H * self.dim, self.kv_rank)),
            "uv": TensorSpec(n["uv"], (H * self.vdim, self.kv_rank)),
        }
        if self.q_rank:
            out["dq_norm"] = TensorSpec(n["dq_norm"], (self.q_rank,), keep_stored_precision=True, init="ones")
        if self.own_cache:
            out["dkv_norm"] = TensorSpec(n["dkv_norm"], (self.kv_rank,), keep_stored_precision=True, init="ones")
        if self.has_sink:
            out["sink"] = TensorSpec(n["sink"], (H,), keep_stored_precision=True, init="zeros")
        return out

    def tensors(self) -> List[TensorSpec]:
        return (self.down.tensors() + (self.uq.tensors() if self.uq else []) + self.o.tensors()
                + list(self._own_specs().values()) + self.position.tensors())

    def load(self, store) -> None:
        self.down.load(store)
        if self.uq:
            self.uq.load(store)
        self.o.load(store)
        own = self._own_specs()
        self.q_gain = store.get(own["dq_norm"]) if self.q_rank else None
        self.kv_gain = store.get(own["dkv_norm"]) if self.own_cache else None
        if self.q_gain is not None and self.kv_gain is not None and self.q_gain.dtype != self.kv_gain.dtype:
            self.q_gain, self.kv_gain = self.q_gain.float(), self.kv_gain.float()
        H = self.num_heads
        uk = store.get(own["uk"]).to(self.dtype)
        self.uk_t = uk.view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = store.get(own["uv"]).to(self.dtype).view(H, self.vdim, self.kv_rank).contiguous()
        self.sinks = store.get(own["sink"]).float() if self.has_sink else None
        self.position.load(store)

    def first_weight(self) -> Optional[torch.Tensor]:
        return self.down.weight

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.o.warm_next = weight

    # ---- what it keeps ------------------------------------------------------------------------------------
    def cache_need(self) -> Optional[PagedCacheNeed]:
        return PagedCacheNeed(1, self.row, self.window or None, planes=1)

    def workspace_bytes(self, tokens: int) -> int:
        width = 2 if self.dtype == torch.bfloat16 else 4
        H = self.num_heads
        values = (self.down.workspace_bytes(tokens) + (self.uq.workspace_bytes(tokens) if self.uq else 0) + self.o.workspace_bytes(tokens)
                  + tokens * (self.q_rank + H * self.kv_rank + 2 * self.v_size) * width + tokens * H * self.kv_rank * 4)
        return values

    # ---- compute ----------------------------------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        kv = ctx.paged_kv(run)
        T = x.shape[0]
        H, rk, dr, dn = self.num_heads, self.kv_rank, self.rot_dim, self.dim
        if kv.writes != self.own_cache:
            raise RuntimeError("latent_attention: a layer with its own down-projection writes its cache, one without reads another's")
        down = self.down.forward(x)                        # [T, q_rank or H (dim + rot_dim) | kv_rank + rot_dim | H vdim]
        freq = self.position.frequencies() if self.position.rotary_dim else None
        if self.q_rank:
            cq = torch.empty((T, self.q_rank), dtype=down.dtype, device=down.device)
            kernels.latent_prep(down, 0, self.q_rank, self.q_rank, rk, dr, self.q_gain, self.kv_gain, self.eps, ctx.positions,
                                freq, self.position.rotary_dim, kv.group.slot_mapping if kv.writes else None,
                                kv.cache if kv.writes else None, cq, rot_gain=self.rot_gain)
            q = self.uq.forward(cq)                                          # [T, H (dim + rot_dim)]
        else:
            if self.own_cache:
                kernels.latent_prep(down, 0, 0, self.q_cols, rk, dr, None, self.kv_gain, self.eps, ctx.positions, freq,
                                    self.position.rotary_dim, kv.group.slot_mapping, kv.cache, None, rot_gain=self.rot_gain)
            q = down[:, :self.q_size]
        # the tensor-core kernel takes the absorbed queries in bfloat16; the all-sizes kernel keeps them in 32 bits
        fast = attention_dispatch.latent_tensor_cores(q.dtype, rk, dr, dn)
        q_abs = torch.empty((T, H * rk), dtype=torch.bfloat16 if fast else torch.float32, device=q.device)
        per_head_products(q.view(T, H, dn + dr)[:, :, :dn].transpose(0, 1), self.uk_t, q_abs.view(T, H, rk).transpose(0, 1))
        latent = torch.empty((T, H * rk), dtype=q.dtype, device=q.device)
        attention_dispatch.latent_attention(q_abs, q, latent, kv, ctx, freq, self.position.rotary_dim, self.sinks,
                                            H, dn, rk, dr, self.scale, self.window, rot_gain=self.rot_gain)
        heads = torch.empty((T, self.v_size), dtype=q.dtype, device=q.device)
        per_head_products(latent.view(T, H, rk).transpose(0, 1), self.uv, heads.view(T, H, self.vdim).transpose(0, 1))
        if self.has_gate:
            gated = torch.empty_like(heads)
            kernels.sigmoid_gate(heads, down[:, self.q_cols + (self.row if self.own_cache else 0):], gated)
            heads = gated
        return self.o.forward(heads)
