"""Interfaces of the parts a layer is made of.

A part is built from its :class:`PartSpec` plus the sizes of its surroundings (hidden size, engine
dtype, checkpoint prefix).  It announces the tensors it expects (``tensors``), takes them from the
weight store (``load``), says what it keeps between steps (``cache_need`` / ``state_need``) and
computes (``forward``).  No part knows which model it sits in.

Interfaces
----------
Norm            ``add_norm(stream) -> normed [T, H]`` folds the pending delta into the 32-bit residual and
                norms it; ``norm_rows(x32) -> [S, H]`` norms given 32-bit rows.
PositionEncoding ``table() -> float32 [positions, rotary_dim/2, 2]`` or None, ``rotary_dim``.
Mixer           ``forward(x [T, H], ctx, run) -> [T, H]``; ``cache_need()``, ``state_need()``.
FeedForward     ``forward(x [T, H], ctx) -> [T, H]``.
Block           ``forward(stream, ctx, run)``: arranges norms, mixer and feed-forward around the residual.
"""
from __future__ import annotations

from typing import List, Optional

import torch

from .context import StepContext
from .spec import PagedCacheNeed, PartSpec, StateNeed, TensorSpec


class ResidualStream:
    """The 32-bit residual rows of a step and a delta that has not been added yet.

    Keeping the last sub-layer's output pending lets the next norm do the add, the store of the new
    residual and the normalisation in one pass.  Two more things may be outstanding: ``pending_norm``, a norm that the
    pending rows go through BEFORE they are added (a layer that norms a sub-layer's output), and ``extra``, 32-bit
    rows that are added as well (a model that feeds its embedding output in again).  A norm that can do all of it in
    its own pass does; anything else calls ``settle()`` first, after which only ``residual`` counts.

    A residual of several streams per token (``residual`` is [T, S, W]) is written to by learned coefficients instead of
    a sum: ``pending`` then waits together with ``writer``, the part that knows how it joins the streams; the next read
    of the streams does the write in its own pass, ``settle()`` does it alone.
    """

    __slots__ = ("residual", "pending", "pending_norm", "extra", "_spare", "writer")

    def __init__(self, residual: torch.Tensor, pending: Optional[torch.Tensor] = None) -> None:
        self.residual = residual
        self.pending = pending
        self.pending_norm: Optional["Norm"] = None
        self.extra: Optional[torch.Tensor] = None
        self._spare: Optional[torch.Tensor] = None
        self.writer = None

    @property
    def plain(self) -> bool:
        """True when what is outstanding is at most a plain delta (``pending``) to be added as it is."""
        return self.pending_norm is None and self.extra is None and self.writer is None and self.residual.dim() == 2

    def wanted_rows(self, indices: torch.Tensor) -> torch.Tensor:
        """32-bit rows [len(indices), W] of the stream at the tokens ``indices`` with everything outstanding folded in
        (for several streams per token: their sum).  The other tokens' rows are left as they are."""
        from .. import kernels
        rows = torch.empty((indices.numel(), self.residual.shape[-1]), dtype=torch.float32, device=indices.device)
        if self.residual.dim() == 3:
            write = self.writer.coefficients() if self.writer is not None else None
            kernels.hyper_gather(self.residual, self.pending if write else None, write, indices, rows)
            return rows
        self.settle()
        kernels.gather_rows(self.residual, self.pending, indices, rows)
        return rows

    def collapsed(self) -> torch.Tensor:
        """The stream of every token as one 32-bit row [T, W], everything outstanding folded in."""
        self.settle()
        if self.residual.dim() == 3:
            from .. import kernels
            T, S, W = self.residual.shape
            out = torch.empty((T, W), dtype=torch.float32, device=self.residual.device)
            ones = torch.ones(S, dtype=torch.float32, device=self.residual.device)
            kernels.hyper_stream(self.residual, None, None, ones, None, None, read_out=out)
            return out
        return self.residual + self.pending.float() if self.pending is not None else self.residual

    def settle(self) -> None:
        """Fold a normed delta and extra rows into the residual.  A plain pending delta stays pending: every norm and
        the gather of the wanted rows add it themselves."""
        if self.writer is not None:
            self.writer.fold(self)
        if self.pending_norm is not None:
            self.pending_norm.fold(self)
        if self.extra is not None:
            from .. import kernels
            kernels.sandwich_layernorm(self.residual, None, None, self.extra, None, None)
            self.extra = None

    def spare(self) -> torch.Tensor:
        """A second buffer of the residual's shape, for kernels that write the new residual beside the old."""
        if self._spare is None:
            self._spare = torch.empty_like(self.residual)
        return self._spare

    def swap(self) -> None:
        """The spare buffer now holds the residual (and no delta is pending any more)."""
        self.residual, self._spare = self._spare, self.residual
        self.pending = None


class LazyNorm:
    """A norm of the residual stream that has not been computed yet.

    A block hands this to a mixer or feed-forward that declares ``accepts_lazy_norm``; its first projection
    may then compute the norm inside its own kernel (and fold the pending delta into the residual there).
    ``materialize()`` gives the normed rows as a tensor, whatever happened before.
    """

    __slots__ = ("stream", "norm", "_rows")

    def __init__(self, stream: ResidualStream, norm: "Norm") -> None:
        self.stream = stream
        self.norm = norm
        self._rows: Optional[torch.Tensor] = None

    @property
    def shape(self):
        return self.stream.residual.shape

    def materialize(self) -> torch.Tensor:
        if self._rows is None:
            self._rows = self.norm.add_norm(self.stream)     # folds a pending delta if there still is one
        return self._rows


class Part:
    # Whether the part's ``forward`` may be recorded into a CUDA graph and replayed for other batches: it reads the
    # batch from the device arrays of the context only, launches the same kernels whatever the batch holds, and never
    # waits for the device.  A part that loops over ``ctx.seq_lens_host`` / ``ctx.state_slots_host``, sizes a launch from
    # values of the batch, or synchronises says False here; a model with such a part runs every step eagerly, with the
    # host arrays of the context filled in.  Under a capture those two host arrays are None, so that a part that reads
    # them without having said so fails at once instead of replaying another batch's values.
    capturable: bool = True

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        self.spec = spec
        self.hidden_size = hidden_size
        self.prefix = prefix
        self.dtype = dtype

    def workspace_bytes(self, tokens: int) -> int:
        """Device memory the part's ``forward`` allocates for intermediate results of a step of ``tokens`` rows (its
        output included).  The engine leaves this much free when it sizes the cache pool from the device's memory."""
        return 0

    def tensors(self) -> List[TensorSpec]:
        return []

    def load(self, store) -> None:  # store: cuinfer_b200.weights.WeightStore
        pass

    # A decode step is a chain of short kernels, each of which waits for its first weights to come from memory.  A
    # part may name the weight it reads first, and be told which weight the step reads right after it: its last
    # kernel can then ask for that weight to be fetched into the L2 while it runs.  Both are hints; the defaults do
    # nothing.  The model wires them after loading, along the order in which its layers run.
    def first_weight(self) -> Optional[torch.Tensor]:
        return None

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        pass


class Norm(Part):
    def add_norm(self, stream: ResidualStream) -> torch.Tensor:
        raise NotImplementedError

    def norm_rows(self, rows: torch.Tensor) -> torch.Tensor:
        raise NotImplementedError

    def fold(self, stream: ResidualStream) -> None:
        """``stream.residual += self(stream.pending)`` (and ``stream.extra``, if the norm can add it in the same pass);
        nothing is pending afterwards.  Only a norm that a block uses on a sub-layer's OUTPUT needs this."""
        raise NotImplementedError(f"{type(self).__name__} cannot norm a sub-layer's output")

    def fusable_rms(self) -> Optional[tuple]:
        """``(gain, eps)`` if this norm is exactly ``x * rsqrt(mean(x^2) + eps) * gain`` over the whole row, so that a
        projection may compute it in its own kernel; None (the default) keeps the norm a kernel of its own."""
        return None

    def workspace_bytes(self, tokens: int) -> int:
        return tokens * self.hidden_size * (2 if self.dtype == torch.bfloat16 else 4)


class PositionEncoding(Part):
    rotary_dim: int = 0

    def table(self) -> Optional[torch.Tensor]:
        return None


class Mixer(Part):
    def cache_need(self) -> Optional[PagedCacheNeed]:
        return None

    def state_need(self) -> Optional[StateNeed]:
        return None

    def forward(self, x: torch.Tensor, ctx: StepContext, run: int) -> torch.Tensor:
        raise NotImplementedError


class FeedForward(Part):
    def forward(self, x: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        raise NotImplementedError


class Block:
    """An arrangement of norms, a mixer and a feed-forward around the residual stream."""

    def __init__(self, spec: PartSpec, *, mixer: Mixer, feed_forward: FeedForward, make_norm, prefix: str) -> None:
        self.spec = spec
        self.mixer = mixer
        self.feed_forward = feed_forward
        self.prefix = prefix

    capturable: bool = True          # as Part.capturable, for what the arrangement itself does

    def parts(self) -> List[Part]:
        raise NotImplementedError

    def forward(self, stream: ResidualStream, ctx: StepContext, run: int) -> None:
        raise NotImplementedError

    def workspace_bytes(self, tokens: int) -> int:
        """Largest sum of intermediate results alive at one time in the block (see Part.workspace_bytes)."""
        return sum(part.workspace_bytes(tokens) for part in self.parts())

    # hints for the L2 (see Part): the weight the layer reads first, and the weight that follows the layer
    def first_weight(self) -> Optional[torch.Tensor]:
        return self.mixer.first_weight()

    def warm_after(self, weight: Optional[torch.Tensor]) -> None:
        self.mixer.warm_after(self.feed_forward.first_weight())
        self.feed_forward.warm_after(weight)
