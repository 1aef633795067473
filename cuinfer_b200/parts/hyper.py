"""Hyper-connections: a residual of several streams per token that sub-layers read from and write to with learned
coefficients.

Instead of one residual row a token keeps S rows ``x_0 .. x_{S-1}``, all equal to the embedding output at the start
(``ModelSpec.residual_streams = S``).  A sub-layer with the coefficients ``in`` [S], ``out`` [S] and ``mix`` [S, S]
(indexed [from, to]) reads ``u = sum_s in[s] x_s``, computes ``y = sublayer(norm(u))`` and writes all streams at once from
the old ones: ``x_t <- sum_s mix[s, t] x_s + out[t] y``.  The model's output is the sum of the streams.  Streams,
coefficients and sums are 32-bit.

:class:`HyperConnection` is one sub-layer's set of coefficients.  ``read`` hands out the normed input rows; the write of
the sub-layer BEFORE it, if one is still outstanding on the stream, happens in the same kernel (one pass over the S rows
of every token does write, read and RMS norm).  ``write`` only leaves the sub-layer's output on the stream, together
with the connection that knows its coefficients.

Block kind ``hyper_prenorm``: ``PartSpec("hyper_prenorm", streams=S, norm_names=(first, second),
connection_names=(first, second), coefficient_names=("in", "out", "mix"))``; a layer whose feed-forward is of kind ``none``
has the first sub-layer only.
"""
from __future__ import annotations

from typing import Callable, List, Optional

import torch

from .. import kernels
from .base import Block, FeedForward, Mixer, Norm, Part, ResidualStream
from .context import StepContext
from .registry import BLOCKS
from .spec import PartSpec, TensorSpec


class HyperConnection(Part):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.streams = int(spec.streams)
        if not 1 <= self.streams <= 16:
            raise ValueError(f"hyper-connections: {self.streams} streams are beyond what the kernel takes (1 to 16)")
        self.names = tuple(spec.get("coefficient_names", ("in", "out", "mix")))
        self.read_w: Optional[torch.Tensor] = None
        self.out_w: Optional[torch.Tensor] = None
        self.mix_w: Optional[torch.Tensor] = None

    def tensors(self) -> List[TensorSpec]:
        S = self.streams
        rd, out, mix = self.names
        # the random-weights mode draws coefficients near a plain residual sum: every stream read a little, the output
        # added to every stream, every stream kept
        return [TensorSpec(f"{self.prefix}.{rd}", (S,), keep_stored_precision=True, init="ones"),
                TensorSpec(f"{self.prefix}.{out}", (S,), keep_stored_precision=True, init="ones"),
                TensorSpec(f"{self.prefix}.{mix}", (S, S), keep_stored_precision=True, init="identity")]

    def load(self, store) -> None:
        rd, out, mix = self.tensors()
        self.read_w = store.get(rd).float().contiguous()
        self.out_w = store.get(out).float().contiguous()
        self.mix_w = store.get(mix).float().contiguous()

    def coefficients(self) -> tuple:
        return (self.mix_w, self.out_w)

    def read(self, stream: ResidualStream, norm: Norm) -> torch.Tensor:
        """The sub-layer's normed input rows [T, W]; the outstanding write of the sub-layer before happens on the way."""
        rms = norm.fusable_rms()
        if rms is None:
            raise ValueError("hyper-connections need a norm that is a plain RMS norm with a gain")
        if stream.residual.dim() != 3 or stream.residual.shape[1] != self.streams:
            raise ValueError(f"hyper-connections: the residual is {list(stream.residual.shape)}, not [T, {self.streams}, W]")
        if stream.pending_norm is not None or stream.extra is not None:
            stream.settle()
        T, _, W = stream.residual.shape
        out = torch.empty((T, W), dtype=self.dtype, device=stream.residual.device)
        before = stream.writer
        kernels.hyper_stream(stream.residual, stream.pending if before is not None else None,
                             before.coefficients() if before is not None else None, self.read_w, rms, out)
        stream.pending = stream.writer = None
        return out

    def write(self, stream: ResidualStream, y: torch.Tensor) -> None:
        stream.pending = y
        stream.writer = self

    def fold(self, stream: ResidualStream) -> None:
        """Do the outstanding write alone."""
        kernels.hyper_stream(stream.residual, stream.pending, self.coefficients(), None, None, None)
        stream.pending = stream.writer = None


@BLOCKS.register("hyper_prenorm")
class HyperPreNormBlock(Block):
    def __init__(self, spec: PartSpec, *, mixer: Mixer, feed_forward: FeedForward,
                 make_norm: Callable[[str], Norm], prefix: str) -> None:
        super().__init__(spec, mixer=mixer, feed_forward=feed_forward, make_norm=make_norm, prefix=prefix)
        first, second = spec.get("norm_names", ("norm1", "norm2"))
        c1, c2 = spec.get("connection_names", ("hc1", "hc2"))
        connection = PartSpec("hyper_connection", streams=int(spec.streams),
                              coefficient_names=spec.get("coefficient_names", ("in", "out", "mix")))

        def make_connection(name: str) -> HyperConnection:
            return HyperConnection(connection, hidden_size=mixer.hidden_size, prefix=f"{prefix}.{name}", dtype=mixer.dtype)

        self.mixer_norm = make_norm(f"{prefix}.{first}")
        self.mixer_connection = make_connection(c1)
        self.has_feed_forward = not getattr(feed_forward, "absent", False)
        self.feed_forward_norm = make_norm(f"{prefix}.{second}") if self.has_feed_forward else None
        self.feed_forward_connection = make_connection(c2) if self.has_feed_forward else None

    def parts(self) -> List[Part]:
        out: List[Part] = [self.mixer_norm, self.mixer_connection, self.mixer]
        if self.has_feed_forward:
            out += [self.feed_forward_norm, self.feed_forward_connection, self.feed_forward]
        return out

    def forward(self, stream: ResidualStream, ctx: StepContext, run: int) -> None:
        h = self.mixer_connection.read(stream, self.mixer_norm)
        self.mixer_connection.write(stream, self.mixer.forward(h, ctx, run))
        if self.has_feed_forward:
            h = self.feed_forward_connection.read(stream, self.feed_forward_norm)
            self.feed_forward_connection.write(stream, self.feed_forward.forward(h, ctx))
