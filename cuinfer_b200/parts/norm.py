"""RMSNorm: ``out = x · rsqrt(mean(x²) + eps) · w`` with the squares, the mean, the rsqrt and the product
in 32 bits and one rounding at the end (csrc/ops/rms_norm.cu:43-71; eps inside the square root, the
weight multiplies directly).  Spec: ``PartSpec("rmsnorm", eps=..., weight_suffix=".weight", one_plus=False)``: the gain is
the tensor ``prefix + weight_suffix``, or, with ``one_plus``, one plus that tensor (a weight stored around zero; the sum
is taken once at load, in 32 bits, and the gain stays 32-bit).

The RMS norm also serves on a sub-layer's OUTPUT (a delta that is normed before it joins the residual): as
``stream.pending_norm`` it is folded by the next RMS norm of the stream in the same kernel, or alone by ``fold``.
"""
from __future__ import annotations

from typing import List

import torch

from .. import kernels
from .base import Norm, ResidualStream
from .registry import NORMS
from .spec import PartSpec, TensorSpec


@NORMS.register("rmsnorm")
class RMSNorm(Norm):
    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.eps = float(spec.eps)
        self.one_plus = bool(spec.get("one_plus", False))
        self.weight: torch.Tensor | None = None

    def tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + self.spec.get("weight_suffix", ".weight"), (self.hidden_size,),
                           keep_stored_precision=True, init="zeros" if self.one_plus else "ones")]

    def load(self, store) -> None:
        self.weight = store.get(self.tensors()[0])
        if self.one_plus:
            self.weight = (1.0 + self.weight.float()).contiguous()

    def fusable_rms(self):
        return (self.weight, self.eps) if self.weight is not None else None

    def add_norm(self, stream: ResidualStream) -> torch.Tensor:
        out = torch.empty(stream.residual.shape, dtype=self.dtype, device=stream.residual.device)
        post = stream.pending_norm
        if isinstance(post, RMSNorm) and stream.extra is None and stream.pending is not None:
            # the delta goes through its own RMS norm, joins the residual and the sum is normed: one kernel
            kernels.rms_stream(stream.residual, stream.pending, (post.weight, post.eps), (self.weight, self.eps), out)
            stream.pending = stream.pending_norm = None
            return out
        stream.settle()
        kernels.add_rmsnorm(stream.residual, stream.pending, self.weight, self.eps, out)
        stream.pending = None
        return out

    def fold(self, stream: ResidualStream) -> None:
        kernels.rms_stream(stream.residual, stream.pending, (self.weight, self.eps), None, None)
        stream.pending = stream.pending_norm = None

    def norm_rows(self, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.shape, dtype=self.dtype, device=rows.device)
        kernels.add_rmsnorm(rows, None, self.weight, self.eps, out)
        return out


@NORMS.register("layernorm")
class LayerNorm(Norm):
    """``(x - mean) / sqrt(var + eps) * gain + bias`` over the row, ``var`` the mean of the squared deviations, all in
    32 bits with one rounding at the end.  Spec: ``PartSpec("layernorm", eps=..., weight_suffix=".weight",
    bias_suffix=".bias")``: the tensors are ``prefix + suffix``.

    It serves on both sides of a sub-layer.  As the norm of a sub-layer's input (``add_norm``) it folds whatever the
    stream has outstanding — a delta that still has to go through ANOTHER layer norm (``stream.pending_norm``), extra
    rows — into the residual in the same kernel.  As the norm of a sub-layer's output it is that ``pending_norm``;
    ``fold`` applies it alone."""

    def __init__(self, spec: PartSpec, *, hidden_size: int, prefix: str, dtype: torch.dtype) -> None:
        super().__init__(spec, hidden_size=hidden_size, prefix=prefix, dtype=dtype)
        self.eps = float(spec.eps)
        self.weight: torch.Tensor | None = None
        self.bias: torch.Tensor | None = None

    def tensors(self) -> List[TensorSpec]:
        return [TensorSpec(self.prefix + self.spec.get("weight_suffix", ".weight"), (self.hidden_size,),
                           keep_stored_precision=True, init="ones"),
                TensorSpec(self.prefix + self.spec.get("bias_suffix", ".bias"), (self.hidden_size,),
                           keep_stored_precision=True, init="zeros")]

    def load(self, store) -> None:
        w, b = self.tensors()
        self.weight, self.bias = store.get(w), store.get(b)
        if self.weight.dtype != self.bias.dtype:
            self.weight, self.bias = self.weight.float(), self.bias.float()

    def _triple(self):
        return (self.weight, self.bias, self.eps)

    def _post_of(self, stream: ResidualStream):
        post = stream.pending_norm
        if post is None:
            return None
        if not isinstance(post, LayerNorm) or post.weight.dtype != self.weight.dtype:
            stream.settle()                       # another kind of norm on the delta: it folds itself
            return None
        return post._triple()

    def add_norm(self, stream: ResidualStream) -> torch.Tensor:
        post = self._post_of(stream)
        out = torch.empty(stream.residual.shape, dtype=self.dtype, device=stream.residual.device)
        kernels.sandwich_layernorm(stream.residual, stream.pending, post, stream.extra, self._triple(), out)
        stream.pending = stream.pending_norm = stream.extra = None
        return out

    def fold(self, stream: ResidualStream) -> None:
        kernels.sandwich_layernorm(stream.residual, stream.pending, self._triple(), stream.extra, None, None)
        stream.pending = stream.pending_norm = stream.extra = None

    def norm_rows(self, rows: torch.Tensor) -> torch.Tensor:
        out = torch.empty(rows.shape, dtype=self.dtype, device=rows.device)
        kernels.sandwich_layernorm(rows, None, None, None, self._triple(), out)
        return out
