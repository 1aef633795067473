"""Choice of the paged-attention kernel for a step (keys and values per head; attention over cached latents: see
``latent_attention`` at the end).

float32 always runs the all-sizes kernel.  bfloat16: a step of single decoded tokens runs the split-KV kernel (its
TMA path where the cache layout allows and a CTA streams at least ``kernels.DECODE_TMA_MIN_KEYS`` keys, else its
cp.async path); any
other step runs the tcgen05 kernel (head size 128, heads per kv head dividing 128) or the mma.sync kernel (head
size 64 or 128); other head sizes fall back to the all-sizes kernel.  ``CUINFER_B200_ATTENTION=mma`` keeps prompt
portions off the tcgen05 kernel (for comparisons).
"""
from __future__ import annotations

import os

import torch

from .. import kernels
from .context import PagedKV, StepContext


_FORCE_MMA = os.environ.get("CUINFER_B200_ATTENTION", "") == "mma"


def paged_attention(qkv: torch.Tensor, out: torch.Tensor, kv: PagedKV, ctx: StepContext, num_heads: int,
                    num_kv_heads: int, head_dim: int, scale: float, window: int, warm: torch.Tensor | None = None) -> None:
    """``warm``: what the step reads right after the attention (the output projection's weight); the decode kernel
    asks for it to be fetched into the L2 when its stream of keys ends."""
    if (qkv.dtype == torch.bfloat16 and ctx.decode_only
            and kernels.paged_attention_decode_supports(head_dim, num_heads, num_kv_heads)):
        longest = max(1, ctx.max_seq_len)
        tma = kernels.decode_tma_takes(kv.group.page_size, head_dim, window)
        splits = kernels.decode_splits(ctx.num_requests, num_kv_heads, longest, kernels.decode_slots(head_dim), tma=tma,
                                       head_dim=head_dim)
        tma = tma and kernels.decode_uses_tma(longest, splits)
        kernels.paged_attention_decode(qkv, out, kv.cache, kv.group.block_table, ctx.seq_lens, num_heads,
                                       num_kv_heads, head_dim, scale, window, splits, tma=tma, warm=warm)
        return
    if qkv.dtype == torch.bfloat16 and not _FORCE_MMA and kernels.attention_tcgen05_supports(
            head_dim, num_heads, num_kv_heads, kv.group.page_size) and out.stride(0) % 8 == 0 and qkv.stride(0) % 8 == 0:
        lens = ctx.query_lens_for_launch()
        kernels.attention_tcgen05(qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens, lens,
                                  num_heads, num_kv_heads, head_dim, scale, window)
        return
    if qkv.dtype == torch.bfloat16 and kernels.paged_attention_prefill_supports(head_dim, num_heads, num_kv_heads):
        lens = ctx.query_lens_for_launch()
        kernels.paged_attention_prefill(qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                        lens, num_heads, num_kv_heads, head_dim, scale, window)
        return
    kernels.paged_attention_generic(
        qkv, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens, ctx.token_request,
        num_heads, num_kv_heads, head_dim, scale, window)


_FORCE_GENERIC_LATENT = os.environ.get("CUINFER_B200_LATENT_ATTENTION", "") == "generic"


def latent_tensor_cores(dtype: torch.dtype, rk: int, dr: int, dn: int) -> bool:
    """Whether attention over cached latents runs on the tensor-core kernel (bfloat16, latent and rotary sizes in
    multiples of 16; with or without a window); else the all-sizes kernel, which is also the 32-bit path.  The query-side product
    then delivers bfloat16 operands instead of 32-bit ones.  ``CUINFER_B200_LATENT_ATTENTION=generic`` keeps everything
    on the all-sizes kernel (for comparisons)."""
    return (dtype == torch.bfloat16 and not _FORCE_GENERIC_LATENT
            and kernels.latent_attention_mma_supports(rk, dr, dn))


def latent_attention(q_abs: torch.Tensor, q: torch.Tensor, out: torch.Tensor, kv: PagedKV, ctx: StepContext, freq, rot_dims: int,
                     sinks, num_heads: int, dn: int, rk: int, dr: int, scale: float, window: int, rot_gain: float = 1.0) -> None:
    """Attention of the step's rows over cached latent rows; ``q_abs`` bfloat16 selects the tensor-core kernel."""
    if q_abs.dtype == torch.bfloat16 and latent_tensor_cores(q.dtype, rk, dr, dn) and q_abs.stride(0) % 8 == 0:
        kernels.latent_attention_mma(q_abs, q, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                     ctx.query_lens_for_launch(), freq, rot_dims, sinks, num_heads, dn, rk, dr, scale,
                                     max(1, ctx.max_seq_len), decode_only=ctx.decode_only, window=window, rot_gain=rot_gain)
        return
    kernels.latent_attention_generic(q_abs, q, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                     ctx.token_request, ctx.positions, freq, rot_dims, sinks, num_heads, dn, rk, dr, scale, window,
                                     rot_gain=rot_gain)


def window_decode_splits(ctx: StepContext, num_kv_heads: int, window: int, keep_first: int) -> int:
    """Over how many CTAs a decode step shares the key tiles of a (request, key head): one CTA walks them one after the
    other otherwise, and a step of few requests leaves most SMs idle.  At least two tiles a CTA, at most eight splits,
    and no more CTAs than the three a SM that are resident at once (a second round of CTAs costs more than it saves)."""
    if not ctx.decode_only:
        return 1
    keys = max(1, ctx.max_seq_len)
    if window:
        keys = min(keys, window + 63) + (64 if keep_first else 0)
    tiles = -(-keys // 64)
    ctas = max(1, ctx.num_requests * num_kv_heads)
    return max(1, min(8, tiles // 2, 444 // ctas))


_FORCE_GENERIC_WINDOW = os.environ.get("CUINFER_B200_WINDOW_ATTENTION", "") == "generic"
# From how many (request, key head) pairs on a step of single tokens runs on the tcgen05 kernel too — one CTA per pair
# walks the keys in tiles of 128 — instead of the kernel that shares a pair's key tiles out to several CTAs.  Measured
# a call at 2 084 / 8 192 keys of 8 key heads: 1 request 37 / 124 us against 31 / 82; 8 requests 38 / 125 against 53 /
# 163; 64 requests 151 / 494 against 438 / 1 669.
TCGEN05_DECODE_MIN_CTAS = 48


def window_attention(q: torch.Tensor, out: torch.Tensor, kv: PagedKV, ctx: StepContext, num_heads: int, num_kv_heads: int,
                     dim: int, vdim: int, scale: float, softcap: float, window: int, keep_first: int, *, chunked: bool = False,
                     slopes: torch.Tensor | None = None, sinks: torch.Tensor | None = None) -> None:
    """Attention over cached [key | value] rows with a capped score and a window that keeps the first tokens (or, with
    ``chunked``, a mask of chunks; ``slopes``: a distance bias per head; ``sinks``: a score per head in the softmax's
    denominator): bfloat16
    steps whose sizes the tensor-core kernel takes run there, decode steps too (the window's 64-key tiles shared out to
    several CTAs, see ``window_decode_splits``; the all-sizes kernel, a warp per token and head with one key per lane,
    measured 16 times slower at a window of 1 024 keys of 128 values); float32 and every other size run the all-sizes kernel.  ``CUINFER_B200_WINDOW_ATTENTION=generic``
    keeps everything on the all-sizes kernel (for comparisons).

    A layer whose scores are plain — no cap, no distance bias, no kept first tokens, no chunks — with keys and values of
    128 is, sink apart, the attention that the tcgen05 kernel computes: steps that are not all single tokens go there,
    the kernel reading the joined rows and adding the sink (5 to 7 times faster than the ``mma.sync`` kernel at 2 048
    tokens), and so do steps of single tokens with enough requests to fill the GPU without splitting keys (see
    ``TCGEN05_DECODE_MIN_CTAS``); ``CUINFER_B200_ATTENTION=mma`` keeps them on the ``mma.sync`` kernel."""
    if (q.dtype == torch.bfloat16 and not _FORCE_GENERIC_WINDOW and not _FORCE_MMA
            and (not ctx.decode_only or ctx.num_requests * num_kv_heads >= TCGEN05_DECODE_MIN_CTAS)
            and dim == vdim and not softcap and not keep_first and not chunked and slopes is None
            and kernels.attention_tcgen05_supports(dim, num_heads, num_kv_heads, kv.group.page_size)
            and q.stride(0) % 8 == 0 and out.stride(0) % 8 == 0 and (sinks is None or sinks.dtype == torch.float32)):
        kernels.attention_tcgen05(q, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                  ctx.query_lens_for_launch(), num_heads, num_kv_heads, dim, scale, window, joined=True, sinks=sinks)
        return
    if (q.dtype == torch.bfloat16 and not _FORCE_GENERIC_WINDOW and q.stride(0) % 8 == 0
            and kernels.window_attention_mma_supports(dim, vdim, num_heads, num_kv_heads)):
        kernels.window_attention_mma(q, out, kv.cache, kv.group.block_table, ctx.query_start_loc, ctx.seq_lens,
                                     ctx.query_lens_for_launch(), num_heads, num_kv_heads, dim, vdim, scale, softcap, window, keep_first,
                                     splits=window_decode_splits(ctx, num_kv_heads, window, keep_first), chunked=chunked,
                                     slopes=slopes, sinks=sinks)
        return
    kernels.window_attention_generic(q, out, kv.cache, kv.group.block_table, ctx.positions, ctx.token_request, num_heads,
                                     num_kv_heads, dim, vdim, scale, softcap, window, keep_first, chunked=chunked,
                                     slopes=slopes, sinks=sinks)
