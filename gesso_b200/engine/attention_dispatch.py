"""Which attention kernel a step's queries run on.

float32 runs always take the FP32-arithmetic kernel.  bfloat16 runs take the tensor-core kernels
when the sizes fit them (head 32/64/96/128, pages in multiples of 16 slots): the split-KV kernel
for steps of single tokens; for steps with portions the tcgen05 flash kernel (head 64, 2 to 16 query
heads per kv head) or else the mma.sync flash kernel; other sizes take the FP32-arithmetic kernel
on bfloat16 data.  A distance bias per head and a sink in the softmax denominator are taken by the mma.sync
kernels and the FP32-arithmetic kernel; values that are the keys themselves and float32 queries by the
FP32-arithmetic kernel only.  Kept first keys under a window, an output gate and attention weights in two
bfloat16 pieces are taken by every kernel (the FP32-arithmetic kernel's weights are float32 anyway);
values of another width than the keys by the FP32-arithmetic kernel only.  Every
branch is one of this library's own kernels.
"""
from __future__ import annotations

import torch

from .. import ops


def paged_attention(rt, q, cache, ctx, window, scale, keep_first: int = 0, gate=None, split_weights: bool = False,
                    sink=None, slopes=None, values_are_keys: bool = False):
    N, nh, hd = q.shape
    nkv, page_size = cache.k_pages.shape[1], cache.k_pages.shape[2]
    vd = cache.v_pages.shape[2]
    if window is None:
        keep_first = 0                       # without a window every earlier key is visible anyway
    # A distance bias on the scores and a sink in the denominator: the mma.sync kernels take them (head 32/64/96/128,
    # values as wide as keys), the tcgen05 kernel does not.  Values that are the keys themselves (latent attention
    # without transposed pages) and float32 queries: the FP32-arithmetic kernel takes them all.
    special = sink is not None or slopes is not None
    if values_are_keys or q.dtype != cache.k_pages.dtype or (special and not (
            q.dtype == torch.bfloat16 and vd == hd and ops.fast_attention_takes(hd, page_size, nh, nkv))):
        return ops.paged_attention_generic(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                           ctx.seg_of_token, window, scale, keep_first, gate, sink=sink, slopes=slopes,
                                           values_are_keys=values_are_keys)
    split_weights = split_weights and ops.ATTN_SPLIT_WEIGHTS
    if q.dtype == torch.bfloat16 and vd == hd and ops.fast_attention_takes(hd, page_size, nh, nkv):
        if ctx.decode_only:
            splits = ops.decode_splits(ctx.n_segs, nkv, ctx.max_kv_len, uneven=True)
            ws = _decode_workspace(rt, q, ctx, nh, nkv, hd, splits) if splits > 1 else None
            return ops.decode_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                        window, scale, splits, ws, ctx.kv_span, keep_first, gate, split_weights,
                                        slopes=slopes, sink=sink)
        if not special and ops.attention_tcgen05_takes(hd, page_size, nh, nkv):
            # head 64 with 2..16 query heads per kv head: S and P in tensor memory, pages by TMA
            return ops.prefill_attention_tcgen05(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.seg_start,
                                                 ctx.seg_pos0, ctx.tile_seg, ctx.tile_q0, window, scale, keep_first, gate,
                                                 split_weights)
        return ops.prefill_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.seg_start,
                                     ctx.seg_pos0, ctx.tile_seg, ctx.tile_q0, window, scale, keep_first, gate,
                                     split_weights, slopes=slopes, sink=sink)
    return ops.paged_attention_generic(q, cache.k_pages, cache.v_pages, cache.block_table,
                                       ctx.positions, ctx.seg_of_token, window, scale, keep_first, gate)


def _decode_workspace(rt, q, ctx, nh, nkv, hd, splits):
    key = ("decode_attention_workspace", ctx.n_segs, nh, nkv, hd, splits)
    ws = rt.shared.get(key)
    if ws is None:
        dev = q.device
        ws = (torch.empty((ctx.n_segs * nh * splits * hd,), dtype=torch.float32, device=dev),
              torch.empty((ctx.n_segs * nh * splits * 2,), dtype=torch.float32, device=dev),
              torch.zeros((ctx.n_segs * nkv,), dtype=torch.int32, device=dev))
        rt.shared[key] = ws
    return ws


def sigmoid_attention(rt, q, cache, ctx, scale, dist_bias=None, temp_coef: float = 0.0, temp_every: int = 0, gate=None,
                      window=None):
    """Attention with sigmoid weights (no softmax) of the step's queries over the paged cache.  bfloat16 runs take
    the tensor-core kernels when the sizes fit them (head 32/64/96/128, values as wide as keys, pages in multiples
    of 16 slots): the split-KV kernel for steps of single tokens, the flash kernel for steps with portions, each
    weight in two bfloat16 pieces.  float32 runs and other sizes run the FP32-arithmetic kernel."""
    N, nh, hd = q.shape
    nkv, page_size = cache.k_pages.shape[1], cache.k_pages.shape[2]
    vd = cache.v_pages.shape[2]
    if (q.dtype == torch.bfloat16 and cache.k_pages.dtype == torch.bfloat16 and vd == hd
            and ops.fast_attention_takes(hd, page_size, nh, nkv)):
        if ctx.decode_only:
            splits = ops.decode_splits(ctx.n_segs, nkv, ctx.max_kv_len, uneven=True)
            ws = _decode_workspace(rt, q, ctx, nh, nkv, hd, splits) if splits > 1 else None
            return ops.sigmoid_decode_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions, scale,
                                                splits, ws, ctx.kv_span, dist_bias, temp_coef, temp_every, gate, window)
        return ops.sigmoid_prefill_attention(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.seg_start,
                                             ctx.seg_pos0, ctx.tile_seg, ctx.tile_q0, scale, dist_bias, temp_coef,
                                             temp_every, gate, window)
    return ops.sigmoid_attention_generic(q, cache.k_pages, cache.v_pages, cache.block_table, ctx.positions,
                                         ctx.seg_of_token, scale, dist_bias, temp_coef, temp_every, gate, window)
