"""Chooses the attention kernels for the rows of a step, and stores the step's keys and values.

Rows of one-token segments (decoding) come first, the rows of longer segments (portions of
prompts) after them, so each kind is one run of rows.  All kernels read the same pages and
keep the same contract: the query at position p sees the keys of its own request up to p
(inside the window, if the mixer has one; a mixer whose ``window`` is negative means blocks of that many
positions, counted from position 0: the query sees its own block's keys up to p).

* bfloat16, head size a multiple of 8, decoding rows: the split-KV decode kernel, which also
  stores the current token's key and value;
* bfloat16, head size 64 or 128, page size a power of two, longer segments: the TMA + tcgen05 kernel,
  after the cache-write kernel; other head sizes in steps of 16 up to 128 (and these two with
  CBIS_TCGEN05=0): the tiled mma.sync kernel;
* 32-bit, head size in steps of 16 up to 128, longer segments: the tiled 32-bit kernel (decoding rows: the general
  kernel);
* everything else: the general kernel, after the cache-write kernel.

A mixer may also name (attributes, all optional): ``v_head_dim`` (values of another width than the keys; with one
cached array for keys and values the values are the first entries of its rows), ``slopes`` (a distance bias per
head), ``sinks`` (a number per head in the softmax's denominator) and ``q_temp`` (a query temperature by position).
``run_attention`` returns how many columns a head's result takes in ``out``.
"""
from __future__ import annotations

import torch

from ..kernels import ops


def _key_chunks(ctx, mixer, nd, T, hd, row_tile=64, blocks_per_tile=1, blocks_per_sm=8, min_chunk=256):
    """Few rows behind a long context give the tiled kernels too few blocks: the keys are then cut into chunks over
    more blocks, whose partial results (in the step's scratch memory) a second kernel merges."""
    limit = ctx.ctx_limit
    chunks = ops.prefill_key_chunks(-(-ctx.max_seg_rows // row_tile), mixer.n_head, ctx.n_segments - nd, limit,
                                    blocks_per_tile, blocks_per_sm, min_chunk)
    partial = None
    if chunks[0] > 1:
        partial, _ = ctx.decode_scratch((T - nd) * mixer.n_head * chunks[0] * (hd + 4), 1)
    return chunks, partial


def _general_chunks(ctx, mixer, rows, hd):
    """The general kernel gives a warp to every (row, head): a few rows behind a long context are cut the same way."""
    limit = ctx.ctx_limit
    chunks = ops.generic_key_chunks(rows, mixer.n_head, limit, hd)
    partial = None
    if chunks[0] > 1:
        partial, _ = ctx.decode_scratch(rows * mixer.n_head * chunks[0] * (hd + 4), 1)
    return chunks, partial


def _extended(ctx, mixer, qkv, cache, view, out, k_pages, v_pages, k_off, v_off, vd, slopes, sinks, q_temp) -> int:
    """Attention with values of their own width, a distance bias, a sink or a query temperature.  bfloat16 with
    widths that are multiples of 8: the decoding rows go to the split-KV decode kernel's lane-group form (up to 256
    wide; it stores the current token's key and value itself), the longer segments, after the cache-write kernel, to
    the tiled tensor-core kernel (up to 128 wide, pages of a power of two).  32-bit, other sizes: the cache-write
    kernel and the general kernel."""
    T, nd, hd, ps = ctx.n_rows, ctx.n_decode, mixer.head_dim, cache.page_size
    extra = dict(v_head_dim=vd, slopes=slopes, sinks=sinks, q_temp=q_temp)
    o = out[:, :mixer.n_head * vd]
    by8 = (qkv.dtype == torch.bfloat16 and hd % 8 == 0 and vd % 8 == 0 and qkv.stride(0) % 8 == 0 and k_off % 8 == 0
           and v_off % 8 == 0 and qkv.data_ptr() % 16 == 0 and o.stride(0) % 8 == 0 and o.data_ptr() % 16 == 0)
    fast_decode = by8 and nd > 0 and max(hd, vd) <= 256
    tiled = by8 and T > nd and max(hd, vd) <= 128 and ps & (ps - 1) == 0 and ops.USE_TILED_EXTENDED
    first = nd if fast_decode else 0        # rows from here on have their keys and values stored by the cache-write kernel
    if fast_decode:
        nsplit = ops.decode_splits(nd, mixer.n_head, ctx.ctx_limit)
        scratch = counters = None
        if nsplit > 1:
            scratch, counters = ctx.decode_scratch(ops.decode_scratch_floats(nd, mixer.n_head, vd, nsplit), nd * mixer.n_head)
        ops.paged_decode_bf16(qkv[:nd], k_off if mixer.own_kv else -1, v_off if mixer.own_kv else -1, k_pages, v_pages,
                              view.block_table, ctx.row_seq, ctx.positions, view.slot_mapping, o[:nd], scratch, counters,
                              mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale, mixer.window, nsplit, **extra)
    if first >= T:
        return vd
    r = slice(first, T)
    if mixer.own_kv:
        ops.kv_write(qkv[r], k_off, v_off, k_pages, v_pages, view.slot_mapping[r], mixer.n_kv_head, hd, ps, v_head_dim=vd)
    if tiled:        # q and out keep their full row numbering, the kernel finds its rows through cu_rows
        chunks, partial = _key_chunks(ctx, mixer, first, T, vd)
        ops.paged_prefill_bf16(qkv, k_pages, v_pages, view.block_table, ctx.cu_rows, ctx.seg_start, o, first,
                               ctx.n_segments - first, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale,
                               mixer.window, chunks, partial, ctx.positions, first, T - first, **extra)
        return vd
    chunks, partial = _general_chunks(ctx, mixer, T - first, vd)
    ops.paged_attention_generic(qkv[r, :mixer.d_q], k_pages, v_pages, view.block_table, ctx.row_seq[r], ctx.positions[r],
                                o[r], mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale, mixer.window, chunks, partial,
                                **extra)
    return vd


def run_attention(ctx, mixer, qkv, cache, view, out) -> int:
    nd = ctx.n_decode
    T = ctx.n_rows
    hd, ps = mixer.head_dim, cache.page_size
    # the pages that stand for keys and for values: "k" and "v", or what the mixer names (a mixer whose keys and
    # values are both one cached array names it twice)
    k_name, v_name = getattr(mixer, "kv_arrays", ("k", "v"))
    k_pages, v_pages = cache.arrays[k_name], cache.arrays[v_name]
    k_off = mixer.d_q
    v_off = k_off if v_name == k_name else k_off + mixer.d_kv      # one array for both: one column block for both
    vd = int(getattr(mixer, "v_head_dim", 0) or hd)
    slopes, sinks, q_temp = (getattr(mixer, a, None) for a in ("slopes", "sinks", "q_temp"))
    if vd != hd or slopes is not None or sinks is not None or q_temp is not None:
        return _extended(ctx, mixer, qkv, cache, view, out, k_pages, v_pages, k_off, v_off, vd, slopes, sinks, q_temp)
    _plain(ctx, mixer, qkv, cache, view, out, nd, T, hd, ps, k_pages, v_pages, k_off, v_off)
    return hd


def _plain(ctx, mixer, qkv, cache, view, out, nd, T, hd, ps, k_pages, v_pages, k_off, v_off) -> None:
    fast_decode = qkv.dtype == torch.bfloat16 and hd % 8 == 0 and hd <= 256 and nd > 0
    first_general = nd if fast_decode else 0
    if fast_decode:
        limit = ctx.ctx_limit
        nsplit = ops.decode_splits(nd, mixer.n_head, limit)
        scratch = counters = None
        if nsplit > 1:
            scratch, counters = ctx.decode_scratch(ops.decode_scratch_floats(nd, mixer.n_head, hd, nsplit),
                                                   nd * mixer.n_head)
        ops.paged_decode_bf16(qkv[:nd], k_off if mixer.own_kv else -1, v_off if mixer.own_kv else -1, k_pages, v_pages,
                              view.block_table, ctx.row_seq, ctx.positions, view.slot_mapping, out[:nd], scratch, counters,
                              mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale, mixer.window, nsplit)
    if first_general < T:
        r = slice(first_general, T)
        if mixer.own_kv:
            ops.kv_write(qkv[r], k_off, v_off, k_pages, v_pages, view.slot_mapping[r], mixer.n_kv_head, hd, ps)
        tiled = qkv.dtype == torch.bfloat16 and ps & (ps - 1) == 0 and first_general == nd
        if tiled and hd in (64, 128) and 8 <= ps <= 128 and ops.USE_TCGEN05:
            # TMA + tcgen05: q and out keep their full row numbering, the kernel finds its rows through cu_rows
            chunks, partial = _key_chunks(ctx, mixer, nd, T, hd, row_tile=128, blocks_per_tile=2, blocks_per_sm=2, min_chunk=8192)
            ops.paged_prefill_tc5(qkv, k_pages, v_pages, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                  ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                  mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        if tiled and hd % 16 == 0 and 16 <= hd <= 128:
            chunks, partial = _key_chunks(ctx, mixer, nd, T, hd)
            ops.paged_prefill_bf16(qkv, k_pages, v_pages, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                   ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                   mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        if qkv.dtype == torch.float32 and hd % 16 == 0 and 16 <= hd <= 128 and ops.USE_TILED_F32:
            # 32-bit: decoding rows through the general kernel, the longer segments 64 rows to a block
            if nd > 0:
                d = slice(0, nd)
                chunks, partial = _general_chunks(ctx, mixer, nd, hd)
                ops.paged_attention_generic(qkv[d, :mixer.d_q], k_pages, v_pages, view.block_table, ctx.row_seq[d],
                                            ctx.positions[d], out[d], mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale,
                                            mixer.window, chunks, partial)
            if ctx.n_segments > nd:
                chunks, partial = _key_chunks(ctx, mixer, nd, T, hd)
                ops.paged_prefill_f32(qkv, k_pages, v_pages, view.block_table, ctx.cu_rows, ctx.seg_start, out, nd,
                                      ctx.n_segments - nd, ctx.max_seg_rows, mixer.n_head, mixer.n_kv_head, hd, ps,
                                      mixer.scale, mixer.window, chunks, partial, ctx.positions, nd, T - nd)
            return
        chunks, partial = _general_chunks(ctx, mixer, T - first_general, hd)
        ops.paged_attention_generic(qkv[r, :mixer.d_q], k_pages, v_pages, view.block_table, ctx.row_seq[r],
                                    ctx.positions[r], out[r], mixer.n_head, mixer.n_kv_head, hd, ps, mixer.scale,
                                    mixer.window, chunks, partial)
