"""Differential attention over a step's batch: picks the kernel for the type and shape.

float32 always runs the plain warp-per-row kernel.  bfloat16 runs the
tensor-core kernel where it takes the shape (key and value sizes in multiples
of 16 up to 256, at most 64 query heads per key/value head) and the plain
kernel otherwise.  Which one ran changes the rounding, never what is computed.

A step of single tokens (a decode step) gives every token a tile of its own
and cuts its keys into ranges, one block each, so that a few long requests
still fill the device; the ranges' sums are merged by a second kernel.  A step
with prompt portions runs the tiles of all its requests, the single tokens
among them, in one launch.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import kernels as K
from . import library as _l
from .attention import _prefill_plan, _sm_count
from .library import check

# PRELUDE_DIFF_ATTN=ref sends bfloat16 to the plain kernel as well
KERNEL = os.environ.get("PRELUDE_DIFF_ATTN", "auto")
# Whether the softmax weights (computed in float32) enter the second product as one bfloat16 number, as in the
# framework's other attention kernels, or as a rounded part plus what the rounding lost (PRELUDE_DIFF_ATTN_SPLIT=1:
# two bfloat16 numbers, 16 bits of the weight, twice the tensor-core work of that product).  Measured against
# 64-bit logits the two differ by less than a twentieth of the error that the bfloat16 queries, keys and values
# cause, so the single number is the default.
SPLIT_WEIGHTS = os.environ.get("PRELUDE_DIFF_ATTN_SPLIT", "0") == "1"


def decode_splits(n_tokens: int, n_kv_heads: int, max_context: int, device, most: int = 32) -> int:
    """Into how many ranges a decode step cuts a token's keys: enough blocks for two per multiprocessor, no range
    shorter than a tile of 64 keys, ``most`` at most (what the merge kernel takes)."""
    tiles = max(1, -(-int(max_context) // 64))
    want = max(1, (2 * _sm_count(device)) // max(1, n_tokens * n_kv_heads))
    return max(1, min(tiles, want, most))


def diff_attention(q: torch.Tensor, gate: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, batch,
                   group: int, spec, lam: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, heads * 2 * head_dim] and gate [T, heads * value_dim] (columns of the merged projection) of the batch's
    tokens against the pages of cache group ``group``; [T, heads, value_dim] goes to ``out`` when given.  While a
    step is being captured piece by piece, attention is what the pieces are cut at (its grid follows how the
    step's tokens are spread over requests), as for the other attention kernels."""
    T = q.shape[0]
    if out is None:
        out = torch.empty((T, spec.num_heads, spec.value_dim), dtype=q.dtype, device=q.device)
    recorder = batch.extras.get("recorder")
    if recorder is not None and recorder.capturing:
        recorder.run_between_pieces(lambda: diff_attention(q, gate, k_pages, v_pages, batch, group, spec, lam, out))
        return out
    table = batch.block_tables[group]
    temp = spec.query_temperature
    coef, every = (temp.coef, temp.every) if temp else (0.0, 1)
    lib = _l.library()
    if (q.dtype != torch.bfloat16 or KERNEL == "ref"
            or not lib.pb_diff_attention_tc_supported(spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim, q.stride(0))):
        n = batch.n_real                                   # the rows after them are padding of a captured step
        K.diff_attention_ref(q[:n], None if gate is None else gate[:n], k_pages, v_pages, batch.positions[:n],
                             batch.table_row_of_token[:n], table, spec.num_heads, spec.softmax_scale, coef, every, lam,
                             spec.norm_eps, 1.0 - spec.lambda_init, spec.window, batch.status, out=out[:n])
        return out
    num_pages, _, page_size, dim = k_pages.shape
    vdim = v_pages.shape[3]
    splits, scratch = 1, None
    if batch.decode_only:
        tile_seq = tile_tok0 = None
        n_tiles = T
        max_ctx = batch.max_kv_len if batch.max_kv_len else table.shape[1] * page_size
        if spec.window:
            max_ctx = min(max_ctx, spec.window + 64)
        splits = decode_splits(T, spec.num_kv_heads, max_ctx, q.device,
                               lib.pb_diff_attention_tc_max_splits(spec.num_heads, spec.num_kv_heads))
        floats = lib.pb_diff_attention_tc_scratch_floats(T, spec.num_heads, spec.num_kv_heads, vdim, splits)
        if floats:
            key = ("diff_attention_scratch", T, spec.num_heads, vdim, splits)
            scratch = batch.extras.get(key)
            if scratch is None:
                scratch = batch.extras[key] = torch.empty(floats, dtype=torch.float32, device=q.device)
    else:
        tile_seq, tile_tok0, n_tiles = _prefill_plan(batch, 64 // (spec.num_heads // spec.num_kv_heads), 0, None)
    check(lib.pb_diff_attention_tc_bf16(
        q.data_ptr(), q.stride(0), K._ptr(gate), gate.stride(0) if gate is not None else 0, k_pages.data_ptr(), v_pages.data_ptr(),
        out.data_ptr(), table.data_ptr(), table.shape[1], batch.positions.data_ptr(), batch.table_row_of_token.data_ptr(),
        batch.cu_q.data_ptr(), K._ptr(tile_seq), K._ptr(tile_tok0), n_tiles, page_size, num_pages, T, spec.num_heads,
        spec.num_kv_heads, dim, vdim, float(spec.softmax_scale), float(coef), int(every), float(lam), float(spec.norm_eps),
        float(1.0 - spec.lambda_init), int(spec.window) if spec.window else 0, 1 if K.kv_swizzled(q.dtype, dim) else 0,
        1 if K.kv_swizzled(q.dtype, vdim) else 0, splits, 1 if SPLIT_WEIGHTS else 0, K._ptr(scratch), batch.status.data_ptr(),
        _l.current_stream_ptr(q.device)), "diff_attention_tc")
    return out
