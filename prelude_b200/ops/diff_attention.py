"""Differential attention over a step's batch: picks the kernel for the type and shape.

float32 always runs the plain warp-per-row kernel, and so does bfloat16 for
shapes the tensor-core kernels do not take.  Which one ran changes the
rounding, never what is computed.
"""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def diff_attention(q: torch.Tensor, gate: Optional[torch.Tensor], k_pages: torch.Tensor, v_pages: torch.Tensor, batch,
                   group: int, spec, lam: float, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, heads * 2 * head_dim] and gate [T, heads * value_dim] (columns of the merged projection) of the batch's
    tokens against the pages of cache group ``group``; [T, heads, value_dim] goes to ``out`` when given."""
    table = batch.block_tables[group]
    temp = spec.query_temperature
    return K.diff_attention_ref(q, gate, k_pages, v_pages, batch.positions, batch.table_row_of_token, table, spec.num_heads,
                                spec.softmax_scale, temp.coef if temp else 0.0, temp.every if temp else 1, lam, spec.norm_eps,
                                1.0 - spec.lambda_init, spec.window, batch.status, out=out)
