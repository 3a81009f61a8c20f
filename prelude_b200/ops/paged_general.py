"""General paged attention over a step's batch: keys and values of different sizes, values that are part of the
cached key rows, a window, a sink.  Picks the kernel for the type and shape; which one ran changes the rounding,
never what is computed."""
from __future__ import annotations

from typing import Optional

import torch

from . import kernels as K


def attention_general(q: torch.Tensor, k_pages: torch.Tensor, v_pages: Optional[torch.Tensor], value_dim: int, batch, group: int,
                      scale: float, window: Optional[int], sink: Optional[torch.Tensor], out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, kd] of the batch's tokens against the pages of cache group ``group``; ``v_pages`` None: the values are
    the first ``value_dim`` elements of the key rows.  Padding rows of a captured step are skipped by the kernel."""
    return K.attention_paged(q, k_pages, v_pages, value_dim, batch.positions, batch.table_row_of_token, batch.block_tables[group],
                             scale, window, sink, status=batch.status, out=out)
