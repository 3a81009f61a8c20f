"""Differential attention over a paged cache.

Every query head holds two score maps: two queries and two keys of ``head_dim``,
one softmax each, over the same values of ``value_dim``.  The head's output is

    o = A_1 - lambda * A_2,   o <- o / sqrt(mean(o^2) + eps) * (1 - lambda_init),
    lambda = exp(<lq1, lk1>) - exp(<lq2, lk2>) + lambda_init      (one number per layer)

then the concatenated heads are multiplied with sigmoid(W_g x) and projected with
W_o.  Positions enter through the query temperature only (``QueryTemperatureSpec``),
which scales the scores in 32-bit.

One merged projection [q | k | v | g] of the mixer's input; keys and values go
into the layer's pages, keys as 2 * kv_heads heads of head_dim (a key/value head's
two maps one after the other), values as kv_heads heads of value_dim; attention
reads queries and gate from the merged projection in place and does difference,
norm, scale and gate in its epilogue.  With ``write_cache=False`` the layer has
no key and value projections: it reads the pages an earlier layer wrote.

lambda is a constant of the loaded weights; it is taken once, in 64-bit, when
they are loaded.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from ..config.spec import DiffAttentionSpec
from ..ops.diff_attention import diff_attention
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import KvPagesNeed, RunContext, register_part


@register_part("mixer", "diff_attention")
class DiffAttention:
    def __init__(self, spec: DiffAttentionSpec, prefix: str):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not divide over {spec.num_kv_heads} key/value heads")
        if not (0 < spec.head_dim <= 256 and 0 < spec.value_dim <= 256):
            raise ValueError(f"differential attention: key size {spec.head_dim} and value size {spec.value_dim} must lie in 1..256")
        self.spec, self.prefix = spec, prefix
        self.q_cols = spec.num_heads * 2 * spec.head_dim
        self.k_cols = spec.num_kv_heads * 2 * spec.head_dim
        self.v_cols = spec.num_kv_heads * spec.value_dim
        self.o_cols = spec.num_heads * spec.value_dim
        self.owns_kv = True
        self.w_in = self.w_o = None
        self.lam = 0.0

    def share_cache(self) -> None:
        """This layer reads another layer's keys and values: it has no projections of its own for them."""
        self.owns_kv = False

    # -- weights ----------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {f"{p}.{s.q_name}": TensorReq((self.q_cols, s.hidden_size)),
               f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.o_cols))}
        if self.owns_kv:
            req[f"{p}.{s.k_name}"] = TensorReq((self.k_cols, s.hidden_size))
            req[f"{p}.{s.v_name}"] = TensorReq((self.v_cols, s.hidden_size))
        if s.gated:
            req[f"{p}.{s.gate_name}"] = TensorReq((self.o_cols, s.hidden_size))
        for n in s.lambda_names:
            req[f"{p}.{n}"] = TensorReq((s.head_dim,), "vector")
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        # q, then k and v where the layer has them, then the gate: one product
        rows = [mat(s.q_name)] + ([mat(s.k_name), mat(s.v_name)] if self.owns_kv else []) + ([mat(s.gate_name)] if s.gated else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = mat(s.o_name).contiguous()
        lq1, lk1, lq2, lk2 = (get(f"{p}.{n}").to(torch.float64) for n in s.lambda_names)
        self.lam = math.exp(float((lq1 * lk1).sum())) - math.exp(float((lq2 * lk2).sum())) + s.lambda_init

    def activation_bytes_per_token(self, elem: int) -> int:
        return (self.q_cols + self.k_cols + self.v_cols + 3 * self.o_cols) * elem + self.spec.hidden_size * elem

    # -- cache ------------------------------------------------------------------
    def cache_need(self) -> KvPagesNeed:
        s = self.spec
        return KvPagesNeed(2 * s.num_kv_heads, s.head_dim, s.window, v_heads=s.num_kv_heads, v_head_dim=s.value_dim)

    # -- one step -----------------------------------------------------------------
    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        if write_cache != self.owns_kv:
            raise ValueError(f"{self.prefix}: the layer {'has' if self.owns_kv else 'has no'} keys and values of its own, "
                             f"the run order says otherwise")
        proj = linear(x, self.w_in)
        q = proj[:, :self.q_cols]
        at = self.q_cols
        table = batch.block_tables[cache.group]
        if write_cache:
            K.kv_write_pages(proj[:, at:at + self.k_cols], proj[:, at + self.k_cols:at + self.k_cols + self.v_cols],
                             cache.k_pages, cache.v_pages, batch.positions, batch.table_row_of_token, table, batch.status)
            at += self.k_cols + self.v_cols
        gate = proj[:, at:at + self.o_cols] if s.gated else None
        o = diff_attention(q, gate, cache.k_pages, cache.v_pages, batch, cache.group, s, self.lam,
                           out=batch.workspace("diff_attention_out", (batch.n_tokens, s.num_heads, s.value_dim), x.dtype))
        return linear(o.view(batch.n_tokens, self.o_cols), self.w_o)
