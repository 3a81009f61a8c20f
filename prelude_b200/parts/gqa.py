"""Grouped-query softmax attention with the options of ``GqaSpec``: keys and values of different sizes, biases on
q, k and v, an RMS norm over the whole q projection and the whole k projection (all heads at once), rotation by
rates, a window, a sink per head.

One merged q/k/v projection; one kernel norms, rotates, stores the queries and writes keys and values into the
layer's pages; then attention over the pages and the output projection.  Where keys and values have one size and
there is no sink, attention runs on the kernels of the plain attention mixer (tensor cores in bfloat16); otherwise
on the general paged kernel.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import GqaSpec
from ..ops import kernels as K
from ..ops.attention import paged_attention
from ..ops.linear import linear
from ..ops.paged_general import attention_general
from ..weights.loader import TensorReq
from .registry import KvPagesNeed, RunContext, make_part, register_part


@register_part("mixer", "gqa")
class Gqa:
    def __init__(self, spec: GqaSpec, prefix: str):
        if spec.num_heads % spec.num_kv_heads:
            raise ValueError(f"{spec.num_heads} query heads do not divide over {spec.num_kv_heads} key/value heads")
        self.spec, self.prefix = spec, prefix
        self.position = make_part("position", spec.position, prefix)
        if getattr(self.position, "rates_host", None) is None:
            raise ValueError("this mixer takes a position encoding given by rates (kind 'rotary_rates')")
        if self.position.rotary_dim > spec.head_dim:
            raise ValueError(f"a rotation of {self.position.rotary_dim} elements does not fit heads of {spec.head_dim}")
        self.q_cols = spec.num_heads * spec.head_dim
        self.k_cols = spec.num_kv_heads * spec.head_dim
        self.v_cols = spec.num_kv_heads * spec.value_dim
        self.o_cols = spec.num_heads * spec.value_dim
        self.w_qkv = self.b_qkv = self.w_o = self.q_norm = self.k_norm = self.sink = None
        # with keys and values of one size and no sink, the plain attention mixer's kernels take the pages
        self.plain_kernels = spec.head_dim == spec.value_dim and not spec.sink

    def parts(self):
        return (self.position,)

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {
            f"{p}.{s.q_name}": TensorReq((self.q_cols, s.hidden_size)),
            f"{p}.{s.k_name}": TensorReq((self.k_cols, s.hidden_size)),
            f"{p}.{s.v_name}": TensorReq((self.v_cols, s.hidden_size)),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.o_cols)),
        }
        if s.qkv_bias:
            for name, n in ((s.q_name, self.q_cols), (s.k_name, self.k_cols), (s.v_name, self.v_cols)):
                req[f"{p}.{name}{s.bias_suffix}"] = TensorReq((n,), "bias")
        if s.whole_qk_norm_eps is not None:
            req[f"{p}.{s.q_name}{s.norm_suffix}"] = TensorReq((self.q_cols,), "norm")
            req[f"{p}.{s.k_name}{s.norm_suffix}"] = TensorReq((self.k_cols,), "norm")
        if s.sink:
            req[f"{p}.{s.sink_name}"] = TensorReq((s.num_heads,), "bias")
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype)

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        self.w_qkv = torch.cat([mat(s.q_name), mat(s.k_name), mat(s.v_name)], dim=0).contiguous()
        self.w_o = mat(s.o_name).contiguous()
        if s.qkv_bias:
            self.b_qkv = torch.cat([vec(s.q_name + s.bias_suffix), vec(s.k_name + s.bias_suffix), vec(s.v_name + s.bias_suffix)]).contiguous()
        if s.whole_qk_norm_eps is not None:
            self.q_norm, self.k_norm = vec(s.q_name + s.norm_suffix), vec(s.k_name + s.norm_suffix)
        if s.sink:
            self.sink = vec(s.sink_name)
        self.position.load(get, ctx)

    def activation_bytes_per_token(self, elem: int) -> int:
        return (2 * self.q_cols + self.k_cols + self.v_cols + 2 * self.o_cols) * elem + self.spec.hidden_size * elem

    def cache_need(self) -> KvPagesNeed:
        s = self.spec
        if s.head_dim == s.value_dim:
            return KvPagesNeed(s.num_kv_heads, s.head_dim, s.window)
        return KvPagesNeed(s.num_kv_heads, s.head_dim, s.window, v_heads=s.num_kv_heads, v_head_dim=s.value_dim)

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s, pos = self.spec, self.position
        T = batch.n_tokens
        rows = self.q_cols + (self.k_cols + self.v_cols if write_cache else 0)
        qkv = linear(x, self.w_qkv[:rows], None if self.b_qkv is None else self.b_qkv[:rows])
        swz = self.plain_kernels and K.kv_swizzled(x.dtype, s.head_dim)
        q = K.qkv_prepare(
            qkv[:, :self.q_cols], qkv[:, self.q_cols:self.q_cols + self.k_cols] if write_cache else None,
            qkv[:, self.q_cols + self.k_cols:] if write_cache else None, n_heads=s.num_heads, q_dim=s.head_dim,
            q_weight=self.q_norm, k_weight=self.k_norm, k_norm_cols=self.k_cols, eps=s.whole_qk_norm_eps or 0.0, rates=pos.rates,
            rot_dims=pos.rotary_dim, adjacent=pos.adjacent, amplitude=pos.amplitude, positions=batch.positions,
            table_row=batch.table_row_of_token, block_table=batch.block_tables[cache.group],
            q_out=batch.workspace("gqa_q", (T, s.num_heads, s.head_dim), x.dtype),
            k_pages=cache.k_pages if write_cache else None, v_pages=cache.v_pages if write_cache else None,
            swizzle_k=swz, swizzle_v=swz, status=batch.status)
        out = batch.workspace("gqa_out", (T, s.num_heads, s.value_dim), x.dtype)
        if self.plain_kernels:
            o = paged_attention(q, cache.k_pages, cache.v_pages, batch, cache.group, s.softmax_scale, s.window, out=out)
        else:
            o = attention_general(q, cache.k_pages, cache.v_pages, s.value_dim, batch, cache.group, s.softmax_scale, s.window,
                                  self.sink, out=out)
        return linear(o.view(T, self.o_cols), self.w_o)
