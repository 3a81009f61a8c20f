"""Attention through one cached latent per token (``LatentAttentionSpec``).

Per token the cache holds the normed latent c (``kv_rank``) and one rotated key part (``rot_dim``) shared by all
heads: one key/value head of ``kv_rank + rot_dim`` elements and no value pages.  A head's plain key is W_uk,h c, so
its score q_plain . (W_uk,h c) equals (W_uk,h^T q_plain) . c: the queries are carried into the latent's space
(one batched product per step) and attention runs against the cached rows as they are, all heads sharing them;
the values are the rows' first ``kv_rank`` elements, and W_uv,h is applied to the attention's output (a second
batched product).  Nothing per head is ever made for a cached token.

Steps: down projections of queries and of latent + key part; norm of the query latent; up projection of the
queries; one kernel norms the latent, rotates the key part and the queries' rotated part and writes the page;
queries into latent space; attention with the sink; values out of latent space; output projection.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import LatentAttentionSpec
from ..ops import kernels as K
from ..ops.linear import batched_linear, linear
from ..ops.paged_general import attention_general
from ..weights.loader import TensorReq
from .registry import KvPagesNeed, RunContext, make_part, register_part


@register_part("mixer", "latent_attention")
class LatentAttention:
    def __init__(self, spec: LatentAttentionSpec, prefix: str):
        self.spec, self.prefix = spec, prefix
        self.position = make_part("position", spec.position, prefix)
        if getattr(self.position, "rates_host", None) is None:
            raise ValueError("this mixer takes a position encoding given by rates (kind 'rotary_rates')")
        if self.position.rotary_dim > spec.rot_dim:
            raise ValueError(f"a rotation of {self.position.rotary_dim} elements does not fit the rotated part of {spec.rot_dim}")
        self.q_dim = spec.head_dim + spec.rot_dim
        self.row = spec.kv_rank + spec.rot_dim                  # what a token keeps in the cache
        self.w_dq = self.w_uq = self.w_dkv = self.w_uk_t = self.w_uv = self.w_o = None
        self.dq_norm = self.dkv_norm = self.sink = None

    def parts(self):
        return (self.position,)

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        req = {
            f"{p}.{s.dq_name}": TensorReq((s.q_rank, s.hidden_size)),
            f"{p}.{s.dq_name}{s.norm_suffix}": TensorReq((s.q_rank,), "norm"),
            f"{p}.{s.uq_name}": TensorReq((s.num_heads * self.q_dim, s.q_rank)),
            f"{p}.{s.dkv_name}": TensorReq((self.row, s.hidden_size)),
            f"{p}.{s.dkv_name}{s.norm_suffix}": TensorReq((s.kv_rank,), "norm"),
            f"{p}.{s.uk_name}": TensorReq((s.num_heads * s.head_dim, s.kv_rank)),
            f"{p}.{s.uv_name}": TensorReq((s.num_heads * s.value_dim, s.kv_rank)),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, s.num_heads * s.value_dim)),
        }
        if s.sink:
            req[f"{p}.{s.sink_name}"] = TensorReq((s.num_heads,), "bias")
        return req

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype).contiguous()

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        self.w_dq, self.w_uq, self.w_dkv, self.w_o = mat(s.dq_name), mat(s.uq_name), mat(s.dkv_name), mat(s.o_name)
        # head h's rows of W_uk, transposed: [heads, kv_rank, head_dim], the weight of "queries into latent space"
        self.w_uk_t = mat(s.uk_name).view(s.num_heads, s.head_dim, s.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = mat(s.uv_name).view(s.num_heads, s.value_dim, s.kv_rank)
        self.dq_norm, self.dkv_norm = vec(s.dq_name + s.norm_suffix), vec(s.dkv_name + s.norm_suffix)
        if s.sink:
            self.sink = vec(s.sink_name)
        self.position.load(get, ctx)

    def activation_bytes_per_token(self, elem: int) -> int:
        s = self.spec
        return (s.q_rank * 2 + s.num_heads * (2 * self.q_dim + 2 * self.row + s.value_dim) + self.row) * elem + s.hidden_size * elem

    def cache_need(self) -> KvPagesNeed:
        return KvPagesNeed(1, self.row, self.spec.window, v_heads=0, v_head_dim=0)

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s, pos = self.spec, self.position
        T, H = batch.n_tokens, s.num_heads
        cq = K.rmsnorm(linear(x, self.w_dq), self.dq_norm, s.norm_eps)
        q = linear(cq, self.w_uq)                                         # [T, H * (head_dim + rot_dim)]
        ckv = linear(x, self.w_dkv) if write_cache else None            # [T, kv_rank + rot_dim]
        q_plain = batch.workspace("latent_q_plain", (T, H, s.head_dim), x.dtype)
        q_lat = batch.workspace("latent_q", (T, H, self.row), x.dtype)
        K.qkv_prepare(q, ckv, None, n_heads=H, q_dim=self.q_dim, k_weight=self.dkv_norm, k_norm_cols=s.kv_rank, eps=s.norm_eps,
                      rates=pos.rates, rot_dims=pos.rotary_dim, adjacent=pos.adjacent, amplitude=pos.amplitude,
                      q_rot_off=s.head_dim, k_rot_off=s.kv_rank, positions=batch.positions, table_row=batch.table_row_of_token,
                      block_table=batch.block_tables[cache.group], q_out=q_plain, q_split=s.head_dim, q_out2=q_lat, q2_off=s.kv_rank,
                      k_pages=cache.k_pages if write_cache else None, status=batch.status)
        # queries into latent space, head by head: q_lat[:, h, :kv_rank] = q_plain[:, h] W_uk,h
        batched_linear(q_plain.transpose(0, 1), self.w_uk_t, q_lat.transpose(0, 1)[:, :, :s.kv_rank])
        o_lat = attention_general(q_lat, cache.k_pages, None, s.kv_rank, batch, cache.group, s.softmax_scale, s.window, self.sink,
                                  out=batch.workspace("latent_o", (T, H, s.kv_rank), x.dtype))
        # values out of latent space: o[:, h] = o_lat[:, h] W_uv,h^T
        o = batch.workspace("latent_values", (T, H, s.value_dim), x.dtype)
        batched_linear(o_lat.transpose(0, 1), self.w_uv, o.transpose(0, 1))
        return linear(o.view(T, H * s.value_dim), self.w_o)
