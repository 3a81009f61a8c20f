"""A selective state-space mixer with scalar decay per head (``StateSpaceSpec``).

One input projection [z | x | B | C | dt]; a causal convolution with SiLU over x, B and C; the recurrence token by
token with the state in float32; the gate, the norm in equal parts, the output projection.  Per sequence it keeps
the state [heads, state, head_dim] (float32) and the convolution's last ``conv_taps`` - 1 inputs, both in the
sequence's state slot.  Everything that depends on how a step's tokens are spread over sequences is read by the
kernels from the step's device arrays, so the mixer can be recorded.
"""
from __future__ import annotations

from typing import Dict

import torch

from ..config.spec import StateSpaceSpec
from ..ops import kernels as K
from ..ops.linear import linear
from ..weights.loader import TensorReq
from .registry import CombinedNeed, RunContext, StateNeed, register_part


@register_part("mixer", "state_space")
class StateSpace:
    def __init__(self, spec: StateSpaceSpec, prefix: str):
        if spec.num_heads % spec.groups:
            raise ValueError(f"{spec.num_heads} heads do not divide over {spec.groups} groups")
        self.spec, self.prefix = spec, prefix
        self.inner = spec.num_heads * spec.head_dim
        if self.inner % spec.norm_groups:
            raise ValueError(f"{self.inner} inner channels do not form {spec.norm_groups} equal parts")
        self.channels = self.inner + 2 * spec.groups * spec.state          # what the convolution covers: x, B, C
        self.proj_cols = self.inner + self.channels + spec.num_heads
        self.w_in = self.w_o = self.conv_w = self.conv_b = self.dt_bias = self.a_log = self.d_skip = self.norm_w = None

    def tensors(self) -> Dict[str, TensorReq]:
        s, p = self.spec, self.prefix
        return {
            f"{p}.{s.in_name}": TensorReq((self.proj_cols, s.hidden_size)),
            f"{p}.{s.conv_name}": TensorReq((self.channels, s.conv_taps), "conv"),
            f"{p}.{s.conv_bias_name}": TensorReq((self.channels,), "bias"),
            f"{p}.{s.dt_bias_name}": TensorReq((s.num_heads,), "bias"),
            f"{p}.{s.a_log_name}": TensorReq((s.num_heads,), "log_rate"),
            f"{p}.{s.d_name}": TensorReq((s.num_heads,), "norm"),
            f"{p}.{s.norm_name}": TensorReq((self.inner,), "norm"),
            f"{p}.{s.o_name}": TensorReq((s.hidden_size, self.inner)),
        }

    def load(self, get, ctx: RunContext) -> None:
        s, p = self.spec, self.prefix

        def mat(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=ctx.dtype).contiguous()

        def vec(name):
            return get(f"{p}.{name}").to(device=ctx.device, dtype=torch.float32).contiguous()

        self.w_in, self.w_o = mat(s.in_name), mat(s.o_name)
        self.conv_w, self.conv_b = vec(s.conv_name), vec(s.conv_bias_name)
        self.dt_bias, self.a_log, self.d_skip, self.norm_w = vec(s.dt_bias_name), vec(s.a_log_name), vec(s.d_name), vec(s.norm_name)

    def activation_bytes_per_token(self, elem: int) -> int:
        return (self.proj_cols + self.channels + self.inner) * elem + self.inner * 4 + self.spec.hidden_size * elem

    def cache_need(self) -> CombinedNeed:
        s = self.spec
        return CombinedNeed((StateNeed((s.num_heads, s.state, s.head_dim), torch.float32),
                             StateNeed((s.conv_taps - 1, self.channels), None)))

    def forward(self, x: torch.Tensor, batch, cache, write_cache: bool = True) -> torch.Tensor:
        s = self.spec
        T = batch.n_tokens
        state, carried = cache.children[0].state, cache.children[1].state
        proj = linear(x, self.w_in)
        z, xbc, dt = proj[:, :self.inner], proj[:, self.inner:self.inner + self.channels], proj[:, self.inner + self.channels:]
        u = K.causal_conv_silu(xbc, self.conv_w, self.conv_b, carried, batch,
                               out=batch.workspace("ssm_conv", (T, self.channels), x.dtype))
        K.conv_state_update(xbc, carried, batch)
        y = K.ssm_scan(u, dt, self.dt_bias, self.a_log, self.d_skip, state, batch, s.groups,
                       out=batch.workspace("ssm_y", (T, self.inner), torch.float32))
        g = K.gated_group_rmsnorm(y, z, self.norm_w, s.norm_groups, s.norm_eps,
                                  out=batch.workspace("ssm_gated", (T, self.inner), x.dtype))
        return linear(g, self.w_o)
