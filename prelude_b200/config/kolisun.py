"""Typed configuration of Kolisun, read from its own config.json keys.

A Kolisun folder names itself with ``"architecture": "Kolisun"`` and gives
``vocab``, ``width``, ``norm.eps`` and a list ``layers``; every entry has a
``type`` (which mixer), the mixer's sizes and constants under ``mixer`` and its
feed-forward under ``mlp`` (``null``: none).  Layers are parsed one by one:
nothing is assumed about their number, order or sizes.

Two mixers exist.  ``parallel`` runs a windowed grouped-query attention
(``left``) and a selective state-space mixer (``right``) side by side and adds
their outputs, each times its scale.  ``latent_attention`` attends through a
low-rank latent per token with a learned sink per head.

What the design fixes, and what this file therefore writes down: a layer norms
each sublayer's output and nothing else; the attention of ``parallel`` has
biases on q, k and v, a norm over the whole q and k projections, rotation of
adjacent pairs with band-scaled rates; the latent attention rotates half-split
pairs with ramp-scaled rates whose amplitude grows by 0.1 ln(factor); the
feed-forward is SiLU-gated; the head is not tied; and the tensor names
(``embed``, ``head``, ``final.norm``, ``l<i>.norm1`` / ``norm2``, ``l<i>.mix.*``,
``l<i>.mlp.*``).
"""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import _Reader
from .registry import ConfigError, extract_eos_token_ids, register_architecture
from .spec import (BlockSpec, GatedMlpSpec, GqaSpec, LatentAttentionSpec, LayerCall, LinearHeadSpec, ModelSpec, NormSpec,
                   ParallelMixerSpec, RotaryBandScaling, RotaryRampScaling, RotaryRatesSpec, StateSpaceSpec)

RAMP_AMPLITUDE_SLOPE = 0.1
MAX_POSITIONS = 1 << 20          # the design names no longest sequence; this bounds positions, not the arithmetic


def _rotary(m: _Reader, adjacent: bool, span: int, problems: list) -> RotaryRatesSpec:
    rot = m.obj("rot")
    dims, base = rot.positive_int("dims"), rot.number("base", positive=True)
    if dims % 2 or dims > span:
        problems.append(f"{rot.where}: `dims`={dims} must be even and at most the {span} elements it turns")
    scaling = None
    if rot.raw.get("scaling") is not None:
        sc = rot.obj("scaling")
        if adjacent:
            scaling = RotaryBandScaling(factor=sc.number("factor", positive=True), low=sc.number("low", positive=True),
                                        high=sc.number("high", positive=True), original=sc.number("original", positive=True))
            if scaling.high == scaling.low:
                problems.append(f"{sc.where}: `high` and `low` must differ")
        else:
            scaling = RotaryRampScaling(factor=sc.number("factor", positive=True), original=sc.number("original", positive=True),
                                        fast=sc.number("fast", positive=True), slow=sc.number("slow", positive=True),
                                        amplitude_slope=RAMP_AMPLITUDE_SLOPE)
    return RotaryRatesSpec(dims=dims, base=base, adjacent=adjacent, scaling=scaling)


def _window_attention(m: _Reader, width: int, eps: float, problems: list) -> GqaSpec:
    heads, kv_heads, dim = m.positive_int("heads"), m.positive_int("kv_heads"), m.positive_int("dim")
    if heads % kv_heads:
        problems.append(f"{m.where}: heads={heads} is not a multiple of kv_heads={kv_heads}")
    window = m.obj("mask").positive_int("size") if m.raw.get("mask") is not None else None
    return GqaSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=dim, value_dim=m.positive_int("vdim"),
                   softmax_scale=m.number("scale", positive=True), position=_rotary(m, True, dim, problems), qkv_bias=True,
                   whole_qk_norm_eps=eps, window=window)


def _state_space(m: _Reader, width: int, eps: float, problems: list) -> StateSpaceSpec:
    heads, groups, parts = m.positive_int("heads"), m.positive_int("groups"), m.positive_int("norm_groups")
    vdim = m.positive_int("vdim")
    if heads % groups:
        problems.append(f"{m.where}: heads={heads} is not a multiple of groups={groups}")
    if (heads * vdim) % parts:
        problems.append(f"{m.where}: {heads * vdim} inner channels do not form {parts} equal parts")
    return StateSpaceSpec(hidden_size=width, num_heads=heads, head_dim=vdim, state=m.positive_int("state"), groups=groups,
                          conv_taps=m.positive_int("conv"), norm_groups=parts, norm_eps=eps)


def _latent_attention(m: _Reader, width: int, eps: float, problems: list) -> LatentAttentionSpec:
    rot_dim = m.positive_int("rot_dim")
    position = _rotary(m, False, rot_dim, problems)     # turns the first rot.dims elements of the rotated part
    return LatentAttentionSpec(hidden_size=width, num_heads=m.positive_int("heads"), head_dim=m.positive_int("dim"), rot_dim=rot_dim,
                               value_dim=m.positive_int("vdim"), kv_rank=m.positive_int("kv_rank"), q_rank=m.positive_int("q_rank"),
                               softmax_scale=m.number("scale", positive=True), norm_eps=eps, position=position, sink=True)


@register_architecture("Kolisun", aliases=("Kolisun", "KolisunModel"), model_types=("kolisun",))
@dataclass(frozen=True)
class KolisunConfig:
    vocab: int
    width: int
    norm_eps: float
    blocks: Tuple[BlockSpec, ...]
    eos_token_ids: Tuple[int, ...] = ()
    raw: Optional[dict] = None

    @classmethod
    def from_dict(cls, raw: dict) -> "KolisunConfig":
        problems: list = []
        top = _Reader(raw, "config", problems)
        vocab, width = top.positive_int("vocab"), top.positive_int("width")
        eps = top.obj("norm").number("eps", positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("config: `layers` must be a non-empty list")
            layers = []
        norm = NormSpec(dim=width, eps=eps, suffix="")
        blocks = []
        for i, layer in enumerate(layers):
            rd = _Reader(layer, f"layers[{i}]", problems)
            kind = rd.raw.get("type")
            m = rd.obj("mixer")
            if kind == "parallel":
                mixer = ParallelMixerSpec(
                    mixers=(_window_attention(m.obj("left"), width, eps, problems), _state_space(m.obj("right"), width, eps, problems)),
                    scales=(m.number("left_scale"), m.number("right_scale")), names=("left", "right"))
            elif kind == "latent_attention":
                mixer = _latent_attention(m, width, eps, problems)
            else:
                problems.append(f"layers[{i}]: unknown layer type {kind!r}; known: ['latent_attention', 'parallel']")
                continue
            ff = None
            mlp = rd.raw.get("mlp")
            if mlp is not None:
                f = _Reader(mlp, f"layers[{i}].mlp", problems)
                if f.raw.get("kind") != "dense":
                    problems.append(f"layers[{i}].mlp: unknown kind {f.raw.get('kind')!r}; known: ['dense']")
                else:
                    ff = GatedMlpSpec(hidden_size=width, intermediate_size=f.positive_int("ff"), activation="silu",
                                      gate_name="gate", up_name="up", down_name="down")
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=None, ff_norm=None, prefix=f"l{i}", mixer_name="mix",
                                    ff_name="mlp", kind="postnorm_residual", mixer_post_norm=norm,
                                    ff_post_norm=norm if ff is not None else None, mixer_post_norm_name="norm1",
                                    ff_post_norm_name="norm2"))
        try:
            eos = extract_eos_token_ids(raw)
        except ConfigError as e:
            problems.append(str(e))
            eos = ()
        if problems:
            raise ConfigError("failed to parse Kolisun config: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, blocks=tuple(blocks), eos_token_ids=eos, raw=copy.deepcopy(raw))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(dim=self.width, eps=self.norm_eps, suffix="")
        return ModelSpec(architecture="Kolisun", vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
                         blocks=self.blocks, order=tuple(LayerCall(block=i) for i in range(len(self.blocks))), final_norm=norm,
                         tie_embeddings=False, embed_name="embed", final_norm_name="final.norm", head_name="head",
                         eos_token_ids=self.eos_token_ids,
                         head=LinearHeadSpec(self.vocab, self.width, tied=False, name="head"))
