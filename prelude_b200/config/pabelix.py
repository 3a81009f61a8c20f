"""Typed configuration of Pabelix, read from its own config.json keys.

A Pabelix folder names itself with ``"architecture": "Pabelix"`` and gives
``vocab``, ``width``, ``norm.eps`` and a list ``layers``; every entry has a
``type`` (which mixer), the mixer's sizes and constants under ``mixer`` and its
feed-forward under ``mlp`` (``null``: none).  Nothing is assumed about how many
layers there are, in which order their kinds come, or which sizes they have:
every layer is parsed on its own.

What the design fixes, and what this file therefore writes down: the base of
the sinusoidal position vector (10000), the slope of the dense feed-forward's
sigmoid (1.702), that a group's score is the sum of its two largest scores,
that the scale of every norm is stored around zero (applied as 1 + w), and the
tensor names (``embed``, ``final.norm``, ``l<i>.norm1`` / ``norm1b`` / ``norm2`` /
``norm2b``, ``l<i>.mix.*``, ``l<i>.mlp.*``).

A layer with ``kv_from: j`` in its mixer has no key and value projections: it
reads the pages that layer j wrote, which maps onto a run-order entry that
owns no cache (``LayerCall(block=i, cache=j, writes_cache=False)``).
"""
from __future__ import annotations

import copy
import math
from dataclasses import dataclass
from typing import Optional, Tuple

from .reader import _Reader, _is_int, _is_num  # noqa: F401
from .registry import ConfigError, extract_eos_token_ids, register_architecture
from .spec import (BlockSpec, ClampedGluSpec, DiffAttentionSpec, LayerCall, ModelSpec, NormSpec, QueryTemperatureSpec,
                   RoutedExpertsSpec, SinusoidEmbeddingSpec)

POSITION_BASE = 10000.0
DENSE_SIGMOID_SLOPE = 1.702
GROUP_SCORE_TOP = 2
MAX_POSITIONS = 1 << 20          # the design names no longest sequence; this bounds tables, not the arithmetic


@register_architecture("Pabelix", aliases=("Pabelix", "PabelixModel"), model_types=("pabelix",))
@dataclass(frozen=True)
class PabelixConfig:
    vocab: int
    width: int
    norm_eps: float
    blocks: Tuple[BlockSpec, ...]
    order: Tuple[LayerCall, ...]
    eos_token_ids: Tuple[int, ...] = ()
    raw: Optional[dict] = None

    # -- parsing --------------------------------------------------------------------
    @classmethod
    def from_dict(cls, raw: dict) -> "PabelixConfig":
        problems: list = []
        top = _Reader(raw, "config", problems)
        vocab, width = top.positive_int("vocab"), top.positive_int("width")
        eps = top.obj("norm").number("eps", positive=True)
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            problems.append("config: `layers` must be a non-empty list")
            layers = []
        norm = NormSpec(dim=width, eps=eps, offset=1.0, suffix="")
        blocks, order = [], []
        for i, layer in enumerate(layers):
            rd = _Reader(layer, f"layers[{i}]", problems)
            kind = rd.raw.get("type")
            if kind != "attention":
                problems.append(f"layers[{i}]: unknown layer type {kind!r}; known: ['attention']")
                continue
            m = rd.obj("mixer")
            heads, kv_heads = m.positive_int("heads"), m.positive_int("kv_heads")
            if heads % kv_heads:
                problems.append(f"layers[{i}].mixer: heads={heads} is not a multiple of kv_heads={kv_heads}")
            temp = None
            if m.raw.get("q_temp") is not None:
                qt = m.obj("q_temp")
                temp = QueryTemperatureSpec(coef=qt.number("coef"), every=qt.positive_int("every"))
            diff = m.number("diff")
            mixer = DiffAttentionSpec(hidden_size=width, num_heads=heads, num_kv_heads=kv_heads, head_dim=m.positive_int("dim"),
                                      value_dim=m.positive_int("vdim"), softmax_scale=m.number("scale", positive=True),
                                      lambda_init=diff, norm_eps=eps, query_temperature=temp)
            src = m.raw.get("kv_from")
            if src is not None:
                if not _is_int(src) or not 0 <= src < i:
                    problems.append(f"layers[{i}].mixer: `kv_from` must name an earlier layer, got {src!r}")
                    src = None
                elif not (src < len(order) and order[src].writes_cache):
                    problems.append(f"layers[{i}].mixer: `kv_from`={src} names a layer without keys and values of its own")
                    src = None
                else:
                    theirs = blocks[src].mixer
                    if (theirs.num_kv_heads, theirs.head_dim, theirs.value_dim) != (kv_heads, mixer.head_dim, mixer.value_dim):
                        problems.append(f"layers[{i}].mixer: its key/value sizes differ from those of layer {src}, whose cache it reads")
                        src = None
            ff, ff_norm = None, None
            mlp = rd.raw.get("mlp")
            if mlp is not None:
                f = _Reader(mlp, f"layers[{i}].mlp", problems)
                fk = f.raw.get("kind")
                if fk == "dense":
                    ff = ClampedGluSpec(hidden_size=width, intermediate_size=f.positive_int("ff"),
                                        limit=f.number("limit", positive=True), alpha=DENSE_SIGMOID_SLOPE)
                elif fk == "moe":
                    r = f.obj("router")
                    n_exp, top_k = r.positive_int("experts"), r.positive_int("top")
                    groups, keep = 1, 1
                    if r.raw.get("groups") is not None:
                        g = r.obj("groups")
                        groups, keep = g.positive_int("count"), g.positive_int("keep")
                    if n_exp % groups:
                        problems.append(f"layers[{i}].mlp.router: {n_exp} experts do not form {groups} equal groups")
                    elif keep > groups or top_k > keep * (n_exp // groups):
                        problems.append(f"layers[{i}].mlp.router: top={top_k} experts cannot come from {keep} of {groups} groups "
                                        f"of {n_exp // groups}")
                    ff = RoutedExpertsSpec(hidden_size=width, expert_size=f.obj("expert").positive_int("ff"), n_experts=n_exp,
                                           top_k=top_k, n_groups=groups, keep_groups=keep, group_score_top=GROUP_SCORE_TOP)
                else:
                    problems.append(f"layers[{i}].mlp: unknown kind {fk!r}; known: ['dense', 'moe']")
                ff_norm = norm
            blocks.append(BlockSpec(mixer=mixer, feed_forward=ff, mixer_norm=norm, ff_norm=ff_norm, prefix=f"l{i}",
                                    mixer_name="mix", ff_name="mlp", mixer_norm_name="norm1", ff_norm_name="norm2",
                                    kind="sandwich_residual", mixer_post_norm=norm, ff_post_norm=ff_norm,
                                    mixer_post_norm_name="norm1b", ff_post_norm_name="norm2b"))
            order.append(LayerCall(block=i) if src is None else LayerCall(block=i, cache=src, writes_cache=False))
        try:
            eos = extract_eos_token_ids(raw)
        except ConfigError as e:
            problems.append(str(e))
            eos = ()
        if problems:
            raise ConfigError("failed to parse Pabelix config: " + "; ".join(problems))
        return cls(vocab=vocab, width=width, norm_eps=eps, blocks=tuple(blocks), order=tuple(order), eos_token_ids=eos,
                   raw=copy.deepcopy(raw))

    def to_dict(self) -> dict:
        return copy.deepcopy(self.raw)

    # -- what the model builder reads ---------------------------------------------------
    def to_model_spec(self) -> ModelSpec:
        norm = NormSpec(dim=self.width, eps=self.norm_eps, offset=1.0, suffix="")
        return ModelSpec(architecture="Pabelix", vocab_size=self.vocab, hidden_size=self.width, max_positions=MAX_POSITIONS,
                         blocks=self.blocks, order=self.order, final_norm=norm, tie_embeddings=True, embed_name="embed",
                         final_norm_name="final.norm", eos_token_ids=self.eos_token_ids,
                         embedding=SinusoidEmbeddingSpec(self.vocab, self.width, name="embed", base=POSITION_BASE))
