"""Plain, slow, whole-sequence implementation of the Pabelix decoder.

The oracle of the Pabelix tests.  It shares no code with the ``prelude_b200``
package: it takes the parsed config.json and a ``dict`` of tensors keyed by
their safetensors names, runs a whole sequence at once with no cache, and
returns the logits of every position (and, on request, the residual stream
after every layer).  One function per mechanism.

The design, in this file's notation (D = width, t = position from 0):

  embedding   r_t = E[id_t] + s(t),  s(t)[2i] = sin(t w_i), s(t)[2i+1] = cos(t w_i), w_i = 10000^(-2i/D)
  norm        n(x; g) = x / sqrt(mean(x^2) + eps) * (1 + g)
  layer       r <- r + n(mixer(n(r; g1)); g1b) ;  r <- r + n(ff(n(r; g2)); g2b)
  attention   two score maps per head over shared values, see ``diff_attention``
  ff dense    W_d [ a * sigmoid(1.702 a) * (b + 1) ],  a = min(W_g x, L), b = clamp(W_u x, -L, L)
  ff routed   sum over chosen experts e of sigmoid(z_e) * W_d,e [ silu(W_g,e x) * W_u,e x ], see ``route``
  output      logits = E n(r; g_final)

All arithmetic is done in ``dtype`` (float64 by default); bfloat16 weights
convert exactly.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def sinusoid(n_positions: int, width: int, dtype=torch.float64, start: int = 0) -> torch.Tensor:
    """s[t, 2i] = sin(t * 10000^(-2i/width)), s[t, 2i+1] = cos of the same angle."""
    i = torch.arange(0, width, 2, dtype=torch.float64)
    rate = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -i / width)
    ang = torch.arange(start, start + n_positions, dtype=torch.float64).reshape(-1, 1) * rate.reshape(1, -1)
    out = torch.empty(n_positions, width, dtype=torch.float64)
    out[:, 0::2] = ang.sin()
    out[:, 1::2] = ang.cos()[:, : out[:, 1::2].shape[1]]
    return out.to(dtype)


def unit_offset_norm(x: torch.Tensor, g: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * (1 + g); without g, no scale at all."""
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if g is None else y * (1.0 + g)


def query_temperature(n_positions: int, coef: float, every: int, dtype, start: int = 0) -> torch.Tensor:
    """tau(t) = 1 + coef * ln(floor((t + 1) / every) + 1)."""
    t = torch.arange(start, start + n_positions, dtype=torch.int64)
    return (1.0 + coef * torch.log(((t + 1) // every + 1).to(torch.float64))).to(dtype)


def diff_attention(x: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float,
                   kv: Optional[tuple] = None):
    """The mixer.  x [T, D] is its (normed) input; w holds q, k, v, lq1, lk1, lq2, lk2, g, o.
    With ``kv`` = (k, v) of another layer the layer projects no keys and values.  Returns (y, (k, v)).

    Per query head h (key/value head h // (H / G)), maps c = 1, 2:
        S_c[t, j] = tau(t) * scale * <q_c[t], k_c[j]>   for j <= t,  A_c = softmax_j(S_c) V
        lam = exp(<lq1, lk1>) - exp(<lq2, lk2>) + diff
        o = A_1 - lam * A_2 ;  o <- o / sqrt(mean(o^2) + eps) * (1 - diff)
    then y = W_o [ concat_h(o) * sigmoid(W_g x) ].
    """
    T = x.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (x @ w["q"].T).reshape(T, H, 2, d)
    if kv is None:
        k = (x @ w["k"].T).reshape(T, G, 2, d)
        v = (x @ w["v"].T).reshape(T, G, dv)
    else:
        k, v = kv
    tau = query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], x.dtype)
    q = q * tau.reshape(T, 1, 1, 1)
    lam = torch.exp((w["lq1"] * w["lk1"]).sum()) - torch.exp((w["lq2"] * w["lk2"]).sum()) + m["diff"]
    visible = torch.ones(T, T, dtype=torch.bool).tril()
    heads = []
    for h in range(H):
        g = h // (H // G)
        maps = []
        for c in range(2):
            s = (q[:, h, c] @ k[:, g, c].T) * m["scale"]
            s = s.masked_fill(~visible, float("-inf"))
            maps.append(torch.softmax(s, dim=-1) @ v[:, g])
        o = maps[0] - lam * maps[1]
        heads.append(unit_offset_norm(o, None, eps) * (1.0 - m["diff"]))
    o = torch.cat(heads, dim=-1) * torch.sigmoid(x @ w["g"].T)
    return o @ w["o"].T, (k, v)


def clamped_glu(x: torch.Tensor, w: Dict[str, torch.Tensor], limit: float) -> torch.Tensor:
    """W_d [ a sigmoid(1.702 a) (b + 1) ], a = min(W_g x, limit), b = clamp(W_u x, -limit, limit)."""
    a = (x @ w["gate"].T).clamp(max=limit)
    b = (x @ w["up"].T).clamp(min=-limit, max=limit)
    return (a * torch.sigmoid(1.702 * a) * (b + 1.0)) @ w["down"].T


def route(z: torch.Tensor, top: int, groups: int, keep: int):
    """Router logits z [T, E] -> (chosen experts [T, top], their weights [T, top]).
    Scores sigmoid(z); experts in ``groups`` equal runs of neighbours; a group's score is the sum
    of its two largest scores; only experts of the ``keep`` best groups may be chosen; the weights
    are the chosen scores themselves."""
    T, E = z.shape
    s = torch.sigmoid(z)
    per = E // groups
    gs = s.reshape(T, groups, per)
    gscore = gs.topk(min(2, per), dim=-1).values.sum(dim=-1)
    best = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(T, groups, dtype=torch.bool)
    allowed.scatter_(1, best, True)
    masked = torch.where(allowed.repeat_interleave(per, dim=1), s, torch.full_like(s, -1.0))
    idx = masked.topk(top, dim=-1).indices
    return idx, s.gather(1, idx)


def routed_experts(x: torch.Tensor, w: Dict[str, torch.Tensor], r: dict) -> torch.Tensor:
    """Weighted sum of the chosen experts' silu-gated feed-forwards; w holds router and e<k>.gate/up/down."""
    groups = r.get("groups") or {"count": 1, "keep": 1}          # no groups named: all experts are one group
    idx, wt = route(x @ w["router"].T, r["top"], groups["count"], groups["keep"])
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        for e, a in zip(idx[t].tolist(), wt[t]):
            g = x[t] @ w[f"e{e}.gate"].T
            u = x[t] @ w[f"e{e}.up"].T
            y[t] += a * ((g * torch.sigmoid(g) * u) @ w[f"e{e}.down"].T)
    return y


def _sub(weights: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in weights.items() if k.startswith(prefix)}


def forward(cfg: dict, weights: Dict[str, torch.Tensor], ids: List[int], dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of the whole sequence ``ids``.  ``layers_out``, a list, receives the residual
    stream after every layer."""
    eps = cfg["norm"]["eps"]
    E = weights["embed"].to(dtype)
    T = len(ids)
    r = E[torch.tensor(ids, dtype=torch.long)] + sinusoid(T, cfg["width"], dtype)
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        g = {n: weights[p + n].to(dtype) for n in ("norm1", "norm1b", "norm2", "norm2b") if p + n in weights}
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown type {layer['type']!r}")
        m = layer["mixer"]
        src = m.get("kv_from")
        y, kept[i] = diff_attention(unit_offset_norm(r, g["norm1"], eps), _sub(weights, p + "mix.", dtype), m, eps,
                                    None if src is None else kept[src])
        r = r + unit_offset_norm(y, g["norm1b"], eps)
        ff = layer.get("mlp")
        if ff is not None:
            x = unit_offset_norm(r, g["norm2"], eps)
            fw = _sub(weights, p + "mlp.", dtype)
            if ff["kind"] == "dense":
                y = clamped_glu(x, fw, ff["limit"])
            elif ff["kind"] == "moe":
                y = routed_experts(x, fw, ff["router"])
            else:
                raise ValueError(f"layer {i}: unknown feed-forward {ff['kind']!r}")
            r = r + unit_offset_norm(y, g["norm2b"], eps)
        if layers_out is not None:
            layers_out.append(r.clone())
    return unit_offset_norm(r, weights["final.norm"].to(dtype), eps) @ E.T
