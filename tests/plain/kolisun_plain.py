"""Plain, slow, whole-sequence implementation of the Kolisun decoder.

The oracle of the Kolisun tests.  It shares no code with the ``prelude_b200``
package: it takes the parsed config.json and a ``dict`` of tensors keyed by
their safetensors names, runs a whole sequence at once with no cache, and
returns the logits of every position (and, on request, the residual stream
after every layer).  One function per mechanism.

The design, in this file's notation (D = width, t = position from 0):

  norm        n(x; g) = x / sqrt(mean(x^2) + eps) * g
  layer       r <- r + n(mixer(r); g1) ;  r <- r + n(ff(r); g2)     (the sublayers read r itself)
  mixers      'parallel': a_l * window_attention(r) + a_r * mamba2(r);  'latent_attention': see there
  ff          W_d [ silu(W_g x) * W_u x ]
  output      logits = W_head n(r; g_final)

All arithmetic is done in ``dtype`` (float64 by default); bfloat16 weights
convert exactly.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Tuple

import torch


def rms_norm(x: torch.Tensor, g: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    y = x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)
    return y if g is None else y * g


def silu(x: torch.Tensor) -> torch.Tensor:
    return x * torch.sigmoid(x)


def softplus(x: torch.Tensor) -> torch.Tensor:
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


# -- rotation rates -------------------------------------------------------------------------------
def plain_rates(dims: int, base: float) -> List[float]:
    return [base ** (-2.0 * i / dims) for i in range(dims // 2)]


def banded_rates(dims: int, base: float, sc: Optional[dict]) -> List[float]:
    """Rates with long wavelengths slowed down by ``factor``, short ones kept, and a linear blend between."""
    out = []
    for f in plain_rates(dims, base):
        if sc is None:
            out.append(f)
            continue
        wave = 2.0 * math.pi / f
        if wave < sc["original"] / sc["high"]:
            out.append(f)
        elif wave > sc["original"] / sc["low"]:
            out.append(f / sc["factor"])
        else:
            s = (sc["original"] / wave - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * f / sc["factor"] + s * f)
    return out


def ramped_rates(dims: int, base: float, sc: Optional[dict]) -> Tuple[List[float], float]:
    """(rates, amplitude): rates blended between f and f / factor along a ramp over the pair index, and the
    factor that both cosine and sine are multiplied with."""
    f = plain_rates(dims, base)
    if sc is None:
        return f, 1.0

    def turn(t):
        return dims * math.log(sc["original"] / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(sc["fast"])), 0)
    hi = min(math.ceil(turn(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rates: List[float], amplitude: float, adjacent: bool) -> torch.Tensor:
    """x [T, heads, d]: the first 2 * len(rates) entries of every head are turned, the rest pass.  ``adjacent``:
    entry 2i goes with 2i + 1; otherwise entry i goes with i + len(rates)."""
    n = len(rates)
    ang = positions.to(x.dtype).reshape(-1, 1, 1) * torch.tensor(rates, dtype=x.dtype).reshape(1, 1, -1)
    c, s = ang.cos() * amplitude, ang.sin() * amplitude
    out = x.clone()
    if adjacent:
        u, v = x[..., 0:2 * n:2], x[..., 1:2 * n:2]
        out[..., 0:2 * n:2] = u * c - v * s
        out[..., 1:2 * n:2] = v * c + u * s
    else:
        u, v = x[..., :n], x[..., n:2 * n]
        out[..., :n] = u * c - v * s
        out[..., n:2 * n] = v * c + u * s
    return out


# -- attention ------------------------------------------------------------------------------------
def masked_softmax_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, scale: float, window: Optional[int],
                             sink: Optional[torch.Tensor] = None) -> torch.Tensor:
    """q [T, H, d], k [T, H, d], v [T, H, e] (keys already spread over the query heads).  Position i sees j with
    0 <= i - j (< window).  ``sink`` [H]: exp(sink_h) joins every denominator of head h and nothing else."""
    T = q.shape[0]
    s = torch.einsum("ihd,jhd->hij", q, k) * scale
    i = torch.arange(T).reshape(-1, 1)
    j = torch.arange(T).reshape(1, -1)
    seen = (j <= i) if window is None else ((j <= i) & (i - j < window))
    s = s.masked_fill(~seen, -math.inf)
    if sink is None:
        p = torch.softmax(s, dim=-1)
    else:
        m = torch.maximum(s.max(dim=-1, keepdim=True).values, sink.to(s.dtype).reshape(-1, 1, 1))
        e = torch.exp(s - m)
        p = e / (e.sum(dim=-1, keepdim=True) + torch.exp(sink.to(s.dtype).reshape(-1, 1, 1) - m))
    return torch.einsum("hij,jhe->ihe", p, v)


def window_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float, start: int = 0) -> torch.Tensor:
    """Grouped-query attention with biases, a norm over the whole of q and of k, adjacent-pair rotation with
    banded rates, and a window."""
    T = h.shape[0]
    H, G, d, e = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = h @ w["q"].T + w["q.b"]
    k = h @ w["k"].T + w["k.b"]
    v = h @ w["v"].T + w["v.b"]
    q = rms_norm(q, w["q.norm"], eps).reshape(T, H, d)
    k = rms_norm(k, w["k.norm"], eps).reshape(T, G, d)
    v = v.reshape(T, G, e)
    rot = m["rot"]
    rates = banded_rates(rot["dims"], rot["base"], rot.get("scaling"))
    pos = torch.arange(start, start + T)
    q, k = rotate(q, pos, rates, 1.0, True), rotate(k, pos, rates, 1.0, True)
    rep = H // G
    k, v = k.repeat_interleave(rep, dim=1), v.repeat_interleave(rep, dim=1)
    window = m["mask"]["size"] if m.get("mask") else None
    o = masked_softmax_attention(q, k, v, m["scale"], window)
    return o.reshape(T, H * e) @ w["o"].T


def latent_attention(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    """Queries, keys and values through low-rank latents; one rotated key part shared by all heads; a sink."""
    T = h.shape[0]
    H, d, r, e, L = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).reshape(T, H, d + r)
    ckv = h @ w["dkv"].T
    c = rms_norm(ckv[:, :L], w["dkv.norm"], eps)
    k_rot = ckv[:, L:].reshape(T, 1, r)
    rot = m["rot"]
    rates, amp = ramped_rates(rot["dims"], rot["base"], rot.get("scaling"))
    pos = torch.arange(T)
    q_rot = rotate(q[..., d:], pos, rates, amp, False)
    k_rot = rotate(k_rot, pos, rates, amp, False)
    k_flat = (c @ w["uk"].T).reshape(T, H, d)
    v = (c @ w["uv"].T).reshape(T, H, e)
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_flat, k_rot.expand(T, H, r)], dim=-1)
    o = masked_softmax_attention(qq, kk, v, m["scale"], None, w["sink"])
    return o.reshape(T, H * e) @ w["o"].T


# -- state-space mixer ----------------------------------------------------------------------------
def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K] (last column: the current token), zeros before the start."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat([torch.zeros(K - 1, C, dtype=u.dtype), u], dim=0)
    out = bias.reshape(1, C).expand(T, C).clone()
    for j in range(K):
        out = out + padded[j:j + T] * taps[:, j].reshape(1, C)
    return out


def state_space(x: torch.Tensor, B: torch.Tensor, C: torch.Tensor, dt: torch.Tensor, a_log: torch.Tensor,
                D: torch.Tensor) -> torch.Tensor:
    """x [T, H, P], B and C [T, H, N] (already spread over the heads), dt [T, H]:
    S_t = exp(-exp(a_log) dt_t) S_(t-1) + dt_t B_t x_t^T ;  y_t = S_t^T C_t + D x_t."""
    T, H, P = x.shape
    N = B.shape[-1]
    S = torch.zeros(H, N, P, dtype=x.dtype)
    y = torch.empty_like(x)
    for t in range(T):
        decay = torch.exp(-torch.exp(a_log) * dt[t])
        S = decay.reshape(H, 1, 1) * S + dt[t].reshape(H, 1, 1) * B[t].reshape(H, N, 1) * x[t].reshape(H, 1, P)
        y[t] = torch.einsum("hnp,hn->hp", S, C[t]) + D.reshape(H, 1) * x[t]
    return y


def mamba2(h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    proj = h @ w["in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    C = xbc[:, inner + G * N:].reshape(T, G, N).repeat_interleave(H // G, dim=1)
    dt = softplus(dt + w["dt_bias"])
    y = state_space(x, B, C, dt, w["A_log"], w["D"]).reshape(T, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * w["norm"]
    return y @ w["o"].T


# -- the model --------------------------------------------------------------------------------------
def sub(tensors: Dict[str, torch.Tensor], prefix: str, dtype) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: v.to(dtype) for k, v in tensors.items() if k.startswith(prefix)}


def mixer(kind: str, h: torch.Tensor, w: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    if kind == "parallel":
        left = window_attention(h, sub(w, "left.", h.dtype), m["left"], eps)
        right = mamba2(h, sub(w, "right.", h.dtype), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    if kind == "latent_attention":
        return latent_attention(h, w, m, eps)
    raise ValueError(f"unknown layer type {kind!r}")


def feed_forward(h: torch.Tensor, w: Dict[str, torch.Tensor]) -> torch.Tensor:
    return (silu(h @ w["gate"].T) * (h @ w["up"].T)) @ w["down"].T


def forward(cfg: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float64, layers_out: Optional[list] = None):
    """Logits [T, vocab] of a whole sequence; ``layers_out`` collects the residual stream after every layer."""
    eps = cfg["norm"]["eps"]
    r = tensors["embed"].to(dtype)[torch.as_tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        a = mixer(layer["type"], r, sub(tensors, f"l{i}.mix.", dtype), layer["mixer"], eps)
        r = r + rms_norm(a, tensors[f"l{i}.norm1"].to(dtype), eps)
        if layer.get("mlp") is not None:
            f = feed_forward(r, sub(tensors, f"l{i}.mlp.", dtype))
            r = r + rms_norm(f, tensors[f"l{i}.norm2"].to(dtype), eps)
        if layers_out is not None:
            layers_out.append(r.clone())
    return rms_norm(r, tensors["final.norm"].to(dtype), eps) @ tensors["head"].to(dtype).T
