"""A plain, slow implementation of the Folivik design from its equations: one function per
mechanism, float64 on the CPU, one sequence at a time, attention as whole matrices and the
recurrence token by token.  It shares no code with the engine; the tests hold the engine to
it.

Notation: T tokens of one sequence at positions 0..T-1, h [T, width] a layer's normed input,
w a dict of float64 tensors by checkpoint name, p the name prefix of the part at hand, mx a
mixer's dict of sizes from the configuration.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ----------------------------------------------------------------------- small pieces
def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight; the weight may be one number."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotate_pairs(x, base: float, dims: int):
    """x [T, heads, d]: the pair (2i, 2i + 1) of the first ``dims`` sizes of every head turns
    by the angle p * base^(-2i / dims) at position p."""
    T = x.shape[0]
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    ang = torch.arange(T, dtype=F64)[:, None, None] * f[None, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def causal_conv(u, w, bias):
    """u [T, C], w [C, taps]: y_t = bias + sum_j w[:, j] u_{t - taps + 1 + j}, zeros before 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u) + bias
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def softmax_attention(q, k, v, scale, window: Optional[int], bias=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G);
    position i sees j <= i (and i - j < window when there is one).  ``scale`` a number or one
    per head; ``bias(h, dist)`` is taken off head h's scores, dist [T, T] = i - j."""
    T, H, _ = q.shape
    G = k.shape[1]
    i, j = torch.arange(T)[:, None], torch.arange(T)[None, :]
    dist = (i - j)
    seen = dist >= 0
    if window is not None:
        seen = seen & (dist < window)
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * (scale[h] if torch.is_tensor(scale) else scale)
        if bias is not None:
            s = s - bias(h, dist.clamp(min=0).to(F64))
        s = s.masked_fill(~seen, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


# ---------------------------------------------------------------------------- mixers
def latent_attention(h, w, p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, d, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    c_q = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (c_q @ w[p + "uq"].T).view(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    base, dims = mx["rot"]["base"], mx["rot"]["dims"]
    k_rot = rotate_pairs(down[:, rank:].view(T, 1, dr), base, dims)
    q_rot = rotate_pairs(q[..., d:], base, dims)
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, dr)], dim=-1)
    o = softmax_attention(qq, kk, v, mx["scale"], None)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def window_attention(h, w, p: str, mx: dict, eps: float):
    """Grouped attention with normed heads, a factor per head on the scores and a bias that
    grows with the logarithm of the distance, inside a sliding window."""
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx["kv_heads"], mx["dim"], mx["vdim"]
    q = rms_norm((h @ w[p + "q"].T).view(T, H, d), w[p + "q.norm"], eps)
    k = rms_norm((h @ w[p + "k"].T).view(T, G, d), w[p + "k.norm"], eps)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    r1, r2 = w[p + "r1"], w[p + "r2"]
    o = softmax_attention(q, k, v, mx["scale"] * w[p + "temp"], mx["mask"]["size"],
                          bias=lambda hd, dist: r1[hd] * torch.log1p(r2[hd] * dist))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def mamba2(h, w, p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, P, N, G = mx["heads"], mx["vdim"], mx["state"], mx["groups"]
    inner = H * P
    u = h @ w[p + "in"].T
    z, xbc, dt = u[:, :inner], u[:, inner:2 * inner + 2 * G * N], u[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w[p + "conv"], w[p + "conv.b"]))
    x = xbc[:, :inner].view(T, H, P)
    B = xbc[:, inner:inner + G * N].view(T, G, N)
    C = xbc[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + w[p + "dt_bias"])
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * dt)
    y = torch.zeros(T, H, P, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S + dt[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + w[p + "D"][hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = mx["norm_groups"]
    y = y.view(T, parts, inner // parts)
    y = (y / torch.sqrt((y * y).mean(-1, keepdim=True) + eps)).reshape(T, inner) * w[p + "norm"]
    return y @ w[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "attention": window_attention, "mamba2": mamba2}


# ---------------------------------------------------------------------- feed-forward
def expert(h, w, p: str):
    return (silu(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


def route(h, w, p: str, router: dict):
    """(ids [T, top], weights [T, top]) over the experts and the identity experts behind them."""
    s = torch.softmax(h @ w[p + "router"].T, dim=-1)
    choice = s + w[p + "correction"]
    n = s.shape[1]
    groups = router.get("groups")
    if groups and groups["count"] > 1:
        per = n // groups["count"]
        best = choice.view(-1, groups["count"], per).max(-1).values
        kept = best.topk(groups["keep"], dim=-1).indices
        allowed = torch.zeros_like(best, dtype=torch.bool).scatter_(1, kept, True)
        choice = choice.masked_fill(~allowed.repeat_interleave(per, dim=1), -math.inf)
    ids = choice.topk(router["top"], dim=-1).indices
    wts = s.gather(1, ids)
    return ids, wts / (wts.sum(-1, keepdim=True) + 1e-20) * router.get("scale", 1.0)


def mixture_of_experts(h, w, p: str, mlp: dict):
    router = mlp["router"]
    real = router["experts"]
    ids, wts = route(h, w, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wts[t]):
            out[t] += a * (expert(h[t:t + 1], w, f"{p}e{e}.")[0] if e < real else h[t])
    if mlp.get("shared"):
        out = out + expert(h, w, p + "shared.")
    return out


# ------------------------------------------------------------------------- the model
def forward(raw: dict, weights: Dict[str, torch.Tensor], tokens: List[int],
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence."""
    w = {n: t.to(F64) for n, t in weights.items()}
    eps = raw["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(raw["layers"]):
        p = f"l{i}."
        x = x + MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.",
                                      layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + mixture_of_experts(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.",
                                       layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
