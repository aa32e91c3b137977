"""A plain, slow implementation of the Ketopel design from its equations: one function per
mechanism, float64 on the CPU, one sequence at a time, attention as whole matrices and the
recurrences token by token.  It shares no code with the engine; the tests hold the engine
to it.

Notation: T tokens of one sequence at positions 0..T-1, h [T, width] a layer's normed input,
w a dict of float64 tensors by checkpoint name, p the name prefix of the part at hand.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


# ----------------------------------------------------------------------- small pieces
def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def silu(z):
    return z * torch.sigmoid(z)


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def rotary_table(rot: dict):
    """(frequencies [dims/2], magnitude).  With ``scaling`` (factor, original, fast, slow):
    the index at which a wave makes t turns over ``original`` positions is
    n(t) = dims ln(original / (2 pi t)) / (2 ln base); between lo = floor(n(fast)) and
    hi = ceil(n(slow)) the frequency goes over from f_i to f_i / factor, and cosines and sines
    grow by 0.1 ln(factor) + 1."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0

    def index_of(turns):
        return dims * math.log(sc["original"] / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(index_of(sc["fast"])), 0)
    hi = min(math.ceil(index_of(sc["slow"])), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / sc["factor"] * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(sc["factor"]) + 1.0


def rotate(x, rot: Optional[dict], interleaved: bool, first_position: int = 0):
    """x [T, heads, d]: the first ``dims`` sizes of every head turn by p f_i, in pairs
    (i, i + dims/2), or (2i, 2i + 1) when ``interleaved``."""
    if not rot:
        return x
    dims = int(rot["dims"])
    half = dims // 2
    f, mag = rotary_table(rot)
    pos = torch.arange(first_position, first_position + x.shape[0], dtype=F64)
    ang = pos[:, None, None] * f[None, None, :]
    c, s = torch.cos(ang) * mag, torch.sin(ang) * mag
    out = x.clone()
    if interleaved:
        a, b = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = a * c - b * s
        out[..., 1:dims:2] = b * c + a * s
    else:
        a, b = x[..., :half], x[..., half:dims]
        out[..., :half] = a * c - b * s
        out[..., half:dims] = b * c + a * s
    return out


def causal_conv(u, w):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_{t - taps + 1 + j}, zeros before 0."""
    T, taps = u.shape[0], w.shape[1]
    y = torch.zeros_like(u)
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j] * u[:T - back]
    return y


def causal_softmax_attention(q, k, v, scale: float, softcap: Optional[float]):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; query head h reads key head h // (H / G)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    mask = torch.tril(torch.ones(T, T, dtype=torch.bool))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~mask, -math.inf)
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


# ---------------------------------------------------------------------------- mixers
def whole_norm_attention(h, w, p: str, mx: dict, eps: float):
    """Grouped softmax attention whose q and k are normed over all heads at once."""
    T = h.shape[0]
    H, G = mx["heads"], mx.get("kv_heads") or mx["heads"]
    d, dv = mx["dim"], mx.get("vdim") or mx["dim"]
    q = rms_norm(h @ w[p + "q"].T, w[p + "q.norm"], eps).view(T, H, d)
    k = rms_norm(h @ w[p + "k"].T, w[p + "k.norm"], eps).view(T, G, d)
    v = (h @ w[p + "v"].T).view(T, G, dv)
    q, k = rotate(q, mx.get("rot"), False), rotate(k, mx.get("rot"), False)
    o = causal_softmax_attention(q, k, v, mx["scale"], mx.get("softcap"))
    return o.reshape(T, H * dv) @ w[p + "o"].T


def lightning_attention(h, w, p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, d, dv = mx["heads"], mx["dim"], mx.get("vdim") or mx["dim"]
    q = silu(h @ w[p + "q"].T).view(T, H, d)
    k = silu(h @ w[p + "k"].T).view(T, H, d)
    v = silu(h @ w[p + "v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = mx["decay"][hd] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = rms_norm(o.reshape(T, H * dv), w[p + "norm"], eps)
    return (o * torch.sigmoid(h @ w[p + "g"].T)) @ w[p + "o"].T


def side_by_side(h, w, p: str, mx: dict, eps: float):
    return (mx.get("left_scale", 1.0) * whole_norm_attention(h, w, p + "left.", mx["left"], eps)
            + mx.get("right_scale", 1.0) * lightning_attention(h, w, p + "right.", mx["right"], eps))


def latent_attention(h, w, p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, d, dr, dv, rank = mx["heads"], mx["dim"], mx["rot_dim"], mx["vdim"], mx["kv_rank"]
    q = (h @ w[p + "q"].T).view(T, H, d + dr)
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :rank], w[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, rank:].view(T, 1, dr), mx["rot"], True)
    q_rot = rotate(q[..., d:], mx["rot"], True)
    k_plain = (c @ w[p + "uk"].T).view(T, H, d)
    v = (c @ w[p + "uv"].T).view(T, H, dv)
    qq = torch.cat([q[..., :d], q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, dr)], dim=-1)
    o = causal_softmax_attention(qq, kk, v, mx["scale"], None)
    o = o * torch.sigmoid(h @ w[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ w[p + "o"].T


def gated_delta_rule(h, w, p: str, mx: dict, eps: float):
    T = h.shape[0]
    H, G, d, dv = mx["heads"], mx.get("kv_heads") or mx["heads"], mx["dim"], mx["vdim"]
    q = silu(causal_conv(h @ w[p + "q"].T, w[p + "q.conv"])).view(T, G, d)
    k = silu(causal_conv(h @ w[p + "k"].T, w[p + "k.conv"])).view(T, G, d)
    v = silu(causal_conv(h @ w[p + "v"].T, w[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w[p + "b"].T)
    decay = torch.exp(-torch.exp(w[p + "A_log"]) * softplus(h @ w[p + "a"].T + w[p + "dt_bias"]))
    o = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            o[t, hd] = S.T @ q[t, g]
    o = rms_norm(o, w[p + "norm"], eps).reshape(T, H * dv)
    return (o * silu(h @ w[p + "g"].T)) @ w[p + "o"].T


MIXERS = {"parallel": side_by_side, "latent_attention": latent_attention,
          "delta": gated_delta_rule}


# ---------------------------------------------------------------------- feed-forward
def dense_feed_forward(h, w, p: str):
    return (gelu_tanh(h @ w[p + "gate"].T) * (h @ w[p + "up"].T)) @ w[p + "down"].T


# ------------------------------------------------------------------------- the model
def layer_order(raw: dict) -> List[tuple]:
    """(layer, pass number or None, first of its pass) for every layer run, in order."""
    n = len(raw["layers"])
    loop = raw.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    runs = [(i, None, False) for i in range(a)]
    for t in range(times):
        runs += [(i, t, i == a) for i in range(a, b)]
    return runs + [(i, None, False) for i in range(b, n)]


def forward(raw: dict, weights: Dict[str, torch.Tensor], tokens: List[int],
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] (float64) of one sequence."""
    w = {n: t.to(F64) for n, t in weights.items()}
    eps = raw["norm"]["eps"]
    x0 = w["embed"][torch.tensor(tokens, dtype=torch.long)] * raw.get("embedding", {}).get("scale", 1.0)
    x = x0.clone()
    for i, t, first in layer_order(raw):
        layer, p = raw["layers"][i], f"l{i}."
        if first:
            if t > 0:
                x = x + x0
            x = x + w["loop.step"][t]
        x = x + MIXERS[layer["type"]](rms_norm(x, w[p + "norm1"], eps), w, p + "mix.",
                                      layer["mixer"], eps)
        if layer.get("mlp") is not None:
            x = x + dense_feed_forward(rms_norm(x, w[p + "norm2"], eps), w, p + "mlp.")
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T
