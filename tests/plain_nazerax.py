"""A plain, slow implementation of the Nazerax design in float64, one function per mechanism, written from
the design's equations and sharing no code with the package.  It is the oracle of the tests.

A model is (cfg, W): cfg the dictionary that config.json holds, W a dictionary name -> float64 tensor (integer
tables stay integers).  `forward(cfg, W, tokens)` runs a whole sequence and returns the logits at every position;
`Stepper` runs a sequence piece by piece from states that it carries, which is how the mechanisms are defined.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def layer_norm_zero_centred(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """RMS norm whose weight is stored around zero."""
    return unit_rms(x, eps) * (1.0 + w)


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ------------------------------------------------------------------------------------------------ embedding
def bigram_rows(tokens: List[int], prev: Optional[int], buckets: int, mul_prev: int, mul_cur: int) -> List[int]:
    """Row of the bigram table for each token; prev is the token before the first of `tokens` (None: the
    sequence starts here)."""
    rows = []
    for t in tokens:
        rows.append(buckets if prev is None else (prev * mul_prev + t * mul_cur) % buckets)
        prev = t
    return rows


def embedding(cfg, W, tokens: List[int], prev: Optional[int]) -> torch.Tensor:
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)].clone()
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        rows = bigram_rows(tokens, prev, big["buckets"], big["mul_prev"], big["mul_cur"])
        x = x + W["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


# -------------------------------------------------------------------------------------------- short convolution
def short_conv(u: torch.Tensor, taps: torch.Tensor, before: torch.Tensor, bias: Optional[torch.Tensor] = None):
    """u [T, C]; taps [C, K], the last column weighing the current row; before [K-1, C]: the rows in front of u (zeros
    at a sequence's start).  Returns (y [T, C], the last K-1 rows seen)."""
    K = taps.shape[1]
    full = torch.cat([before, u], dim=0)
    T = u.shape[0]
    y = torch.zeros_like(u)
    for t in range(T):
        for j in range(K):
            y[t] += taps[:, j] * full[t + j]
    if bias is not None:
        y = y + bias
    return y, full[full.shape[0] - (K - 1):].clone() if K > 1 else before


# ------------------------------------------------------------------------------------------------------ wkv
def wkv_mixer(m, eps, W, p, h: torch.Tensor, state: Dict) -> torch.Tensor:
    """state: 'prev' [E] the previous token's input, 'S' [heads, dim, dim]."""
    H, D = m["heads"], m["dim"]
    T = h.shape[0]
    if "prev" not in state:
        state["prev"] = torch.zeros(h.shape[1], dtype=F64)
        state["S"] = torch.zeros(H, D, D, dtype=F64)
    before = torch.cat([state["prev"][None], h[:-1]], dim=0)
    state["prev"] = h[-1].clone()
    mixed = {s: h + (before - h) * W[p + "mu." + s] for s in "rkvgw"}
    r = (mixed["r"] @ W[p + "r"].T).view(T, H, D)
    k = (mixed["k"] @ W[p + "k"].T).view(T, H, D)
    v = (mixed["v"] @ W[p + "v"].T).view(T, H, D)
    gate = silu(mixed["g"] @ W[p + "g"].T)
    lw = torch.tanh(mixed["w"] @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"]
    decay = torch.exp(-torch.exp(lw)).view(T, H, D)
    u = W[p + "u"].view(H, D)
    S = state["S"]
    out = torch.zeros(T, H, D, dtype=F64)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]                     # [H, D(key), D(value)]
        out[t] = torch.einsum("hij,hi->hj", S + u[:, :, None] * kv, r[t])
        S = decay[t][:, :, None] * S + kv
    state["S"] = S
    o = unit_rms(out, eps).reshape(T, H * D) * W[p + "norm"] * gate
    return o @ W[p + "o"].T


# --------------------------------------------------------------------------------------------------- mamba2
def mamba2_mixer(m, eps, W, p, h: torch.Tensor, state: Dict) -> torch.Tensor:
    """state: 'conv' [taps-1, channels] the convolution's last inputs, 'S' [heads, N, vdim]."""
    H, P, N, G, K, NG = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"], m["norm_groups"]
    inner, T = H * P, h.shape[0]
    C = inner + 2 * G * N
    if "S" not in state:
        state["S"] = torch.zeros(H, N, P, dtype=F64)
        state["conv"] = torch.zeros(K - 1, C, dtype=F64)
    proj = h @ W[p + "in"].T
    z, xbc, dt = proj[:, :inner], proj[:, inner:inner + C], proj[:, inner + C:]
    y, state["conv"] = short_conv(xbc, W[p + "conv"], state["conv"], W[p + "conv.b"])
    y = silu(y)
    x = y[:, :inner].view(T, H, P)
    Bm = y[:, inner:inner + G * N].view(T, G, N)
    Cm = y[:, inner + G * N:].view(T, G, N)
    dt = softplus(dt + W[p + "dt_bias"])                              # [T, H]
    decay = torch.exp(-torch.exp(W[p + "A_log"]) * dt)                # [T, H]
    per = H // G
    S = state["S"]
    out = torch.zeros(T, H, P, dtype=F64)
    for t in range(T):
        for hh in range(H):
            g = hh // per
            S[hh] = decay[t, hh] * S[hh] + dt[t, hh] * Bm[t, g][:, None] * x[t, hh][None, :]
            out[t, hh] = S[hh].T @ Cm[t, g] + W[p + "D"][hh] * x[t, hh]
    state["S"] = S
    gated = out.reshape(T, inner) * silu(z)
    normed = unit_rms(gated.view(T, NG, inner // NG), eps).reshape(T, inner) * W[p + "norm"]
    return normed @ W[p + "o"].T


# ------------------------------------------------------------------------------------------------- attention
def rotate_interleaved(x: torch.Tensor, positions: torch.Tensor, dims: int, base: float) -> torch.Tensor:
    """x [T, heads, dim]: the pairs (2i, 2i+1), i < dims/2, are turned by position * base^(-2i/dims)."""
    if not dims:
        return x
    i = torch.arange(dims // 2, dtype=F64)
    ang = positions.to(F64)[:, None] * base ** (-2.0 * i / dims)       # [T, dims/2]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    out = x.clone()
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def attention_mixer(m, eps, W, p, h: torch.Tensor, state: Dict) -> torch.Tensor:
    """state: 'k' [n, G, dim], 'v' [n, G, vdim]: everything so far (the window is applied when reading), 'conv_q',
    'conv_k', 'conv_v': the convolutions' last inputs."""
    H, D = m["heads"], m["dim"]
    G, Dv = m.get("kv_heads") or H, m.get("vdim") or D
    K = m.get("conv") or 1
    T = h.shape[0]
    if "k" not in state:
        state["k"], state["v"] = torch.zeros(0, G, D, dtype=F64), torch.zeros(0, G, Dv, dtype=F64)
        for n, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
            state["conv_" + n] = torch.zeros(K - 1, c, dtype=F64)
    start = state["k"].shape[0]
    pos = torch.arange(start, start + T)
    proj = {}
    for n in "qkv":
        y = h @ W[p + n].T
        if K > 1:
            y, state["conv_" + n] = short_conv(y, W[p + n + ".conv"], state["conv_" + n])
        proj[n] = y
    rot = m.get("rot") or {}
    q = rotate_interleaved(proj["q"].view(T, H, D), pos, rot.get("dims", 0), rot.get("base", 1.0))
    k = rotate_interleaved(proj["k"].view(T, G, D), pos, rot.get("dims", 0), rot.get("base", 1.0))
    v = proj["v"].view(T, G, Dv)
    state["k"], state["v"] = torch.cat([state["k"], k]), torch.cat([state["v"], v])
    scale = m["scale"] if m.get("scale") is not None else D ** -0.5
    size = (m.get("mask") or {}).get("size")
    gate = torch.sigmoid(h @ W[p + "g"].T)                            # [T, H]
    out = torch.zeros(T, H, Dv, dtype=F64)
    per = H // G
    for t in range(T):
        i = start + t
        lo = 0 if size is None else max(0, i - size + 1)
        for hh in range(H):
            g = hh // per
            s = (state["k"][lo:i + 1, g] @ q[t, hh]) * scale
            e = torch.exp(s)
            w = e / (1.0 + e.sum())                                   # a sink of score 0 that has no value
            out[t, hh] = (w[:, None] * state["v"][lo:i + 1, g]).sum(dim=0) * gate[t, hh]
    return out.reshape(T, H * Dv) @ W[p + "o"].T


# --------------------------------------------------------------------------------------------- feed-forward
def dense_ff(W, p, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


MIXERS = {"wkv": wkv_mixer, "mamba2": mamba2_mixer, "attention": attention_mixer}


def run_order(cfg) -> List[tuple]:
    """(layer, first of a pass but the first) for every layer run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop or loop.get("times", 1) <= 1:
        return [(i, False) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, False) for i in range(a)]
    for rep in range(times):
        order += [(i, rep > 0 and i == a) for i in range(a, b)]
    return order + [(i, False) for i in range(b, n)]


class Stepper:
    """One sequence, fed piece by piece."""

    def __init__(self, cfg, W):
        self.cfg, self.W = cfg, W
        self.order = run_order(cfg)
        self.states = [dict() for _ in self.order]
        self.prev_token: Optional[int] = None
        self.trace: List[torch.Tensor] = []            # the stream after every layer run of the last piece

    def feed(self, tokens: List[int]) -> torch.Tensor:
        cfg, W = self.cfg, self.W
        eps = cfg["norm"]["eps"]
        x0 = embedding(cfg, W, tokens, self.prev_token)
        self.prev_token = tokens[-1]
        x = x0.clone()
        self.trace = []
        for r, (i, again) in enumerate(self.order):
            layer, p = cfg["layers"][i], f"l{i}."
            if again:
                x = x + x0
            term = MIXERS[layer["type"]](layer["mixer"], eps, W, p + "mix.", layer_norm_zero_centred(x, W[p + "norm1"], eps),
                                         self.states[r])
            if layer.get("mlp") is not None:
                term = term + dense_ff(W, p + "mlp.", layer_norm_zero_centred(x, W[p + "norm2"], eps))
            x = x + term
            self.trace.append(x.clone())
        logits = layer_norm_zero_centred(x, W["final.norm"], eps) @ W["head"].T
        cap = cfg.get("logit_softcap")
        if cap:
            logits = cap * torch.tanh(logits / cap)
        return logits


def forward(cfg, W, tokens: List[int]) -> torch.Tensor:
    return Stepper(cfg, W).feed(list(tokens))
