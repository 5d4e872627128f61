"""A plain, slow implementation of the Fomodra design in float64, one function per mechanism, written from the
design's equations and sharing no code with the package.  It is the oracle of the tests.

A model is (cfg, W): cfg the dictionary that config.json holds, W a dictionary name -> float64 tensor.
`forward(cfg, W, tokens)` runs a whole sequence from its first token and returns the logits at every position (and,
when asked, the residual stream after every layer).  Nothing is carried between calls: a sequence that the package
runs in pieces, in a batch or token by token is compared with this one pass over all of it.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    return unit_rms(x, eps) * w


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def softplus(z: torch.Tensor) -> torch.Tensor:
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


# ------------------------------------------------------------------------------------------------ embedding
def embedding(cfg, W, tokens: List[int]) -> torch.Tensor:
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)].clone()
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        n, rows, prev = big["buckets"], [], None
        for t in tokens:
            rows.append(n if prev is None else (prev * big["mul_prev"] + t * big["mul_cur"]) % n)
            prev = t
        x = x + W["bigram"][torch.tensor(rows, dtype=torch.long)]
    return x


# ------------------------------------------------------------------------------------------------- rotation
def rotary_frequencies(rot) -> torch.Tensor:
    dims = rot["dims"]
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, orig = float(sc["factor"]), float(sc["low"]), float(sc["high"]), float(sc["original"])
        out = []
        for x in f.tolist():
            wave = 2.0 * math.pi / x
            if wave < orig / high:
                out.append(x)
            elif wave > orig / low:
                out.append(x / factor)
            else:
                s = (orig / wave - low) / (high - low)
                out.append((1.0 - s) * x / factor + s * x)
        f = torch.tensor(out, dtype=F64)
    return f


def rotate(x: torch.Tensor, positions: torch.Tensor, rot) -> torch.Tensor:
    """x [T, heads, n]: the first rot.dims entries of every head are turned, entry i with entry i + dims/2."""
    dims = rot["dims"]
    half = dims // 2
    ang = positions.to(F64)[:, None] * rotary_frequencies(rot)[None, :]          # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# -------------------------------------------------------------------------------------------------- masks
def visible(T: int, mask, kind: str) -> torch.Tensor:
    """[T, T] of booleans: whether position i (row) sees position j (column)."""
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    ok = j <= i
    if mask is None:
        return ok
    if kind == "window":
        return ok & (i - j < mask["size"])
    if kind == "chunk":
        return ok & (i // mask["size"] == j // mask["size"])
    raise ValueError(kind)


def softmax_attention(q, k, v, scale: float, seen: torch.Tensor, sink: Optional[torch.Tensor]) -> torch.Tensor:
    """q [T, H, D], k [T, G, D], v [T, G, Dv] -> [T, H, Dv]; sink [H]: a learned score that only the denominator counts."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~seen, -math.inf)
        m = s.max(dim=-1, keepdim=True).values
        if sink is not None:
            m = torch.maximum(m, sink[h].expand_as(m))
        e = torch.exp(s - m)
        den = e.sum(dim=-1, keepdim=True)
        if sink is not None:
            den = den + torch.exp(sink[h] - m)
        out[:, h] = (e / den) @ v[:, g]
    return out


# ---------------------------------------------------------------------------------------------- attention
def attention_keys_values(m, W, p: str, h: torch.Tensor, positions: torch.Tensor):
    """Rotated keys [T, G, D] and values [T, G, Dv] of a layer that has projections of its own."""
    G, D, Dv = m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    k, v = h @ W[p + "k"].T, h @ W[p + "v"].T
    if p + "k.b" in W:
        k, v = k + W[p + "k.b"], v + W[p + "v.b"]
    k = k.view(T, G, D)
    if m.get("rot"):
        k = rotate(k, positions, m["rot"])
    return k, v.view(T, G, Dv)


def attention_mixer(m, W, p: str, h: torch.Tensor, kv, mask_kind: str, with_sink: bool) -> torch.Tensor:
    """kv: (keys, values) as some layer cached them (its own or another's)."""
    H, D, Dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = h @ W[p + "q"].T
    if p + "q.b" in W:
        q = q + W[p + "q.b"]
    q = q.view(T, H, D)
    if m.get("rot"):
        q = rotate(q, positions, m["rot"])
    k, v = kv
    o = softmax_attention(q, k, v, float(m["scale"]), visible(T, m.get("mask"), mask_kind), W[p + "sink"] if with_sink else None)
    return o.reshape(T, H * Dv) @ W[p + "o"].T


# ------------------------------------------------------------------------------------------ latent attention
def latent_mixer(m, eps: float, W, p: str, h: torch.Tensor) -> torch.Tensor:
    H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, D + R)
    q_plain, q_rot = q[..., :D], rotate(q[..., D:], positions, m["rot"])
    down = h @ W[p + "dkv"].T
    c = rms_norm(down[:, :C], W[p + "dkv.norm"], eps)
    k_rot = rotate(down[:, None, C:], positions, m["rot"])                      # [T, 1, R], shared by the heads
    k_plain = (c @ W[p + "uk"].T).view(T, H, D)
    v = (c @ W[p + "uv"].T).view(T, H, Dv)
    qq = torch.cat([q_plain, q_rot], dim=-1)
    kk = torch.cat([k_plain, k_rot.expand(T, H, R)], dim=-1)
    o = softmax_attention(qq, kk, v, float(m["scale"]), visible(T, m.get("mask"), "window"), W[p + "sink"])
    gate = torch.sigmoid(h @ W[p + "g"].T)                                     # [T, H]
    o = o * gate[:, :, None]
    return o.reshape(T, H * Dv) @ W[p + "o"].T


# -------------------------------------------------------------------------------------------- selective scan
def causal_conv(u: torch.Tensor, taps: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """u [T, C]; taps [C, K], the last column weighing the current row, zeros in front of the sequence."""
    T, K = u.shape[0], taps.shape[1]
    full = torch.cat([torch.zeros(K - 1, u.shape[1], dtype=F64), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + full[j:j + T] * taps[:, j]
    return y + bias


def selective_scan_mixer(m, W, p: str, h: torch.Tensor) -> torch.Tensor:
    inner, N, R = m["inner"], m["state"], m["dt_rank"]
    T = h.shape[0]
    xz = h @ W[p + "in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    x = silu(causal_conv(x, W[p + "conv"], W[p + "conv.b"]))
    low = x @ W[p + "x"].T
    dt, B, C = low[:, :R], low[:, R:R + N], low[:, R + N:]
    dt = softplus(dt @ W[p + "dt"].T + W[p + "dt.b"])                          # [T, inner]
    A = -torch.exp(W[p + "A_log"])                                              # [inner, N]
    S = torch.zeros(inner, N, dtype=F64)
    y = torch.zeros(T, inner, dtype=F64)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * x[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + W[p + "D"] * x[t]
    return (y * silu(z)) @ W[p + "o"].T


def parallel_mixer(m, eps: float, W, p: str, h: torch.Tensor) -> torch.Tensor:
    left = m["left"]
    kv = attention_keys_values(left, W, p + "left.", h, torch.arange(h.shape[0]))
    a = attention_mixer(left, W, p + "left.", h, kv, "chunk", with_sink=False)
    b = selective_scan_mixer(m["right"], W, p + "right.", h)
    return 0.5 * (rms_norm(a, W[p + "left.out"], eps) + rms_norm(b, W[p + "right.out"], eps))


# ---------------------------------------------------------------------------------------------- feed-forward
def expert(W, p: str, h: torch.Tensor, limit: float) -> torch.Tensor:
    g = torch.clamp(h @ W[p + "gate"].T, max=limit)
    u = torch.clamp(h @ W[p + "up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


def route(mlp, W, p: str, h: torch.Tensor):
    """Chosen experts [T, top] and their weights; identity experts have the last numbers."""
    z = h @ W[p + "router"].T
    s = torch.softmax(z, dim=-1)
    choice = s + W[p + "correction"]
    ids = torch.topk(choice, mlp["router"]["top"], dim=-1).indices
    w = torch.gather(s, 1, ids)
    return ids, w / (w.sum(dim=-1, keepdim=True) + 1e-20)


def moe(mlp, W, p: str, h: torch.Tensor, ids=None) -> torch.Tensor:
    n = mlp["router"]["experts"]
    if ids is None:
        ids, w = route(mlp, W, p, h)
    else:                                        # a choice given from outside: the weights follow it
        s = torch.softmax(h @ W[p + "router"].T, dim=-1)
        w = torch.gather(s, 1, ids)
        w = w / (w.sum(dim=-1, keepdim=True) + 1e-20)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for r in range(ids.shape[1]):
            e = int(ids[t, r])
            y = h[t] if e >= n else expert(W, f"{p}e{e}.", h[t:t + 1], float(mlp["expert"]["limit"]))[0]
            out[t] = out[t] + w[t, r] * y
    if mlp.get("shared"):
        out = out + expert(W, p + "shared.", h, float(mlp["shared"]["limit"]))
    return out


def token_side(cfg, W, i: int, x: torch.Tensor, tokens: List[int], eps: float) -> torch.Tensor:
    dim = cfg["token_side"]["dim"]
    e = W["side.embed"][torch.tensor(tokens, dtype=torch.long)][:, i * dim:(i + 1) * dim]
    y = (gelu_tanh(x @ W[f"l{i}.side.gate"].T) * e) @ W[f"l{i}.side.proj"].T
    return x + rms_norm(y, W[f"l{i}.side.norm"], eps)


# --------------------------------------------------------------------------------------------------- model
def forward(cfg, W: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None,
            choices: Optional[Dict[int, torch.Tensor]] = None, routed: Optional[dict] = None) -> torch.Tensor:
    """Logits [T, vocab] of a whole sequence.  layers_out: a list that receives the stream after every layer.
    choices: layer -> experts [T, top] to use instead of the router's own choice; routed: a dictionary that receives
    every layer's router scores with the correction added (for tests that look for near ties)."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    x = embedding(cfg, W, tokens)
    positions = torch.arange(T)
    cached = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        h = rms_norm(x, W[f"l{i}.norm1"], eps)
        if layer["type"] == "attention":
            if m.get("kv_from") is not None:
                kv = cached[m["kv_from"]]
            else:
                kv = cached[i] = attention_keys_values(m, W, p, h, positions)
            y = attention_mixer(m, W, p, h, kv, "window", with_sink=True)
        elif layer["type"] == "latent_attention":
            y = latent_mixer(m, eps, W, p, h)
        elif layer["type"] == "parallel":
            y = parallel_mixer(m, eps, W, p, h)
        else:
            raise ValueError(layer["type"])
        x = x + rms_norm(y, W[f"l{i}.norm1b"], eps)
        if layer.get("mlp"):
            h = rms_norm(x, W[f"l{i}.norm2"], eps)
            if routed is not None:
                routed[i] = torch.softmax(h @ W[f"l{i}.mlp.router"].T, dim=-1) + W[f"l{i}.mlp.correction"]
            y = moe(layer["mlp"], W, f"l{i}.mlp.", h, None if choices is None else choices.get(i))
            x = x + rms_norm(y, W[f"l{i}.norm2b"], eps)
        if cfg.get("token_side"):
            x = token_side(cfg, W, i, x, tokens, eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
