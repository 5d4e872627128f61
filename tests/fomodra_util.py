"""Small Fomodra configurations with weights of the tests' own making, as the plain implementation's dict and as an
engine of the package.

The configurations differ from each other in every size and constant and avoid coincidences that would hide a fault:
heads and key/value heads differ, key and value sizes differ, fewer entries are rotated than a head holds in one layer
and all of them in another, windows and chunks shorter than a page and longer, a layer without a mask and without a
rotation, a layer that reads another layer's keys behind a window of its own, a layer without a feed-forward, states
that fill a lane's share exactly and states that do not, mixtures with and without identity experts and shared expert,
multipliers of the pair hash that overflow 32 bits.  Scales are chosen so that attention is peaked and decays are slow.
"""
import copy
import functools

import torch


def _moe(experts, identity, top, ff, limit, shared=None):
    m = {"kind": "moe", "router": {"experts": experts, "identity": identity, "top": top}, "expert": {"ff": ff, "limit": limit}}
    if shared:
        m["shared"] = {"ff": shared[0], "limit": shared[1]}
    return m


SMALL = {
    "architecture": "Fomodra", "vocab": 197, "width": 72, "norm": {"eps": 1e-5}, "token_side": {"dim": 5},
    "embedding": {"bigram": {"buckets": 101, "mul_prev": 13, "mul_cur": 5}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.3, "mask": {"size": 13},
                                        "rot": {"base": 100.0, "dims": 16}}, "mlp": _moe(5, 2, 3, 28, 1.5, (20, 2.5))},
        {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.4, "mask": {"size": 11},
                                                "rot": {"base": 50.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}},
                                       "right": {"inner": 40, "state": 20, "dt_rank": 5, "conv": 3}}, "mlp": _moe(4, 0, 2, 16, 1.0)},
        {"type": "latent_attention", "mixer": {"heads": 3, "dim": 20, "rot_dim": 12, "vdim": 28, "kv_rank": 36, "scale": 0.25,
                                               "mask": {"size": 17}, "rot": {"base": 50.0, "dims": 8}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 40, "scale": 0.25, "mask": {"size": 29}, "kv_from": 0,
                                        "rot": {"base": 100.0, "dims": 16}}, "mlp": _moe(3, 1, 1, 24, 2.0, (12, 1.0))},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 32, "vdim": 32, "scale": 0.2}, "mlp": _moe(6, 1, 2, 8, 1.0)},
    ],
}

# Sizes that reach the tensor-core products (multiples of 8), the tiled attention kernel of prompts and the decode kernel
# of single tokens (keys and values of 64 and of 128 entries), the tiled path of latent attention (dim + rot_dim = vdim =
# 64) and the experts' tiles.
WIDE = {
    "architecture": "Fomodra", "vocab": 520, "width": 256, "norm": {"eps": 1e-6}, "token_side": {"dim": 16},
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 9999991, "mul_cur": 3}},
    "layers": [
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.2, "mask": {"size": 70},
                                        "rot": {"base": 10000.0, "dims": 64}}, "mlp": _moe(8, 2, 3, 48, 1.25, (80, 2.5))},
        {"type": "parallel", "mixer": {"left": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.15, "mask": {"size": 96},
                                                "rot": {"base": 5000.0, "dims": 64, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 128}}},
                                       "right": {"inner": 512, "state": 16, "dt_rank": 16, "conv": 4}}, "mlp": _moe(8, 0, 2, 56, 1.5)},
        {"type": "latent_attention", "mixer": {"heads": 4, "dim": 48, "rot_dim": 16, "vdim": 64, "kv_rank": 64, "scale": 0.2,
                                               "mask": {"size": 100}, "rot": {"base": 5000.0, "dims": 16}}, "mlp": _moe(4, 4, 2, 32, 1.5, (64, 1.0))},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 64, "vdim": 64, "scale": 0.15, "mask": {"size": 150}, "kv_from": 0,
                                        "rot": {"base": 10000.0, "dims": 64}}, "mlp": _moe(6, 1, 2, 72, 0.75)},
        {"type": "parallel", "mixer": {"left": {"heads": 4, "kv_heads": 1, "dim": 64, "vdim": 64, "scale": 0.2, "mask": {"size": 64},
                                                "rot": {"base": 100.0, "dims": 32}},
                                       "right": {"inner": 256, "state": 64, "dt_rank": 8, "conv": 2}}, "mlp": None},
    ],
}

CONFIGS = {"small": SMALL, "wide": WIDE}


def config(name):
    return copy.deepcopy(CONFIGS[name])


def all_chosen(cfg):
    """The same model with every expert chosen for every token: no choice is left that a rounding could turn, so runs in
    bfloat16 can be compared row by row.  The weights of the original fit."""
    cfg = copy.deepcopy(cfg)
    for layer in cfg["layers"]:
        if layer.get("mlp"):
            r = layer["mlp"]["router"]
            r["top"] = r["experts"] + r.get("identity", 0)
    return cfg


def make_weights(cfg, seed=0, gain=1.3):
    """name -> float32 tensor holding bfloat16 values.  Projections N(0, gain^2/in), so that rows stay of order one."""
    g = torch.Generator().manual_seed(seed)
    E, V, w = cfg["width"], cfg["vocab"], {}

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def near_one(n):
        return 1.0 + 0.2 * torch.randn(n, generator=g)

    def between(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    def attention(p, m, bias, sink):
        H, D, G, Dv = m["heads"], m["dim"], m.get("kv_heads") or m["heads"], m.get("vdim") or m["dim"]
        names = [("q", H * D, gain)] + ([] if m.get("kv_from") is not None else [("k", G * D, gain), ("v", G * Dv, gain)])
        for n, rows, gn in names:
            w[p + n] = mat(rows, E, gn)
            if bias:
                w[p + n + ".b"] = 0.3 * torch.randn(rows, generator=g)
        w[p + "o"] = mat(E, H * Dv)
        if sink:
            w[p + "sink"] = between(H, -1.0, 2.0)

    w["embed"] = torch.randn(V, E, generator=g) * 0.7
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        w["bigram"] = torch.randn(big["buckets"] + 1, E, generator=g) * 0.5
    side = cfg.get("token_side")
    if side:
        w["side.embed"] = torch.randn(V, side["dim"] * len(cfg["layers"]), generator=g)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        for n in ("norm1", "norm1b"):
            w[f"l{i}.{n}"] = near_one(E)
        if layer["type"] == "attention":
            attention(p, m, True, True)
        elif layer["type"] == "latent_attention":
            H, D, R, Dv, C = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            w[p + "q"], w[p + "dkv"], w[p + "dkv.norm"] = mat(H * (D + R), E, gain), mat(C + R, E, gain), near_one(C)
            w[p + "uk"], w[p + "uv"], w[p + "o"] = mat(H * D, C, gain), mat(H * Dv, C, gain), mat(E, H * Dv)
            w[p + "sink"], w[p + "g"] = between(H, -1.0, 2.0), mat(H, E, 2.0)
        else:
            attention(p + "left.", m["left"], False, False)
            r, q = m["right"], p + "right."
            I, N, R, K = r["inner"], r["state"], r["dt_rank"], r["conv"]
            w[q + "in"], w[q + "conv"], w[q + "conv.b"] = mat(2 * I, E, gain), between((I, K), -0.6, 0.6), between(I, -0.2, 0.2)
            w[q + "x"], w[q + "dt"], w[q + "dt.b"] = mat(R + 2 * N, I, gain), mat(I, R, 1.0), between(I, -4.0, -1.0)
            w[q + "A_log"], w[q + "D"], w[q + "o"] = between((I, N), -2.0, 1.0), near_one(I), mat(E, I)
            w[p + "left.out"], w[p + "right.out"] = near_one(E), near_one(E)
        mlp = layer.get("mlp")
        if mlp:
            q, F = f"l{i}.mlp.", mlp["expert"]["ff"]
            n, extra = mlp["router"]["experts"], mlp["router"].get("identity", 0)
            for n2 in ("norm2", "norm2b"):
                w[f"l{i}.{n2}"] = near_one(E)
            for e in range(n):
                w[f"{q}e{e}.gate"], w[f"{q}e{e}.up"], w[f"{q}e{e}.down"] = mat(F, E, 1.5), mat(F, E, 1.5), mat(E, F)
            w[q + "router"], w[q + "correction"] = mat(n + extra, E, 2.5), 0.05 * torch.randn(n + extra, generator=g)
            if mlp.get("shared"):
                Fs = mlp["shared"]["ff"]
                w[q + "shared.gate"], w[q + "shared.up"], w[q + "shared.down"] = mat(Fs, E, 1.5), mat(Fs, E, 1.5), mat(E, Fs)
        if side:
            d = side["dim"]
            w[f"l{i}.side.gate"], w[f"l{i}.side.proj"], w[f"l{i}.side.norm"] = mat(d, E, 1.5), mat(E, d), 0.5 * near_one(E)
    w["final.norm"] = near_one(E)
    w["head"] = mat(V, E, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def weights(name, seed=0):
    return make_weights(CONFIGS[name], seed)


def as_plain(w):
    """The weights as the plain implementation takes them (float64)."""
    return {k: v.double() for k, v in w.items()}


def build(cfg, w, dtype):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.weights import TensorSource
    return _build(copy.deepcopy(cfg), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="test weights"),
                  dtype, "cuda:0")


@functools.lru_cache(maxsize=None)
def llm(name, dtype, dense=False, seed=0):
    cfg = all_chosen(CONFIGS[name]) if dense else CONFIGS[name]
    return build(cfg, weights(name, seed), dtype)


def new_engine(name, dtype, dense=False, n_tokens=2048, n_slots=8, **kw):
    from gguf_rs_cli_b200.engine.step import Engine
    return Engine(llm(name, dtype, dense).model, n_tokens=n_tokens, n_slots=n_slots, **kw)


def tokens_of(name, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CONFIGS[name]["vocab"], (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name, n, seed, dense=False):
    from tests import plain_fomodra as P
    cfg = all_chosen(CONFIGS[name]) if dense else CONFIGS[name]
    return P.forward(cfg, as_plain(weights(name)), tokens_of(name, n, seed)).float()
