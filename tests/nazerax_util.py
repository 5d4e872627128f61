"""Small Nazerax configurations with weights of the tests' own making, as the plain implementation's dict and as an
engine of the package.

The configurations differ from each other in every size and constant and avoid coincidences that would hide a fault:
heads and key/value heads differ, key and value sizes differ, fewer entries are rotated than a head holds in one layer
and all of them in another, a window shorter than a page and one longer, a layer without a window, one without a
convolution, one without a feed-forward, heads * dim of a wkv layer unlike the width, groups and norm groups of a
state-space layer unlike each other and unlike 1, convolutions of 2, 3 and 4 taps, a looped stretch that starts behind
the first layer and runs three times, multipliers of the pair hash that overflow 32 bits.  Scales are chosen so that
attention is peaked and decays are slow.
"""
import copy
import functools

import torch

from tests import plain_nazerax as P

SMALL = {
    "architecture": "Nazerax", "vocab": 197, "width": 72, "norm": {"eps": 1e-5}, "logit_softcap": 9.0,
    "embedding": {"bigram": {"buckets": 101, "mul_prev": 13, "mul_cur": 5}},
    "loop": {"start": 1, "stop": 4, "times": 3},
    "layers": [
        {"type": "attention", "mixer": {"heads": 6, "kv_heads": 3, "dim": 24, "vdim": 40, "conv": 4, "scale": 0.3,
                                        "mask": {"size": 13}, "rot": {"base": 100.0, "dims": 16}}, "mlp": {"kind": "dense", "ff": 136}},
        {"type": "wkv", "mixer": {"heads": 3, "dim": 20}, "mlp": None},
        {"type": "mamba2", "mixer": {"heads": 6, "vdim": 12, "state": 20, "groups": 3, "norm_groups": 2, "conv": 2},
         "mlp": {"kind": "dense", "ff": 100}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 16, "vdim": 8, "scale": 0.4,
                                        "rot": {"base": 50.0, "dims": 16}}, "mlp": {"kind": "dense", "ff": 64}},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 36}, "mlp": {"kind": "dense", "ff": 90}},
    ],
}
SMALL_RANKS = {1: 12, 4: 7}

# Sizes that reach the tensor-core products (multiples of 8), the tiled attention kernel of prompts and the decode kernel
# of single tokens (keys and values of 64 and of 128 entries); the looped stretch holds an attention layer, so that every
# pass keeps keys of its own.
WIDE = {
    "architecture": "Nazerax", "vocab": 520, "width": 256, "norm": {"eps": 1e-6}, "logit_softcap": 30.0,
    "embedding": {"bigram": {"buckets": 1000, "mul_prev": 9999991, "mul_cur": 3}},
    "loop": {"start": 0, "stop": 2, "times": 2},
    "layers": [
        {"type": "mamba2", "mixer": {"heads": 4, "vdim": 64, "state": 64, "groups": 1, "norm_groups": 1, "conv": 4},
         "mlp": {"kind": "dense", "ff": 360}},
        {"type": "attention", "mixer": {"heads": 8, "kv_heads": 2, "dim": 64, "vdim": 64, "conv": 3, "scale": 0.2,
                                        "mask": {"size": 70}, "rot": {"base": 5000.0, "dims": 32}}, "mlp": {"kind": "dense", "ff": 512}},
        {"type": "wkv", "mixer": {"heads": 2, "dim": 128}, "mlp": {"kind": "dense", "ff": 360}},
        {"type": "attention", "mixer": {"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "conv": 2, "scale": 0.15,
                                        "mask": {"size": 200}, "rot": {"base": 10000.0, "dims": 128}}, "mlp": None},
        {"type": "mamba2", "mixer": {"heads": 8, "vdim": 16, "state": 128, "groups": 2, "norm_groups": 4, "conv": 3},
         "mlp": {"kind": "dense", "ff": 200}},
    ],
}
WIDE_RANKS = {2: 32}

CONFIGS = {"small": (SMALL, SMALL_RANKS), "wide": (WIDE, WIDE_RANKS)}


def config(name):
    return copy.deepcopy(CONFIGS[name][0])


def make_weights(cfg, ranks, seed=0, gain=1.3):
    """name -> float32 tensor holding bfloat16 values.  Projections N(0, gain^2/in), so that rows stay of order one;
    norm weights around zero; decays slow, so that the first tokens still show at the end of a long sequence."""
    g = torch.Generator().manual_seed(seed)
    E, w = cfg["width"], {}

    def mat(o, i, gain=1.0):
        return torch.randn(o, i, generator=g) * gain / i ** 0.5

    def around_zero(n):
        return 0.2 * torch.randn(n, generator=g)

    def between(n, lo, hi):
        return torch.rand(n, generator=g) * (hi - lo) + lo

    w["embed"] = torch.randn(cfg["vocab"], E, generator=g) * 0.7
    big = (cfg.get("embedding") or {}).get("bigram")
    if big:
        w["bigram"] = torch.randn(big["buckets"] + 1, E, generator=g) * 0.5
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.mix.", layer["mixer"]
        w[f"l{i}.norm1"] = around_zero(E)
        if layer["type"] == "wkv":
            H, D, r = m["heads"], m["dim"], ranks[i]
            for s in "rkvgw":
                w[p + "mu." + s] = between(E, 0.0, 1.0)
            for s in "rkvg":
                w[p + s] = mat(H * D, E, gain)
            w[p + "w1"], w[p + "w2"] = mat(r, E, 2.0), mat(H * D, r, 1.5)
            w[p + "w0"] = between(H * D, -5.0, -1.5)
            w[p + "u"] = torch.randn(H, D, generator=g) * 0.5
            w[p + "norm"], w[p + "o"] = 1.0 + around_zero(H * D), mat(E, H * D)
        elif layer["type"] == "mamba2":
            H, Pv, N, G, K = m["heads"], m["vdim"], m["state"], m["groups"], m["conv"]
            inner, C = H * Pv, H * Pv + 2 * G * N
            w[p + "in"] = mat(inner + C + H, E, gain)
            w[p + "conv"], w[p + "conv.b"] = between((C, K), -0.6, 0.6), between(C, -0.2, 0.2)
            w[p + "dt_bias"], w[p + "A_log"], w[p + "D"] = between(H, -4.0, -1.0), between(H, -1.0, 1.0), 1.0 + around_zero(H)
            w[p + "norm"], w[p + "o"] = 1.0 + around_zero(inner), mat(E, inner)
        else:
            H, D = m["heads"], m["dim"]
            G, Dv, K = m.get("kv_heads") or H, m.get("vdim") or D, m.get("conv") or 1
            w[p + "q"], w[p + "k"], w[p + "v"] = mat(H * D, E, 2 * gain), mat(G * D, E, 2 * gain), mat(G * Dv, E, gain)
            w[p + "g"], w[p + "o"] = mat(H, E, 2.0), mat(E, H * Dv)
            if K > 1:
                for s, c in (("q", H * D), ("k", G * D), ("v", G * Dv)):
                    w[p + s + ".conv"] = between((c, K), -0.6, 0.6)
        if layer.get("mlp"):
            q, F = f"l{i}.mlp.", layer["mlp"]["ff"]
            w[f"l{i}.norm2"] = around_zero(E)
            w[q + "gate"], w[q + "up"], w[q + "down"] = mat(F, E, 1.5), mat(F, E, 1.5), mat(E, F)
    w["final.norm"] = around_zero(E)
    w["head"] = mat(cfg["vocab"], E, 3.0)
    return {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@functools.lru_cache(maxsize=None)
def weights(name, seed=0):
    cfg, ranks = CONFIGS[name]
    return make_weights(cfg, ranks, seed)


def as_plain(w):
    """The weights as the plain implementation takes them (float64)."""
    return {k: v.double() for k, v in w.items()}


def build(cfg, w, dtype):
    from gguf_rs_cli_b200.api import _build
    from gguf_rs_cli_b200.weights import TensorSource
    return _build(copy.deepcopy(cfg), TensorSource(tensors={k: v.to(torch.bfloat16) for k, v in w.items()}, where="test weights"),
                  dtype, "cuda:0")


@functools.lru_cache(maxsize=None)
def llm(name, dtype, seed=0):
    return build(CONFIGS[name][0], weights(name, seed), dtype)


def new_engine(name, dtype, n_tokens=2048, n_slots=8, **kw):
    from gguf_rs_cli_b200.engine.step import Engine
    return Engine(llm(name, dtype).model, n_tokens=n_tokens, n_slots=n_slots, **kw)


def tokens_of(name, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, CONFIGS[name][0]["vocab"], (n,), generator=g).tolist()


@functools.lru_cache(maxsize=None)
def plain_logits(name, n, seed):
    return P.forward(CONFIGS[name][0], as_plain(weights(name)), tokens_of(name, n, seed)).float()
