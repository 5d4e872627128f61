"""Typed configuration of the Nazerax design and its description as parts.

A Nazerax model is a list of layers in which mixer and feed-forward read two norms of the same x,
x <- x + mixer(norm1(x)) + ff(norm2(x)); the norms are RMS norms whose weights are stored around zero.  A layer's
mixer is `wkv` (time mixing in the manner of RWKV: a matrix per head that decays per key channel, with a token shift in
front of every projection), `mamba2` (a selective state-space mixer in its duality form) or `attention` (grouped-query
attention with a short convolution on q, k and v, a rotation of the heads' first entries in neighbouring pairs, a
window, a softmax that may attend to nothing, and one sigmoid gate per head); its feed-forward is a gated SiLU unit or
absent.  The embedding adds a row that the pair (previous token, token) chooses by a hash; a stretch of layers may run
several times in a row with the same weights, every pass with state of its own and, from the second on, with the
embedding's result added again; the logits are bounded by a tanh.  config.json gives every size and every constant;
the rank of the decay's low-rank pair is the tensors' own size.  The reference knows one architecture only
(src/model/config.rs:20-47) and has none of these parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .debonex import NO_POSITION_LIMIT, _get
from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, Run

MIXER_TYPES = ("wkv", "mamba2", "attention")


@dataclass(frozen=True)
class NazeraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]            # None: the layer has no feed-forward


@dataclass(frozen=True)
class NazeraxConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[NazeraxLayer] = field(default_factory=list)
    bigram: Optional[Dict[str, int]] = None      # buckets, mul_prev, mul_cur; None: no such table
    loop: Optional[Dict[str, int]] = None        # start, stop, times; None: every layer runs once
    logit_softcap: Optional[float] = None

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NazeraxConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {list(MIXER_TYPES)}")
            out.append(NazeraxLayer(kind, _read_mixer(kind, entry.get("mixer"), where + ".mixer"),
                                    _read_mlp(entry.get("mlp"), where + ".mlp")))
        bigram = None
        big = (raw.get("embedding") or {}).get("bigram") if isinstance(raw.get("embedding"), dict) else None
        if big is not None:
            bigram = {"buckets": _get(big, "buckets", "embedding.bigram"),
                      "mul_prev": _get(big, "mul_prev", "embedding.bigram", positive=False),
                      "mul_cur": _get(big, "mul_cur", "embedding.bigram", positive=False)}
        loop = None
        if raw.get("loop") is not None:
            lp = raw["loop"]
            loop = {"start": _get(lp, "start", "'loop'", positive=False), "stop": _get(lp, "stop", "'loop'"),
                    "times": _get(lp, "times", "'loop'")}
            if not 0 <= loop["start"] < loop["stop"] <= len(out):
                raise ConfigError(f"config.json: 'loop' runs layers {loop['start']} .. {loop['stop'] - 1}, the model has {len(out)}")
        cap = raw.get("logit_softcap")
        return cls(vocab=_get(raw, "vocab", "the top level"), width=_get(raw, "width", "the top level"),
                   norm_eps=_get(raw.get("norm"), "eps", "'norm'", float), layers=out, bigram=bigram, loop=loop,
                   logit_softcap=None if cap is None else _get(raw, "logit_softcap", "the top level", float))


def _read_mixer(kind: str, raw, where: str) -> Dict[str, Any]:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    if kind == "wkv":
        return {k: _get(raw, k, where) for k in ("heads", "dim")}
    if kind == "mamba2":
        m = {k: _get(raw, k, where) for k in ("heads", "vdim", "state", "conv")}
        m["groups"] = _get(raw, "groups", where) if raw.get("groups") is not None else 1
        m["norm_groups"] = _get(raw, "norm_groups", where) if raw.get("norm_groups") is not None else 1
        if m["heads"] % m["groups"]:
            raise ConfigError(f"config.json: {where}: heads {m['heads']} is not a multiple of groups {m['groups']}")
        if (m["heads"] * m["vdim"]) % m["norm_groups"]:
            raise ConfigError(f"config.json: {where}: heads * vdim = {m['heads'] * m['vdim']} does not form {m['norm_groups']} "
                              f"equal parts (norm_groups)")
        return m
    m = {k: _get(raw, k, where) for k in ("heads", "dim")}
    m["vdim"] = _get(raw, "vdim", where) if raw.get("vdim") is not None else m["dim"]
    m["kv_heads"] = _get(raw, "kv_heads", where) if raw.get("kv_heads") is not None else m["heads"]
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    m["scale"] = _get(raw, "scale", where, float) if raw.get("scale") is not None else m["dim"] ** -0.5
    m["conv"] = _get(raw, "conv", where) if raw.get("conv") is not None else 1
    m["mask"] = m["rot"] = None
    if raw.get("mask") is not None:
        m["mask"] = {"size": _get(raw["mask"], "size", where + ".mask")}
    if raw.get("rot") is not None and raw["rot"].get("dims") != 0:          # no entries to rotate: no rotation
        m["rot"] = {"base": _get(raw["rot"], "base", where + ".rot", float), "dims": _get(raw["rot"], "dims", where + ".rot")}
        if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["dim"]:
            raise ConfigError(f"config.json: {where}.rot.dims {m['rot']['dims']} must be even and at most dim {m['dim']}")
    return m


def _read_mlp(raw, where: str) -> Optional[Dict[str, Any]]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, dict) else raw
    if kind != "dense":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (dense)")
    return {"kind": "dense", "ff": _get(raw, "ff", where)}


def run_order(cfg: NazeraxConfig) -> List[Run]:
    """Every layer once, the looped stretch `times` times in a row; the first run of every pass but the first adds the
    embedding's result to the stream again.  A run is a schedule entry of its own, so each pass has its own cache and state."""
    n = len(cfg.layers)
    if cfg.loop is None:
        return [Run(i) for i in range(n)]
    a, b, times = cfg.loop["start"], cfg.loop["stop"], cfg.loop["times"]
    order = [Run(i) for i in range(a)]
    for rep in range(times):
        order += [Run(i, add_input=rep > 0 and i == a) for i in range(a, b)]
    return order + [Run(i) for i in range(b, n)]


def build_nazerax_spec(cfg: NazeraxConfig) -> ModelSpec:
    E, layers = cfg.width, []

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(size=E, eps=cfg.norm_eps, offset=1.0), {"weight": name})

    for i, layer in enumerate(cfg.layers):
        p, m, position = f"l{i}.mix.", layer.mixer, None
        if layer.type == "wkv":
            mixer = PartSpec("wkv", dict(hidden_size=E, heads=m["heads"], dim=m["dim"], eps=cfg.norm_eps),
                             {"mu_" + s: p + "mu." + s for s in "rkvgw"} |
                             {n: p + n for n in ("r", "k", "v", "g", "w1", "w2", "w0", "u", "norm", "o")})
        elif layer.type == "mamba2":
            mixer = PartSpec("ssd", dict(hidden_size=E, heads=m["heads"], vdim=m["vdim"], state=m["state"], groups=m["groups"],
                                         conv=m["conv"], norm_groups=m["norm_groups"], eps=cfg.norm_eps),
                             {"in": p + "in", "conv": p + "conv", "conv_bias": p + "conv.b", "dt_bias": p + "dt_bias",
                              "A_log": p + "A_log", "D": p + "D", "norm": p + "norm", "o": p + "o"})
        else:
            if m["rot"] is not None:
                position = PartSpec("rope", dict(head_dim=m["dim"], rotary_dim=m["rot"]["dims"], theta=m["rot"]["base"],
                                                 pairing="interleaved", scaling=None))
            mixer = PartSpec("attention", dict(hidden_size=E, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                               v_head_dim=m["vdim"], scale=m["scale"], window=(m["mask"] or {}).get("size"),
                                               bias=False, out_gate="head", sink=True, conv=m["conv"]),
                             {"q": p + "q", "k": p + "k", "v": p + "v", "o": p + "o", "g": p + "g", "q_conv": p + "q.conv",
                              "k_conv": p + "k.conv", "v_conv": p + "v.conv"})
        norms, ff = {"mixer": norm(f"l{i}.norm1")}, None
        if layer.mlp is not None:
            q = f"l{i}.mlp."
            norms["feed_forward"] = norm(f"l{i}.norm2")
            ff = PartSpec("gated_mlp", dict(hidden_size=E, intermediate_size=layer.mlp["ff"], activation="silu", term_f32=True),
                          {"gate": q + "gate", "up": q + "up", "down": q + "down"})
        layers.append(LayerSpec(block="parallel", mixer=mixer, feed_forward=ff, norms=norms, position=position))
    if cfg.bigram is not None:
        embedding = PartSpec("embedding_bigram", dict(vocab_size=cfg.vocab, hidden_size=E, **cfg.bigram),
                             {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("embedding", dict(vocab_size=cfg.vocab, hidden_size=E), {"weight": "embed"})
    spec = ModelSpec(
        architecture="Nazerax", vocab_size=cfg.vocab, hidden_size=E, embedding=embedding, layers=layers,
        schedule=run_order(cfg), final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=E, tied_to=None, tied=False, softcap=cfg.logit_softcap),
                      {"weight": "head"}),
        max_position=NO_POSITION_LIMIT)
    spec.validate()
    return spec


register_architecture("Nazerax", NazeraxConfig, build_nazerax_spec, "nazerax")
