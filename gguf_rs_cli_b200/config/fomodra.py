"""Typed configuration of the Fomodra design and its description as parts.

A Fomodra model is a list of layers that norm what a sublayer reads and what it gives:
x <- x + norm1b(mixer(norm1(x))), x <- x + norm2b(ff(norm2(x))), all RMS norms with plain weights; behind the
feed-forward every layer may add an input of its own that depends on the token alone (a slice of a per-token table gates
a low-rank view of x, is projected back and normed in).  A layer's mixer is `attention` (grouped-query attention with
q/k/v biases, a rotation of the heads' first entries in halves, a sliding window, a learned sink per head in the
softmax's denominator; a layer may read an earlier layer's keys and values instead of making its own),
`latent_attention` (keys and values of all heads from one cached latent row per position plus one shared rotated key
part; window, learned sink, one sigmoid gate per head) or `parallel` (chunked attention and a selective scan side by
side, each normed over the width, half their sum).  The feed-forward is a mixture of experts with a softmax router, a
correction that only the choice sees, identity experts and a shared expert.  The embedding adds a row that the pair
(previous token, token) chooses by a hash.  config.json gives every size and every constant.  The reference knows one
architecture only (src/model/config.rs:20-47) and has none of these parts.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional

from .debonex import NO_POSITION_LIMIT, _get
from .registry import ConfigError, register_architecture
from .specs import LayerSpec, ModelSpec, PartSpec, Run

MIXER_TYPES = ("attention", "latent_attention", "parallel")


@dataclass(frozen=True)
class FomodraLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]            # None: the layer has no feed-forward


@dataclass(frozen=True)
class FomodraConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[FomodraLayer] = field(default_factory=list)
    bigram: Optional[Dict[str, int]] = None      # buckets, mul_prev, mul_cur; None: no such table
    side_dim: Optional[int] = None               # columns of the per-token table that each layer owns; None: no such input

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "FomodraConfig":
        layers = raw.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        out = []
        for i, entry in enumerate(layers):
            where = f"layers[{i}]"
            kind = entry.get("type") if isinstance(entry, dict) else None
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not one of {list(MIXER_TYPES)}")
            out.append(FomodraLayer(kind, _read_mixer(kind, entry.get("mixer"), where + ".mixer"),
                                    _read_mlp(entry.get("mlp"), where + ".mlp")))
        for i, layer in enumerate(out):
            src = layer.mixer.get("kv_from") if layer.type == "attention" else None
            if src is None:
                continue
            where = f"layers[{i}].mixer.kv_from"
            if not 0 <= src < i or out[src].type != "attention" or out[src].mixer.get("kv_from") is not None:
                raise ConfigError(f"config.json: {where} = {src} must name an earlier attention layer with keys and values of its own")
            a, b = layer.mixer, out[src].mixer
            if any(a[k] != b[k] for k in ("kv_heads", "dim", "vdim", "rot")):
                raise ConfigError(f"config.json: {where}: layer {src} has other key/value heads, sizes or rotation than layer {i}")
        bigram = None
        big = (raw.get("embedding") or {}).get("bigram") if isinstance(raw.get("embedding"), dict) else None
        if big is not None:
            bigram = {"buckets": _get(big, "buckets", "embedding.bigram"),
                      "mul_prev": _get(big, "mul_prev", "embedding.bigram", positive=False),
                      "mul_cur": _get(big, "mul_cur", "embedding.bigram", positive=False)}
        side = raw.get("token_side")
        return cls(vocab=_get(raw, "vocab", "the top level"), width=_get(raw, "width", "the top level"),
                   norm_eps=_get(raw.get("norm"), "eps", "'norm'", float), layers=out, bigram=bigram,
                   side_dim=None if side is None else _get(side, "dim", "'token_side'"))


def _read_rot(raw, where: str, limit: int) -> Optional[Dict[str, Any]]:
    if raw is None or raw.get("dims") == 0:          # no entries to rotate: no rotation
        return None
    rot = {"base": _get(raw, "base", where, float), "dims": _get(raw, "dims", where), "scaling": None}
    if rot["dims"] % 2 or rot["dims"] > limit:
        raise ConfigError(f"config.json: {where}.dims {rot['dims']} must be even and at most {limit}")
    sc = raw.get("scaling")
    if sc is not None:
        rot["scaling"] = {"factor": _get(sc, "factor", where + ".scaling", float), "low": _get(sc, "low", where + ".scaling", float),
                          "high": _get(sc, "high", where + ".scaling", float),
                          "original": _get(sc, "original", where + ".scaling", float)}
    return rot


def _read_attention(raw, where: str) -> Dict[str, Any]:
    m = {k: _get(raw, k, where) for k in ("heads", "dim")}
    m["vdim"] = _get(raw, "vdim", where) if raw.get("vdim") is not None else m["dim"]
    m["kv_heads"] = _get(raw, "kv_heads", where) if raw.get("kv_heads") is not None else m["heads"]
    if m["heads"] % m["kv_heads"]:
        raise ConfigError(f"config.json: {where}: heads {m['heads']} is not a multiple of kv_heads {m['kv_heads']}")
    m["scale"] = _get(raw, "scale", where, float) if raw.get("scale") is not None else m["dim"] ** -0.5
    m["mask"] = None if raw.get("mask") is None else {"size": _get(raw["mask"], "size", where + ".mask")}
    m["rot"] = _read_rot(raw.get("rot"), where + ".rot", m["dim"])
    m["kv_from"] = None if raw.get("kv_from") is None else _get(raw, "kv_from", where, positive=False)
    return m


def _read_mixer(kind: str, raw, where: str) -> Dict[str, Any]:
    if not isinstance(raw, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    if kind == "attention":
        return _read_attention(raw, where)
    if kind == "latent_attention":
        m = {k: _get(raw, k, where) for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank")}
        m["scale"] = _get(raw, "scale", where, float) if raw.get("scale") is not None else (m["dim"] + m["rot_dim"]) ** -0.5
        m["mask"] = None if raw.get("mask") is None else {"size": _get(raw["mask"], "size", where + ".mask")}
        m["rot"] = _read_rot(raw.get("rot"), where + ".rot", m["rot_dim"])
        if m["rot_dim"] % 2:
            raise ConfigError(f"config.json: {where}.rot_dim {m['rot_dim']} must be even")
        return m
    if not isinstance(raw.get("left"), dict) or not isinstance(raw.get("right"), dict):
        raise ConfigError(f"config.json: {where} must hold the objects 'left' and 'right'")
    left = _read_attention(raw["left"], where + ".left")
    if left["kv_from"] is not None:
        raise ConfigError(f"config.json: {where}.left cannot read another layer's keys and values")
    right = {k: _get(raw["right"], k, where + ".right") for k in ("inner", "state", "dt_rank", "conv")}
    return {"left": left, "right": right}


def _read_mlp(raw, where: str) -> Optional[Dict[str, Any]]:
    if raw is None:
        return None
    kind = raw.get("kind") if isinstance(raw, dict) else raw
    if kind != "moe":
        raise ConfigError(f"config.json: {where}.kind {kind!r} is not supported (moe)")
    router, expert = raw.get("router"), raw.get("expert")
    m = {"kind": "moe", "experts": _get(router, "experts", where + ".router"), "top": _get(router, "top", where + ".router"),
         "identity": _get(router, "identity", where + ".router", positive=False) if (router or {}).get("identity") is not None else 0,
         "ff": _get(expert, "ff", where + ".expert"), "limit": _get(expert, "limit", where + ".expert", float), "shared": None}
    if m["top"] > m["experts"] + m["identity"]:
        raise ConfigError(f"config.json: {where}.router: top {m['top']} of {m['experts']} + {m['identity']} experts")
    if raw.get("shared") is not None:
        m["shared"] = {"ff": _get(raw["shared"], "ff", where + ".shared"), "limit": _get(raw["shared"], "limit", where + ".shared", float)}
    return m


def _rope(m, head_dim: int) -> Optional[PartSpec]:
    rot = m["rot"]
    if rot is None:
        return None
    sc = rot["scaling"]
    scaling = None if sc is None else {"rope_type": "llama3", "factor": sc["factor"], "low_freq_factor": sc["low"],
                                       "high_freq_factor": sc["high"], "original_max_position_embeddings": sc["original"]}
    return PartSpec("rope", dict(head_dim=head_dim, rotary_dim=rot["dims"], theta=rot["base"], pairing="half", scaling=scaling))


def _cache_spans(cfg: "FomodraConfig") -> Dict[int, Optional[int]]:
    """For every attention layer, how many of the last positions its cache must keep (None: all): the widest window among
    the layer that owns the keys and the layers that read them."""
    owner = {i: (l.mixer["kv_from"] if l.mixer["kv_from"] is not None else i) for i, l in enumerate(cfg.layers) if l.type == "attention"}
    spans: Dict[int, Optional[int]] = {}
    for i, o in owner.items():
        size = (cfg.layers[i].mixer["mask"] or {}).get("size")
        if o not in spans:
            spans[o] = size
        elif spans[o] is not None:
            spans[o] = None if size is None else max(spans[o], size)
    return {i: spans[o] for i, o in owner.items()}


def _attention(E: int, m, p: str, chunked: bool, bias: bool, sink: bool, cache_span="own") -> PartSpec:
    size = (m["mask"] or {}).get("size")
    more = {} if cache_span == "own" else {"cache_span": cache_span}
    shares = m["kv_from"] is not None
    names = ["q", "o"] + ([] if shares else ["k", "v"])
    tensors = {n: p + n for n in names}
    if bias:
        tensors.update({n + "_bias": p + n + ".b" for n in names if n != "o"})
    if sink:
        tensors["sink"] = p + "sink"
    return PartSpec("attention", dict(hidden_size=E, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                                      v_head_dim=m["vdim"], scale=m["scale"], window=None if chunked else size,
                                      chunk=size if chunked else None, bias=bias, sink="learned" if sink else False,
                                      shares_kv=shares, exact=True, **more), tensors)


def build_fomodra_spec(cfg: FomodraConfig) -> ModelSpec:
    E, layers, schedule = cfg.width, [], []
    spans = _cache_spans(cfg)

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(size=E, eps=cfg.norm_eps), {"weight": name})

    for i, layer in enumerate(cfg.layers):
        p, m, position = f"l{i}.mix.", layer.mixer, None
        if layer.type == "attention":
            position = _rope(m, m["dim"])
            mixer = _attention(E, m, p, chunked=False, bias=True, sink=True, cache_span=spans[i])
        elif layer.type == "latent_attention":
            position = _rope(m, m["rot_dim"])
            mixer = PartSpec("latent_attention", dict(hidden_size=E, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"],
                                                      vdim=m["vdim"], kv_rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps,
                                                      window=(m["mask"] or {}).get("size"), sink="learned", out_gate="head"),
                             {"q": p + "q", "dkv": p + "dkv", "dkv_norm": p + "dkv.norm", "uk": p + "uk", "uv": p + "uv",
                              "o": p + "o", "sink": p + "sink", "g": p + "g"})
        else:
            left, right = m["left"], m["right"]
            position = _rope(left, left["dim"])
            q = p + "right."
            scan = PartSpec("selective_scan", dict(hidden_size=E, inner=right["inner"], state=right["state"], dt_rank=right["dt_rank"],
                                                   conv=right["conv"]),
                            {"in": q + "in", "conv": q + "conv", "conv_bias": q + "conv.b", "x": q + "x", "dt": q + "dt",
                             "dt_bias": q + "dt.b", "A_log": q + "A_log", "D": q + "D", "o": q + "o"})
            mixer = PartSpec("pair", dict(hidden_size=E, eps=cfg.norm_eps, mix=0.5,
                                          left=_attention(E, left, p + "left.", chunked=True, bias=False, sink=False), right=scan),
                             {"left_out": p + "left.out", "right_out": p + "right.out"})
        norms = {"mixer": norm(f"l{i}.norm1"), "mixer_out": norm(f"l{i}.norm1b")}
        ff = None
        if layer.mlp is not None:
            mlp, q = layer.mlp, f"l{i}.mlp."
            norms["feed_forward"], norms["feed_forward_out"] = norm(f"l{i}.norm2"), norm(f"l{i}.norm2b")
            shared = mlp["shared"]
            ff = PartSpec("moe", dict(hidden_size=E, experts=mlp["experts"], top=mlp["top"], groups=1, keep=1, scale=1.0,
                                      expert_ff=mlp["ff"], limit=mlp["limit"], shared_ff=None if shared is None else shared["ff"],
                                      shared_limit=None if shared is None else shared["limit"], score="softmax", correction=True,
                                      identity=mlp["identity"]),
                          {"router": q + "router", "experts": q + "e", "shared": q + "shared", "correction": q + "correction"})
        extras = {}
        if cfg.side_dim is not None:
            norms["side"] = norm(f"l{i}.side.norm")
            extras["side"] = PartSpec("token_side", dict(hidden_size=E, vocab_size=cfg.vocab, dim=cfg.side_dim,
                                                         columns=cfg.side_dim * len(cfg.layers), offset=i * cfg.side_dim,
                                                         activation="gelu_tanh"),
                                      {"table": "side.embed", "gate": f"l{i}.side.gate", "proj": f"l{i}.side.proj"})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, feed_forward=ff, norms=norms, position=position, extras=extras))
        schedule.append(Run(i, cache_of=m.get("kv_from") if layer.type == "attention" else None))
    if cfg.bigram is not None:
        embedding = PartSpec("embedding_bigram", dict(vocab_size=cfg.vocab, hidden_size=E, **cfg.bigram),
                             {"weight": "embed", "pairs": "bigram"})
    else:
        embedding = PartSpec("embedding", dict(vocab_size=cfg.vocab, hidden_size=E), {"weight": "embed"})
    spec = ModelSpec(
        architecture="Fomodra", vocab_size=cfg.vocab, hidden_size=E, embedding=embedding, layers=layers, schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", dict(vocab_size=cfg.vocab, hidden_size=E, tied_to=None, tied=False), {"weight": "head"}),
        max_position=NO_POSITION_LIMIT)
    spec.validate()
    return spec


register_architecture("Fomodra", FomodraConfig, build_fomodra_spec, "fomodra")
