"""Fomodra on the host: configuration and refusals, tensor names, the cache that layers with windows of their own
share, and the plain implementation against closed forms and against itself with a mechanism left out."""
import copy
import math

import pytest
import torch

from gguf_rs_cli_b200.config import ConfigError, load_config
from gguf_rs_cli_b200.models.decoder import Decoder, tensor_requests
from tests import plain_fomodra as P
from tests.fomodra_util import CONFIGS, all_chosen, as_plain, config, make_weights, tokens_of, weights


def spec_of(cfg):
    arch, typed = load_config(copy.deepcopy(cfg))
    return arch.build_spec(typed)


@pytest.mark.parametrize("name", ["small", "wide"])
def test_tensor_names_and_shapes_are_those_of_the_weights(name):
    spec = spec_of(CONFIGS[name])
    asked = {r.name: tuple(r.shape) for r in tensor_requests(spec)}
    have = {k: tuple(v.shape) for k, v in weights(name).items()}
    assert asked == have


def test_registry_picks_the_design_by_its_name():
    arch, typed = load_config(config("small"))
    assert arch.name == "Fomodra" and typed.side_dim == 5 and typed.bigram["buckets"] == 101
    spec = arch.build_spec(typed)
    assert [l.block for l in spec.layers] == ["sandwich"] * 5
    assert [l.mixer.kind for l in spec.layers] == ["attention", "pair", "latent_attention", "attention", "attention"]
    assert [r.cache_of for r in spec.schedule] == [None, None, None, 0, None]
    assert spec.layers[2].feed_forward is None and spec.layers[0].feed_forward.params["identity"] == 2
    assert spec.layers[1].mixer.params["left"].params["chunk"] == 11 and spec.layers[1].mixer.params["left"].params["window"] is None


def test_absent_keys_mean_absent_mechanisms():
    cfg = config("small")
    del cfg["token_side"], cfg["embedding"]
    for layer in cfg["layers"]:
        if layer.get("mlp"):
            layer["mlp"].pop("shared", None)
            layer["mlp"]["router"].pop("identity", None)
    spec = spec_of(cfg)
    assert spec.embedding.kind == "embedding" and all(not l.extras and "side" not in l.norms for l in spec.layers)
    assert all(l.feed_forward is None or (l.feed_forward.params["shared_ff"] is None and l.feed_forward.params["identity"] == 0)
               for l in spec.layers)
    names = {r.name for r in tensor_requests(spec)}
    assert "bigram" not in names and "side.embed" not in names and not any(".shared." in n for n in names)


def test_layers_that_share_keys_keep_the_widest_window():
    cfg = config("small")
    spec = spec_of(cfg)
    model = Decoder(spec, torch.float32, "meta")
    layout = model.cache_layout()
    assert layout.kv[0].window == 29 and 3 not in layout.kv          # layer 0 sees 13 positions, its reader 29
    assert model.layers[0].mixer.window == 13 and model.layers[3].mixer.window == 29
    cfg["layers"][3]["mixer"].pop("mask")                              # a reader without a window: all positions are kept
    assert Decoder(spec_of(cfg), torch.float32, "meta").cache_layout().kv[0].window is None
    assert layout.kv[1].window == 11 and layout.kv[2].window == 17 and layout.kv[4].window is None
    assert set(layout.states) == {"embed.prev", "run1.right.S", "run1.right.conv"}
    assert layout.states["run1.right.S"][0] == (40, 20)


@pytest.mark.parametrize("change,text", [
    (lambda c: c["layers"][0].update(type="conv"), "type"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=3), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(kv_from=1), "kv_from"),
    (lambda c: c["layers"][3]["mixer"].update(dim=32), "kv_from"),
    (lambda c: c["layers"][0]["mixer"].update(heads=5), "kv_heads"),
    (lambda c: c["layers"][0]["mixer"]["rot"].update(dims=26), "dims"),
    (lambda c: c["layers"][0]["mlp"].update(kind="dense"), "kind"),
    (lambda c: c["layers"][0]["mlp"]["router"].update(top=9), "top"),
    (lambda c: c["layers"][1]["mixer"].pop("right"), "right"),
    (lambda c: c["layers"][2]["mixer"].pop("kv_rank"), "kv_rank"),
    (lambda c: c.pop("norm"), "eps"),
])
def test_refusals_name_the_key(change, text):
    cfg = config("small")
    change(cfg)
    with pytest.raises(ConfigError, match=text):
        load_config(cfg)


# ------------------------------------------------------------ the plain implementation
def test_masks():
    w = P.visible(9, {"size": 3}, "window")
    c = P.visible(9, {"size": 3}, "chunk")
    assert w[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert c[5].tolist() == [False, False, False, True, True, True, False, False, False]
    assert w[6].tolist() == [False] * 4 + [True] * 3 + [False] * 2 and c[6].tolist() == [False] * 6 + [True] + [False] * 2
    assert P.visible(4, None, "window").tolist() == torch.ones(4, 4).tril().bool().tolist()


def test_rotation_and_frequency_scaling():
    rot = {"base": 100.0, "dims": 4}
    x = torch.arange(12, dtype=P.F64).view(1, 2, 6)
    y = P.rotate(x, torch.tensor([3]), rot)
    f = [1.0, 100.0 ** -0.5]
    for h in range(2):
        for i in range(2):
            u, v, a = float(x[0, h, i]), float(x[0, h, i + 2]), 3 * f[i]
            assert abs(float(y[0, h, i]) - (u * math.cos(a) - v * math.sin(a))) < 1e-12
            assert abs(float(y[0, h, i + 2]) - (v * math.cos(a) + u * math.sin(a))) < 1e-12
        assert y[0, h, 4:].tolist() == x[0, h, 4:].tolist()
    sc = {"base": 10000.0, "dims": 16, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    plain = P.rotary_frequencies({"base": 10000.0, "dims": 16})
    scaled = P.rotary_frequencies(sc)
    assert scaled[0] == plain[0] and abs(float(scaled[-1]) - float(plain[-1]) / 4.0) < 1e-15
    assert any(float(p) / 4 < float(s) < float(p) for p, s in zip(plain, scaled))        # the stretch between the two rules


def test_sink_takes_its_share_and_identity_experts_return_the_row():
    q, k, v = torch.zeros(1, 1, 4, dtype=P.F64), torch.zeros(1, 1, 4, dtype=P.F64), torch.ones(1, 1, 2, dtype=P.F64)
    seen = torch.ones(1, 1, dtype=torch.bool)
    out = P.softmax_attention(q, k, v, 1.0, seen, torch.tensor([0.0], dtype=P.F64))
    assert torch.allclose(out, torch.full((1, 1, 2), 0.5, dtype=P.F64))
    big = P.softmax_attention(q, k, v, 1.0, seen, torch.tensor([50.0], dtype=P.F64))
    assert float(big.abs().max()) < 1e-20
    mlp = {"router": {"experts": 0, "identity": 2, "top": 2}, "expert": {"ff": 4, "limit": 1.0}}
    W = {"m.router": torch.randn(2, 6, dtype=P.F64), "m.correction": torch.zeros(2, dtype=P.F64)}
    h = torch.randn(3, 6, dtype=P.F64)
    assert torch.allclose(P.moe(mlp, W, "m.", h), h)


def test_correction_moves_the_choice_and_not_the_weights():
    mlp = {"router": {"experts": 3, "identity": 0, "top": 1}, "expert": {"ff": 4, "limit": 1.0}}
    h = torch.tensor([[1.0, 0.0]], dtype=P.F64)
    W = {"m.router": torch.tensor([[2.0, 0.0], [1.0, 0.0], [0.0, 0.0]], dtype=P.F64), "m.correction": torch.tensor([0.0, 0.9, 0.0], dtype=P.F64)}
    ids, wt = P.route(mlp, W, "m.", h)
    assert ids.tolist() == [[1]] and abs(float(wt[0, 0]) - 1.0) < 1e-12
    mlp["router"]["top"] = 2
    ids, wt = P.route(mlp, W, "m.", h)
    s = torch.softmax(torch.tensor([2.0, 1.0, 0.0], dtype=P.F64), 0)
    assert ids.tolist() == [[1, 0]] and abs(float(wt[0, 0]) - float(s[1] / (s[0] + s[1]))) < 1e-12


def test_selective_scan_against_its_closed_form_for_constant_inputs():
    """With constant x, dt, B and C the state is a geometric sum."""
    m = {"inner": 2, "state": 3, "dt_rank": 1, "conv": 1}
    E, T = 2, 6
    W = {"p.in": torch.cat([torch.eye(2), torch.zeros(2, 2)]).double(), "p.conv": torch.ones(2, 1, dtype=P.F64), "p.conv.b": torch.zeros(2, dtype=P.F64),
         "p.x": torch.zeros(7, 2, dtype=P.F64), "p.dt": torch.zeros(2, 1, dtype=P.F64), "p.dt.b": torch.tensor([0.3, -0.5], dtype=P.F64),
         "p.A_log": torch.tensor([[0.0, 0.5, -1.0], [0.2, 0.1, 0.0]], dtype=P.F64), "p.D": torch.zeros(2, dtype=P.F64), "p.o": torch.eye(2, dtype=P.F64)}
    W["p.x"][1:4, 0] = torch.tensor([1.0, 2.0, -1.0], dtype=P.F64)         # B = x_0 * these
    W["p.x"][4:7, 1] = torch.tensor([0.5, 1.0, 2.0], dtype=P.F64)          # C = x_1 * these
    h = torch.tensor([[1.5, -0.7]], dtype=P.F64).repeat(T, 1)
    # z = 0 makes the gate silu(0) = 0: move the gate's rows to give z = x instead
    W["p.in"][2:] = torch.eye(2, dtype=P.F64)
    got = P.selective_scan_mixer(m, W, "p.", h)
    x = P.silu(h[0])
    dt = P.softplus(W["p.dt.b"])
    A = -torch.exp(W["p.A_log"])
    B, C = x[0] * torch.tensor([1.0, 2.0, -1.0], dtype=P.F64), x[1] * torch.tensor([0.5, 1.0, 2.0], dtype=P.F64)
    for t in range(T):
        a = torch.exp(dt[:, None] * A)
        S = (dt * x)[:, None] * B[None, :] * (1 - a ** (t + 1)) / (1 - a)
        y = (S @ C) * P.silu(h[0])
        assert torch.allclose(got[t], y, atol=1e-12)


@pytest.mark.parametrize("name", ["small"])
def test_every_mechanism_moves_the_logits(name):
    cfg, w = config(name), as_plain(weights(name))
    toks = tokens_of(name, 60, 3)
    base = P.forward(cfg, w, toks)
    top = float(base.abs().max())

    def moved(c2=None, w2=None, rows=slice(None)):
        return float((P.forward(c2 or cfg, w2 or w, toks) - base)[rows].abs().max()) / top

    c = copy.deepcopy(cfg); c["layers"][0]["mixer"]["mask"]["size"] += 1
    assert moved(c) > 0.02, "window of attention"
    c = copy.deepcopy(cfg); c["layers"][1]["mixer"]["left"]["mask"]["size"] += 1
    assert moved(c) > 0.02, "chunk of the left mixer"
    c = copy.deepcopy(cfg); c["layers"][2]["mixer"]["mask"]["size"] -= 1
    assert moved(c) > 0.01, "window of latent attention"
    c = copy.deepcopy(cfg); c["layers"][3]["mixer"]["mask"]["size"] = 13
    assert moved(c) > 0.01, "own window of the layer that reads another's keys"
    c = copy.deepcopy(cfg); del c["layers"][1]["mixer"]["left"]["rot"]["scaling"]
    assert moved(c) > 0.01, "frequency scaling"
    c = copy.deepcopy(cfg); c["layers"][0]["mixer"]["rot"]["dims"] = 8
    assert moved(c) > 0.02, "rotated entries"
    c = copy.deepcopy(cfg); del c["token_side"]
    assert moved(c) > 0.05, "token side input"
    c = copy.deepcopy(cfg); del c["embedding"]
    assert moved(c, rows=slice(1, None)) > 0.05, "pair embedding"
    for key, what in (("l0.mix.sink", "sink"), ("l2.mix.sink", "latent sink"), ("l0.mlp.correction", "correction"), ("l0.mix.q.b", "bias"),
                      ("l1.mix.right.D", "skip"), ("l2.mix.g", "gate")):
        w2 = dict(w); w2[key] = w[key] + 3.0 * torch.linspace(-1.0, 1.0, w[key].numel(), dtype=P.F64).view(w[key].shape)
        assert moved(w2=w2) > 0.005, what
    w2 = dict(w); w2["l1.mix.right.A_log"] = w["l1.mix.right.A_log"] + 1.0
    assert moved(w2=w2) > 0.005, "decay of the scan"
    c = copy.deepcopy(cfg); c["layers"][0]["mlp"]["router"]["identity"] = 0
    w2 = dict(w); w2["l0.mlp.router"], w2["l0.mlp.correction"] = w["l0.mlp.router"][:5], w["l0.mlp.correction"][:5]
    assert moved(c, w2) > 0.01, "identity experts"
    assert float((P.forward(all_chosen(cfg), w, toks) - base).abs().max()) / top > 0.01, "the router's choice"
