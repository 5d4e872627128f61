"""Nazerax without a device: the configuration reader and what it refuses, the model as parts and tensor names, the run
order of a looped stretch with its states, and the plain implementation against closed forms and against itself."""
import copy
import math

import pytest
import torch

from tests import plain_nazerax as P
from tests.nazerax_util import CONFIGS, as_plain, config, make_weights, tokens_of, weights


def test_config_reads_every_size_and_constant():
    from gguf_rs_cli_b200.config import load_config
    arch, cfg = load_config(config("small"))
    assert arch.name == "Nazerax" and (cfg.vocab, cfg.width, cfg.norm_eps, cfg.logit_softcap) == (197, 72, 1e-5, 9.0)
    assert cfg.bigram == {"buckets": 101, "mul_prev": 13, "mul_cur": 5} and cfg.loop == {"start": 1, "stop": 4, "times": 3}
    assert [l.type for l in cfg.layers] == ["attention", "wkv", "mamba2", "attention", "wkv"]
    assert cfg.layers[1].mlp is None and cfg.layers[0].mlp == {"kind": "dense", "ff": 136}
    spec = arch.build_spec(cfg)
    assert all(l.block == "parallel" for l in spec.layers) and spec.embedding.kind == "embedding_bigram"
    assert spec.head.params["softcap"] == 9.0 and spec.final_norm.params["offset"] == 1.0
    a = spec.layers[0].mixer.params
    assert (a["window"], a["v_head_dim"], a["scale"], a["conv"], a["sink"], a["out_gate"], a["num_kv_heads"]) == (13, 40, 0.3, 4, True, "head", 3)
    assert spec.layers[0].position.params["pairing"] == "interleaved" and spec.layers[0].position.params["rotary_dim"] == 16
    b = spec.layers[3].mixer.params                  # what the configuration leaves out does not exist
    assert (b["window"], b["conv"], b["v_head_dim"]) == (None, 1, 8)
    assert spec.layers[1].mixer.kind == "wkv" and spec.layers[1].feed_forward is None and set(spec.layers[1].norms) == {"mixer"}
    s = spec.layers[2].mixer
    assert s.kind == "ssd" and (s.params["state"], s.params["groups"], s.params["norm_groups"], s.params["conv"]) == (20, 3, 2, 2)
    assert spec.layers[2].feed_forward.kind == "gated_mlp" and spec.layers[2].feed_forward.params["term_f32"]
    # the stretch 1..3 three times in a row, every pass but the first starting with the embedding's result
    assert [(r.layer, r.add_input) for r in spec.schedule] == \
        [(0, False), (1, False), (2, False), (3, False), (1, True), (2, False), (3, False), (1, True), (2, False), (3, False), (4, False)]


def test_config_defaults_and_refusals():
    from gguf_rs_cli_b200.config import ConfigError, load_config
    raw = config("wide")
    del raw["loop"], raw["embedding"], raw["logit_softcap"]
    arch, cfg = load_config(raw)
    spec = arch.build_spec(cfg)
    assert spec.embedding.kind == "embedding" and spec.head.params["softcap"] is None
    assert [r.layer for r in spec.schedule] == [0, 1, 2, 3, 4] and not any(r.add_input for r in spec.schedule)
    for path, value, text in [(("layers", 0, "type"), "conv", "type"), (("layers", 1, "mixer", "kv_heads"), 3, "kv_heads"),
                              (("layers", 1, "mixer", "rot", "dims"), 66, "rot.dims"), (("layers", 1, "mlp", "kind"), "moe", "kind"),
                              (("layers", 0, "mixer", "groups"), 3, "groups"), (("layers", 4, "mixer", "norm_groups"), 3, "norm_groups"),
                              (("loop", "stop"), 6, "loop"), (("loop", "start"), 2, "loop")]:
        bad = config("wide")
        node = bad
        for k in path[:-1]:
            node = node[k]
        node[path[-1]] = value
        with pytest.raises(ConfigError, match=text):
            arch, c = load_config(bad)
            arch.build_spec(c)
    bad = config("wide")
    del bad["layers"][0]["mixer"]["state"]
    with pytest.raises(ConfigError, match="state"):
        load_config(bad)


@pytest.mark.parametrize("name", sorted(CONFIGS))
def test_tensor_names_and_shapes(name):
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import tensor_requests
    arch, cfg = load_config(config(name))
    reqs = {r.name: r for r in tensor_requests(arch.build_spec(cfg))}
    w = weights(name)
    assert set(reqs) == set(w)
    for n, r in reqs.items():
        assert len(r.shape) == w[n].dim() and all(a in (-1, b) for a, b in zip(r.shape, w[n].shape)), (n, r.shape, tuple(w[n].shape))


def test_states_of_every_pass_are_its_own():
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import Decoder
    arch, cfg = load_config(config("small"))
    layout = Decoder(arch.build_spec(cfg), torch.float32, "meta").cache_layout()
    assert layout.states["embed.prev"] == ((), "int32")
    # layer 1 (wkv) runs as runs 1, 4 and 7, layer 2 (state-space) as 2, 5, 8; layer 3 keeps keys in runs 3, 6, 9
    for r in (1, 4, 7):
        assert layout.states[f"run{r}.S"] == ((3, 20, 20), "float32") and layout.states[f"run{r}.prev"] == ((72,), "float32")
    for r in (2, 5, 8):
        assert layout.states[f"run{r}.S"] == ((6, 20, 12), "float32") and layout.states[f"run{r}.conv"] == ((1, 72 + 2 * 3 * 20), "float32")
    assert sorted(layout.kv) == [0, 3, 6, 9] and layout.kv[0].window == 13 and layout.kv[3].window is None
    assert "run3.conv" not in layout.states and layout.states["run0.conv"][0][0] == 3


# ------------------------------------------------------------------------------------- the plain implementation
def test_pair_rows_and_first_token():
    assert P.bigram_rows([4, 9, 9], None, 101, 13, 5) == [101, (4 * 13 + 9 * 5) % 101, (9 * 13 + 9 * 5) % 101]
    assert P.bigram_rows([7], 3, 10, 9999991, 3) == [(3 * 9999991 + 21) % 10]


def test_short_convolution_against_torch():
    g = torch.Generator().manual_seed(0)
    u, taps, bias = torch.randn(9, 5, generator=g).double(), torch.randn(5, 3, generator=g).double(), torch.randn(5, generator=g).double()
    y, last = P.short_conv(u, taps, torch.zeros(2, 5, dtype=torch.float64), bias)
    ref = torch.nn.functional.conv1d(torch.nn.functional.pad(u.T[None], (2, 0)), taps[:, None, :], bias, groups=5)[0].T
    assert torch.allclose(y, ref, atol=1e-12) and torch.equal(last, u[-2:])
    # in two pieces, the second from what the first left
    y1, keep = P.short_conv(u[:4], taps, torch.zeros(2, 5, dtype=torch.float64), bias)
    y2, _ = P.short_conv(u[4:], taps, keep, bias)
    assert torch.allclose(torch.cat([y1, y2]), ref, atol=1e-12)


def test_sink_takes_its_share():
    """With all scores 0 over n keys each weight is 1 / (n + 1): the sink holds one share and gives nothing."""
    m = {"heads": 1, "dim": 4, "scale": 1.0}
    E = 4
    W = {"x.q": torch.zeros(4, E), "x.k": torch.zeros(4, E), "x.v": torch.eye(4), "x.g": torch.zeros(1, E), "x.o": torch.eye(4)}
    W = {k: v.double() for k, v in W.items()}
    h = torch.ones(3, E, dtype=torch.float64)
    out = P.attention_mixer(m, 1e-6, W, "x.", h, {})
    for t in range(3):
        assert torch.allclose(out[t], torch.full((4,), 0.5 * (t + 1) / (t + 2), dtype=torch.float64))


def test_wkv_bonus_and_decay_by_hand():
    """One head of one channel: S_t = w S_(t-1) + k v, o_t = r (S_(t-1) + u k v)."""
    m = {"heads": 1, "dim": 1}
    one = torch.ones(1, 1, dtype=torch.float64)
    W = {"x.mu." + s: torch.zeros(1, dtype=torch.float64) for s in "rkvgw"}
    W.update({"x.r": one * 2, "x.k": one * 3, "x.v": one * 5, "x.g": one, "x.w1": one * 0, "x.w2": one * 0,
              "x.w0": torch.tensor([math.log(math.log(2.0))], dtype=torch.float64), "x.u": one * 0.25, "x.norm": one[0], "x.o": one})
    h = torch.ones(3, 1, dtype=torch.float64)
    state = {}
    P.wkv_mixer(m, 1e-12, W, "x.", h, state)
    assert abs(float(state["S"]) - 15 * (1 + 0.5 + 0.25)) < 1e-9          # decay exp(-exp(w0)) = 1/2
    # what is read at the second token, before the norm: r (S_1 + u k v) = 2 (15 + 0.25 * 15)
    kv, S1 = 15.0, 15.0
    raw = 2 * (S1 + 0.25 * kv)
    assert raw == 37.5


def test_in_pieces_as_whole_and_every_mechanism_counts():
    cfg, w = config("small"), as_plain(weights("small"))
    toks = tokens_of("small", 40, 3)
    whole = P.forward(cfg, w, toks)
    st = P.Stepper(cfg, w)
    pieces = torch.cat([st.feed(toks[a:b]) for a, b in [(0, 1), (1, 3), (3, 20), (20, 21), (21, 40)]])
    assert torch.allclose(pieces, whole, atol=1e-9)
    top = float(whole.abs().max())

    def moved(other_cfg, other_w=None):
        return float((P.forward(other_cfg, other_w or w, toks) - whole).abs().max()) / top

    for change in [lambda c: c.pop("loop"), lambda c: c.pop("logit_softcap"), lambda c: c.pop("embedding"),
                   lambda c: c["loop"].update(times=2), lambda c: c["layers"][0]["mixer"]["mask"].update(size=12),
                   lambda c: c["layers"][0]["mixer"]["rot"].update(dims=14), lambda c: c["layers"][0]["mixer"].update(conv=1),
                   lambda c: c["layers"][3]["mixer"].update(scale=0.5), lambda c: c["layers"][2]["mixer"].update(norm_groups=3),
                   lambda c: c["embedding"]["bigram"].update(mul_prev=14)]:
        other = copy.deepcopy(cfg)
        change(other)
        assert moved(other) > 1e-3, "a mechanism that changes nothing"
    for name in ["l1.mix.u", "l1.mix.mu.w", "l2.mix.D", "l2.mix.conv.b", "l0.mix.g", "l4.mix.w0", "l2.mix.dt_bias", "l0.norm2"]:
        other = dict(w)
        other[name] = w[name] + 0.5
        assert moved(cfg, other) > 1e-3, f"{name} changes nothing"


def test_random_weights_folder_has_every_tensor(tmp_path):
    from gguf_rs_cli_b200.config import load_config
    from gguf_rs_cli_b200.models.decoder import tensor_requests
    from gguf_rs_cli_b200.weights import SafetensorsFile
    from gguf_rs_cli_b200.weights.random_init import write_random_model
    folder = write_random_model(str(tmp_path / "m"), config("small"), seed=1)
    arch, cfg = load_config(folder)
    names = {r.name for r in tensor_requests(arch.build_spec(cfg))}
    f = SafetensorsFile(str(tmp_path / "m" / "model.safetensors"))
    assert set(f.names()) == names
