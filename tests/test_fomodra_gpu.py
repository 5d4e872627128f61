"""Fomodra in the package against the plain implementation (tests/plain_fomodra.py), in 32-bit and in bfloat16: every
mechanism alone, whole prompts against token-by-token decoding, prompts cut into portions down to two tokens, unequal
batches against each request alone, slots and pages that are used again, keys far back, at page borders and just inside
and outside every window and chunk, the first tokens of a sequence, long decoding through rings of pages that go round,
sizes that fit no fast kernel, and greedy generation through the package's entry point.

A router's choice is discrete: where two scores are closer than bfloat16's rounding, bfloat16 takes another expert than
the float64 oracle.  So whole models run with their routers in 32-bit, and in bfloat16 as twins in which every expert is
chosen (the same weights; `all_chosen`); the routed kernels themselves are tested in bfloat16 with the choice given."""
import copy
import math

import pytest
import torch

from tests import plain_fomodra as P
from tests.fomodra_util import CONFIGS, all_chosen, as_plain, build, config, llm, make_weights, new_engine, plain_logits, tokens_of, weights
from tests.gpu_util import TOL

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["small", "wide"]
MODEL_TOL = 3e-4


def assert_close(got, want, dtype, what="", tol=None):
    """32-bit: the largest error against the largest value of the compared block, 1e-4 for a mechanism alone and 3e-4
    for whole models (a layer alone stays below 3e-5 from the plain implementation's own stream; the norm of every
    result on its way into the stream and peaked softmaxes pass a row's error on enlarged, measured up to ten times from
    layer to layer on single rows; a key left out, a state not carried or a wrong edge moves results by far more).
    bfloat16, row by row: the root mean square of a row's error is held to 10% of the block's root mean square; of a
    whole model's rows one in twenty may be off by more, up to the block's root mean square (a result that is normed on
    its way into the stream turns with the rounding where it is close to zero: a side input of one column changes its
    sign; the 32-bit runs show such rows as their worst too, five orders of magnitude lower)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err, ref = float((got - want).abs().max()), max(float(want.abs().max()), 1e-6)
    if dtype == "float32":
        assert err <= (tol or TOL[dtype]) * ref, f"{what}: max error {err:.3e} against max |ref| {ref:.3e} ({dtype})"
        return
    g2, w2 = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
    rms_ref = max(float(w2.pow(2).mean().sqrt()), 1e-6)
    rows = (g2 - w2).pow(2).mean(-1).sqrt()
    worst, over = float(rows.max()), int((rows > 0.1 * rms_ref).sum())
    allowed = 0 if tol is None else g2.shape[0] // 20
    assert over <= allowed and worst <= rms_ref, \
        f"{what}: {over} of {g2.shape[0]} rows are off by more than 10% of {rms_ref:.3e}, the worst by {worst:.3e} (max error {err:.3e}, {dtype})"


def assert_model(got, want, dtype, what=""):
    assert_close(got, want, dtype, what, tol=MODEL_TOL)


def entry(slot, tokens, want):
    from gguf_rs_cli_b200.engine.step import Entry
    return Entry(slot, tokens, want)


def tdtype(name):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def dense(dtype):
    """bfloat16 runs the twin in which every expert is chosen."""
    return dtype == "bfloat16"


def plan_for(eng, lens, slots=None):
    slots = slots or [eng.open() for _ in lens]
    ctx, _, _ = eng.plan([entry(s, [1] * n, ()) for s, n in zip(slots, lens)])
    return ctx, slots


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("E,two,then", [(5, False, True), (72, True, True), (256, True, False), (1000, False, False), (12304, True, True)])
def test_norm_of_a_result_into_the_stream_and_of_the_next_input_in_one_pass(E, two, then, dtype):
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(E)
    T, eps, td = 6, 1e-5, tdtype(dtype)
    x = torch.randn(T, E, generator=g)
    y, y2 = torch.randn(T, E, generator=g) * 3, torch.randn(T, E, generator=g).to(td).float()
    ws = [(1 + 0.3 * torch.randn(E, generator=g)).to(td).float() for _ in range(4)]
    u = 0.5 * (P.rms_norm(y.double(), ws[0].double(), eps) + P.rms_norm(y2.double(), ws[1].double(), eps)) if two else y.double()
    want_x = x.double() + P.rms_norm(u, ws[2].double(), eps)
    xd = x.to(DEV)
    h = torch.empty(T, E, dtype=td, device=DEV) if then else None
    xb = torch.empty(T, E, dtype=torch.bfloat16, device=DEV)
    kernels.norm_sandwich(xd, y.to(DEV), ws[2].to(td).to(DEV), eps, y2=y2.to(td).to(DEV) if two else None,
                          inner_weights=(ws[0].to(td).to(DEV), ws[1].to(td).to(DEV)) if two else None, mix=0.5,
                          next_weight=ws[3].to(td).to(DEV) if then else None, h=h, xb=xb)
    assert_close(xd, want_x.float(), "float32", "the sum left in x")
    assert torch.equal(xb.float().cpu(), xd.to(torch.bfloat16).float().cpu())
    if then:
        assert_close(h, P.rms_norm(want_x, ws[3].double(), eps).float(), dtype, "the next sublayer's rows")
    if two:
        out = torch.empty(T, E, device=DEV)
        kernels.norm_sandwich(None, y.to(DEV), None, eps, y2=y2.to(td).to(DEV), inner_weights=(ws[0].to(td).to(DEV), ws[1].to(td).to(DEV)),
                              mix=0.5, u_out=out)
        assert_close(out, u.float(), "float32", "the blend alone")


def scan_plain(x, z, B, C, dt_raw, bias, a_log, skip):
    """x, z, dt_raw [T, I]; B, C [T, N]: the recurrence from a zero state in float64."""
    T, I = x.shape
    S = torch.zeros(I, a_log.shape[1], dtype=P.F64)
    A, out = -torch.exp(a_log), torch.zeros(T, I, dtype=P.F64)
    for t in range(T):
        dt = P.softplus(dt_raw[t] + bias)
        S = torch.exp(dt[:, None] * A) * S + (dt * x[t])[:, None] * B[t][None, :]
        out[t] = (S @ C[t] + skip * x[t]) * P.silu(z[t])
    return out


@pytest.mark.parametrize("I,N,R", [(5, 3, 2), (40, 20, 5), (64, 16, 4), (32, 64, 8), (136, 33, 1), (16, 256, 3)])
def test_selective_scan_at_every_shape_in_portions_and_segments(I, N, R):
    """Two sequences in unequal portions, one of which is long enough to be walked in segments side by side; the state
    goes from step to step."""
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32", n_tokens=4096)
    g = torch.Generator().manual_seed(I * N)
    lens = (700, 90)
    data = []
    for n in lens:
        data.append({"x": torch.randn(n, I, generator=g), "z": torch.randn(n, I, generator=g), "low": torch.randn(n, R + 2 * N, generator=g),
                     "dt": torch.randn(n, I, generator=g)})
    bias, a_log, skip = torch.rand(I, generator=g) * 3 - 4, torch.rand(I, N, generator=g) * 3 - 2, torch.randn(I, generator=g)
    want = [scan_plain(d["x"].double(), d["z"].double(), d["low"][:, R:R + N].double(), d["low"][:, R + N:].double(), d["dt"].double(),
                       bias.double(), a_log.double(), skip.double()) for d in data]
    state = torch.zeros(eng.cache.n_slots, I, N, device=DEV)
    slots, fed, got = [eng.open(), eng.open()], [0, 0], [[], []]
    for cut in [(1, 3), (2, 1), (300, 20), (7, 1), (390, 65)]:
        ctx, _ = plan_for(eng, cut, slots)
        cat = {k: torch.cat([data[i][k][fed[i]:fed[i] + cut[i]] for i in range(2)]).to(DEV) for k in data[0]}
        out = torch.empty(sum(cut), I, device=DEV)
        kernels.selective_scan(cat["x"], cat["z"], cat["low"], R, N, cat["dt"], bias.to(DEV), a_log.to(DEV), skip.to(DEV), state, out, ctx)
        eng.cache.advance(slots, list(cut))
        got[0].append(out[:cut[0]].cpu())
        got[1].append(out[cut[0]:].cpu())
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    for i in range(2):
        assert_close(torch.cat(got[i]), want[i].float(), "float32", f"scan inner={I} state={N} sequence {i}")


@pytest.mark.parametrize("n,extra,top", [(5, 2, 3), (12, 0, 2), (1, 1, 2), (40, 3, 8), (3, 0, 3)])
def test_router_with_softmax_scores_and_a_correction_for_the_choice(n, extra, top):
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(n + extra)
    T, K = 9, 24
    h = torch.randn(T, K, generator=g)
    W = {"m.router": torch.randn(n + extra, K, generator=g).double(), "m.correction": (0.3 * torch.randn(n + extra, generator=g)).double()}
    mlp = {"router": {"experts": n, "identity": extra, "top": top}}
    ids_want, w_want = P.route(mlp, W, "m.", h.double())
    ids, wts = torch.empty(T, top, dtype=torch.int32, device=DEV), torch.empty(T, top, device=DEV)
    kernels.moe_router(h.to(DEV), W["m.router"].float().to(DEV), 1, 1, top, 1.0, ids, wts, softmax=True,
                       correction=W["m.correction"].float().to(DEV))
    assert ids.cpu().tolist() == ids_want.tolist()
    assert_close(wts, w_want.float(), "float32", "weights")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 50])
def test_experts_with_identity_experts_for_a_given_choice(T, dtype):
    """Few tokens take the token-by-token kernels, many the sorted tiles; experts numbered behind those with matrices give
    the token's own row."""
    from gguf_rs_cli_b200 import kernels
    name, i = "wide", 2                              # four experts with matrices, four without
    cfg, w = config(name), weights(name)
    mlp, p = cfg["layers"][i]["mlp"], f"l{i}.mlp."
    model = llm(name, dtype).model
    ff = model.layers[i].feed_forward
    g = torch.Generator().manual_seed(T)
    h = torch.randn(T, cfg["width"], generator=g).to(torch.bfloat16).float()
    eng = new_engine(name, dtype)
    ctx, _ = plan_for(eng, [T])
    got = ff.forward(h.to(tdtype(dtype)).to(DEV), ctx).clone()
    ids = ctx.ws.get("moe.ids", (T, ff.top), torch.int32).cpu().long()
    assert int((ids >= 4).sum()) > 0 and int((ids < 4).sum()) > 0
    want = P.moe(mlp, as_plain(w), p, h.double(), ids=ids)
    assert_close(got, want.float(), dtype, f"{T} tokens")


def test_token_side_gate():
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(5)
    T, V, dim, L = 7, 30, 5, 4
    a, table = torch.randn(T, dim, generator=g), torch.randn(V, dim * L, generator=g)
    toks = torch.randint(0, V, (T,), generator=g)
    out = torch.empty(T, dim, device=DEV)
    kernels.token_side_gate(a.to(DEV), table.to(DEV), 2 * dim, toks.to(torch.int32).to(DEV), out)
    assert_close(out, (P.gelu_tanh(a.double()) * table.double()[toks][:, 2 * dim:3 * dim]).float(), "float32")


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request_alone(name, dtype):
    for n, seed in ((1, 1), (2, 2), (150, 3), (400, 4)):
        eng = new_engine(name, dtype, dense(dtype))
        s = eng.open()
        got = eng.step([entry(s, tokens_of(name, n, seed), range(n))])
        assert_model(got, plain_logits(name, n, seed, dense(dtype)), dtype, f"{name}: prompt of {n}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_stream_after_every_layer(name, dtype):
    cfg = all_chosen(CONFIGS[name]) if dense(dtype) else CONFIGS[name]
    toks, want = tokens_of(name, 90, 7), []
    P.forward(cfg, as_plain(weights(name)), toks, layers_out=want)
    model = llm(name, dtype, dense(dtype)).model
    eng = new_engine(name, dtype, dense(dtype))
    got, undo = [], []
    for layer in model.layers:
        orig = layer.block.forward
        undo.append((layer.block, orig))

        def fwd(stream, ctx, run, orig=orig):
            orig(stream, ctx, run)
            got.append(stream.x.clone())
        layer.block.forward = fwd
    try:
        eng.step([entry(eng.open(), toks, [0])])
    finally:
        for block, orig in undo:
            block.forward = orig
    assert len(got) == len(want)
    for i, (a, b) in enumerate(zip(got, want)):
        assert_model(a, b.float(), dtype, f"{name}: stream after layer {i}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(name, dtype):
    n = 45
    toks, want = tokens_of(name, n, 11), plain_logits(name, n, 11, dense(dtype))
    eng = new_engine(name, dtype, dense(dtype))
    s = eng.open()
    got = torch.cat([eng.step([entry(s, [t], [0])]).clone() for t in toks])
    assert_model(got, want, dtype, f"{name}: decoded from the first token")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(name, dtype):
    n = 333
    toks, want = tokens_of(name, n, 12), plain_logits(name, n, 12, dense(dtype))
    for cuts in ([2, 2, 60, 5, 64, 128, 70, 2], [1, 63, 64, 65, 3, 137], [300, 33]):
        eng = new_engine(name, dtype, dense(dtype))
        s, at, got = eng.open(), 0, []
        for c in cuts:
            got.append(eng.step([entry(s, toks[at:at + c], range(c))]).clone())
            at += c
        assert at == n
        assert_model(torch.cat(got), want, dtype, f"{name}: portions {cuts}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_slots_and_pages_used_again(name, dtype):
    """Three requests of unequal lengths start together and are decoded together; the shortest ends, its slot and pages
    go to a new request that starts alone while... no request joins a running batch: the new one runs after them, in the
    slot and the pages that were given back."""
    eng = new_engine(name, dtype, dense(dtype), n_tokens=1024, n_slots=3)
    lens, extra = [70, 3, 131], 9
    seqs = [tokens_of(name, n + extra, 20 + i) for i, n in enumerate(lens)]
    wants = [plain_logits(name, n + extra, 20 + i, dense(dtype)) for i, n in enumerate(lens)]
    slots = [eng.open() for _ in lens]
    gots = [eng.step([entry(s, q[:n], [n - 1]) for s, q, n in zip(slots, seqs, lens)]).clone()]
    rows = [torch.stack([w[n - 1] for w, n in zip(wants, lens)])]
    for j in range(extra):
        live = [i for i in range(3) if not (i == 1 and j >= 4)]            # the short request ends early
        gots.append(eng.step([entry(slots[i], [seqs[i][lens[i] + j]], [0]) for i in live]).clone())
        rows.append(torch.stack([wants[i][lens[i] + j] for i in live]))
        if j == 3:
            eng.close(slots[1])
    assert_model(torch.cat(gots), torch.cat(rows), dtype, f"{name}: prompts together, then decoded together")
    eng.close(slots[0])
    eng.close(slots[2])
    eng.check()
    # everything was given back: three new requests fill the same slots and pages
    for rounds in range(2):
        lens2 = [200, 64, 65]
        seqs2 = [tokens_of(name, n, 40 + i) for i, n in enumerate(lens2)]
        slots2 = [eng.open() for _ in lens2]
        got = eng.step([entry(s, q, [0, n - 1]) for s, q, n in zip(slots2, seqs2, lens2)])
        want = torch.cat([plain_logits(name, n, 40 + i, dense(dtype))[[0, n - 1]] for i, n in enumerate(lens2)])
        assert_model(got, want, dtype, f"{name}: slots and pages used again")
        for s in slots2:
            eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_through_rings_that_go_round(name, dtype):
    """Steps of at most 16 tokens keep the rings of the windowed layers short: 260 decoded tokens take every ring round."""
    n0, n = 50, 310
    toks, want = tokens_of(name, n, 31), plain_logits(name, n, 31, dense(dtype))
    eng = new_engine(name, dtype, dense(dtype), max_step_tokens=16)
    s = eng.open()
    for at in range(0, n0 - 2, 16):
        eng.step([entry(s, toks[at:at + 16], [])])
    got = [eng.step([entry(s, toks[48:50], [0, 1])]).clone()]
    got += [eng.step([entry(s, [toks[i]], [0])]).clone() for i in range(n0, n)]
    assert_model(torch.cat(got), want[48:], dtype, f"{name}: long decoding")


ODD = {
    "architecture": "Fomodra", "vocab": 91, "width": 50, "norm": {"eps": 1e-4}, "token_side": {"dim": 1},
    "layers": [
        {"type": "parallel", "mixer": {"left": {"heads": 5, "kv_heads": 5, "dim": 6, "vdim": 6, "scale": 0.5, "mask": {"size": 1}},
                                       "right": {"inner": 17, "state": 33, "dt_rank": 1, "conv": 1}},
         "mlp": {"kind": "moe", "router": {"experts": 1, "top": 1}, "expert": {"ff": 7, "limit": 0.5}}},
        {"type": "latent_attention", "mixer": {"heads": 1, "dim": 10, "rot_dim": 2, "vdim": 9, "kv_rank": 7, "scale": 0.3, "mask": {"size": 2},
                                               "rot": {"base": 10.0, "dims": 2}},
         "mlp": {"kind": "moe", "router": {"experts": 2, "identity": 3, "top": 5}, "expert": {"ff": 3, "limit": 3.0}, "shared": {"ff": 5, "limit": 0.7}}},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 2, "scale": 0.3, "rot": {"base": 20.0, "dims": 10}}, "mlp": None},
        {"type": "attention", "mixer": {"heads": 3, "kv_heads": 1, "dim": 10, "vdim": 2, "scale": 0.4, "kv_from": 2, "mask": {"size": 5},
                                        "rot": {"base": 20.0, "dims": 10}}, "mlp": None},
        {"type": "parallel", "mixer": {"left": {"heads": 1, "kv_heads": 1, "dim": 256, "vdim": 4, "scale": 0.1, "mask": {"size": 70}},
                                       "right": {"inner": 3, "state": 1, "dt_rank": 9, "conv": 16}}, "mlp": None},
    ],
}


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_fit_no_fast_kernel_and_values_of_one(dtype):
    """A width that is no multiple of 8, one head, one expert, a chunk of one position and a window of two, no pair
    embedding, no convolution and one of 16 taps, a state of one entry, all experts chosen, a layer that keeps all keys
    for a reader with a window."""
    cfg = copy.deepcopy(ODD)
    if dtype == "bfloat16":
        # a side input of one column is a fixed row times a sign, which bfloat16 turns wherever the column is close to zero
        cfg["token_side"]["dim"] = 3
    w = make_weights(cfg, seed=9)
    model = build(cfg, w, dtype).model
    from gguf_rs_cli_b200.engine.step import Engine
    toks = torch.randint(0, cfg["vocab"], (150,), generator=torch.Generator().manual_seed(2)).tolist()
    want = P.forward(cfg, as_plain(w), toks).float()
    for cuts in ([150], [70, 2, 1, 77], [1] * 40):
        eng = Engine(model, n_tokens=1024, n_slots=2)
        s, at, got = eng.open(), 0, []
        for c in cuts:
            got.append(eng.step([entry(s, toks[at:at + c], range(c))]).clone())
            at += c
        assert_model(torch.cat(got), want[:at], dtype, f"odd sizes, portions {cuts[:4]}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_latent_rows_of_more_than_640_entries(dtype):
    """A latent of 700 entries: the cached rows are longer than the general attention kernel's middle instance takes."""
    cfg = {"architecture": "Fomodra", "vocab": 64, "width": 64, "norm": {"eps": 1e-5},
           "layers": [{"type": "latent_attention", "mlp": None,
                       "mixer": {"heads": 2, "dim": 8, "rot_dim": 4, "vdim": 8, "kv_rank": 700, "scale": 0.3, "mask": {"size": 40},
                                 "rot": {"base": 100.0, "dims": 4}}}]}
    w = make_weights(cfg, seed=4)
    toks = torch.randint(0, 64, (90,), generator=torch.Generator().manual_seed(4)).tolist()
    want = P.forward(cfg, as_plain(w), toks).float()
    from gguf_rs_cli_b200.engine.step import Engine
    eng = Engine(build(cfg, w, dtype).model, n_tokens=512, n_slots=2)
    s = eng.open()
    got = [eng.step([entry(s, toks[:70], range(70))]).clone()] + [eng.step([entry(s, [t], [0])]).clone() for t in toks[70:]]
    assert_model(torch.cat(got), want, dtype, "a long latent row")


# ------------------------------------------------------------ keys that stand out
def spike_model(kind, size, dims=(24, 16)):
    """One layer whose attention is decided by one key: token t + 1024 is the partner of token t; its query is the key
    of t (the query projection is the key projection behind an orthogonal map S of the rows, and the partner's row is
    S^T times the row of t), so a partner's score with its token's key is large and all others are a few units.  The
    partner's result is then the value of t if it may see t, and else something else altogether."""
    g = torch.Generator().manual_seed(7)
    E, V = 64, 2048
    D, Dv = dims
    S, _ = torch.linalg.qr(torch.randn(E, E, generator=g))
    base = torch.randn(1024, E, generator=g)
    base = base / base.pow(2).mean(-1, keepdim=True).sqrt()
    k = torch.randn(D, E, generator=g) / E ** 0.5
    w = {"embed": torch.cat([base, base @ S]), "l0.norm1": torch.ones(E), "l0.norm1b": torch.ones(E), "final.norm": torch.ones(E),
         "head": torch.randn(V, E, generator=g) / E ** 0.5}
    scale = 36.0 / D
    att = {"heads": 2, "kv_heads": 1, "dim": D, "vdim": Dv, "scale": scale, "mask": {"size": size}}
    if kind == "latent_attention":
        mixer = {"heads": 2, "dim": D, "rot_dim": 4, "vdim": Dv, "kv_rank": D, "scale": scale / 3, "mask": {"size": size}, "rot": {"base": 10.0, "dims": 4}}
        p = "l0.mix."
        w[p + "q"] = torch.cat([k @ S, torch.zeros(4, E), k @ S, torch.zeros(4, E)])
        w[p + "dkv"], w[p + "dkv.norm"] = torch.cat([k, torch.zeros(4, E)]), torch.ones(D)
        w[p + "uk"] = torch.cat([torch.eye(D), torch.eye(D)])
        w[p + "uv"], w[p + "o"] = torch.randn(2 * Dv, D, generator=g) / D ** 0.5 * 3, torch.randn(E, 2 * Dv, generator=g) / 6
        w[p + "sink"], w[p + "g"] = torch.tensor([1.0, -1.0]), torch.zeros(2, E)
    else:
        p = "l0.mix." if kind == "attention" else "l0.mix.left."
        w[p + "q"], w[p + "k"] = torch.cat([k @ S, k @ S]), k
        w[p + "v"], w[p + "o"] = torch.randn(Dv, E, generator=g) / E ** 0.5 * 3, torch.randn(E, 2 * Dv, generator=g) / 6
        if kind == "attention":
            mixer = att
            w[p + "sink"] = torch.tensor([1.0, -1.0])
            for n, rows in (("q", 2 * D), ("k", D), ("v", Dv)):
                w[p + n + ".b"] = torch.zeros(rows)
        else:
            mixer = {"left": att, "right": {"inner": 8, "state": 4, "dt_rank": 2, "conv": 2}}
            q = "l0.mix.right."
            w[q + "in"], w[q + "conv"], w[q + "conv.b"] = torch.randn(16, E, generator=g) / 8, torch.rand(8, 2, generator=g), torch.zeros(8)
            w[q + "x"], w[q + "dt"], w[q + "dt.b"] = torch.randn(10, 8, generator=g) / 3, torch.randn(8, 2, generator=g), torch.full((8,), -2.0)
            w[q + "A_log"], w[q + "D"], w[q + "o"] = torch.zeros(8, 4), torch.ones(8), torch.randn(E, 8, generator=g) / 3
            w["l0.mix.left.out"], w["l0.mix.right.out"] = torch.ones(E), 0.2 * torch.ones(E)
    cfg = {"architecture": "Fomodra", "vocab": V, "width": E, "norm": {"eps": 1e-6}, "layers": [{"type": kind, "mixer": mixer, "mlp": None}]}
    return cfg, {n: t.to(torch.bfloat16).float() for n, t in w.items()}


@pytest.mark.parametrize("kind,size,dims", [("attention", 70, (24, 16)), ("attention", 70, (64, 64)), ("parallel", 70, (24, 16)),
                                            ("parallel", 64, (128, 128)), ("latent_attention", 70, (24, 16)), ("latent_attention", 100, (60, 64))])
@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_that_stand_out_at_every_edge_in_prompt_and_decode(dtype, kind, size, dims):
    """All tokens differ; for chosen pairs (i, j) position i holds the partner of the token at position j, whose key then
    takes all of i's attention if and only if i may see j.  Pairs: j just inside and just outside the window or chunk,
    across page borders, at the sequence's first positions, and hundreds of positions back."""
    cfg, w = spike_model(kind, size, dims)
    n = 700
    toks = torch.randperm(1024, generator=torch.Generator().manual_seed(1))[:n].tolist()
    if kind == "parallel":          # i sees j if both lie in one chunk
        c = size
        pairs = [(c - 1, 0), (c, 4), (c + 5, c + 2), (2 * c - 1, c + 1), (2 * c + 3, 2 * c - 2), (3 * c + 5, 3 * c), (9 * c + 9, 9 * c - 1),
                 (9 * c + 10, 9 * c), (650, 3), (5, 2), (1, 0), (135, 126), (200, 66)]
        assert not {i for i, _ in pairs} & {j for _, j in pairs}
    else:
        pairs = [(200, 200 - size + 1), (210, 210 - size), (size - 1, 0), (size, 0), (size + 2, 3), (64 + size - 1, 64), (64 + size + 3, 65),
                 (128, 127), (129, 64), (650, 3), (660, 660 - size + 1), (670, 670 - size), (699, 699 - size + 1), (690, 690 - size), (5, 0), (1, 0)]
    for i, j in pairs:
        toks[i] = toks[j] + 1024
    pw = as_plain(w)
    want = P.forward(cfg, pw, toks).float()
    # the pairs do decide the logits: a mask one position longer moves them far
    longer = copy.deepcopy(cfg)
    m = longer["layers"][0]["mixer"]
    (m["left"] if kind == "parallel" else m)["mask"]["size"] = size + 1
    i_out = pairs[1][0]              # the second pair lies just outside
    top = float(want.abs().max())
    assert float((P.forward(longer, pw, toks[:i_out + 1]).float()[i_out] - want[i_out]).abs().max()) > 0.2 * top
    rows = sorted({i for i, _ in pairs})
    model = build(cfg, w, dtype).model
    from gguf_rs_cli_b200.engine.step import Engine
    for max_step, cuts in [(None, [n]), (None, [190, 12, 2, 96, 400]), (64, [64] * 10 + [60])]:
        eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=max_step)
        s, at = eng.open(), 0
        for c in cuts:
            wanted = [r - at for r in rows if at <= r < at + c]
            got = eng.step([entry(s, toks[at:at + c], wanted)])
            if wanted:
                assert_model(got, want[[at + x for x in wanted]], dtype, f"portion {at}..{at + c} of {cuts}")
            at += c
        eng.close(s)
    # decoded one by one from position 180 on, in a cache whose ring goes round; and from the very first token
    for start in (180, 0):
        eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=32)
        s = eng.open()
        for at in range(0, start - 20, 32):
            eng.step([entry(s, toks[at:at + 32], [])])
        if start:
            eng.step([entry(s, toks[160:180], [])])
        for i in range(start, n if start else 140):
            got = eng.step([entry(s, [toks[i]], [0])])
            if i in rows:
                assert_model(got[0], want[i], dtype, f"position {i} decoded alone")
        eng.close(s)


def test_a_reader_of_another_layers_keys_sees_its_own_window():
    """Two attention layers on one cache: the first sees 20 positions, its reader 90; a partner 60 positions back shows in
    the reader's result only.  The cache keeps the wider of the two."""
    cfg, w = spike_model("attention", 20, (64, 64))
    second = copy.deepcopy(cfg["layers"][0])
    second["mixer"].update(kv_from=0, mask={"size": 90})
    cfg["layers"].append(second)
    for n in ("q", "q.b", "o", "sink"):
        w["l1.mix." + n] = w["l0.mix." + n]
    w["l1.norm1"], w["l1.norm1b"] = w["l0.norm1"], w["l0.norm1b"]
    toks = torch.randperm(1024, generator=torch.Generator().manual_seed(3))[:300].tolist()
    for i, j in [(100, 40), (150, 131), (200, 111), (250, 160), (260, 171)]:
        toks[i] = toks[j] + 1024
    want = P.forward(cfg, as_plain(w), toks).float()
    narrow = copy.deepcopy(cfg)
    narrow["layers"][1]["mixer"]["mask"]["size"] = 20
    assert float((P.forward(narrow, as_plain(w), toks).float()[100] - want[100]).abs().max()) > 0.2 * float(want.abs().max())
    from gguf_rs_cli_b200.engine.step import Engine
    for dtype in DTYPES:
        model = build(cfg, w, dtype).model
        eng = Engine(model, n_tokens=1024, n_slots=2, max_step_tokens=64)
        s = eng.open()
        got = [eng.step([entry(s, toks[:64], range(64))]).clone(), eng.step([entry(s, toks[64:90], range(26))]).clone()]
        got += [eng.step([entry(s, [t], [0])]).clone() for t in toks[90:]]
        assert_model(torch.cat(got), want, dtype, "two windows on one cache")


def test_fast_attention_paths_agree_with_the_general_kernel():
    """The wide model in bfloat16 twice: with the tiled kernel of prompts and the decode kernel of single tokens where its
    layers take them, and with the general kernel in their place."""
    name = "wide"
    model = llm(name, "bfloat16", True).model
    fast = [l.mixer for l in model.layers if l.mixer.spec.kind == "attention"] + [l.mixer.left for l in model.layers if l.mixer.spec.kind == "pair"]
    assert sum(m._exact_tiled() for m in fast) >= 3 and sum(m._exact_decode() for m in fast) >= 3
    latent = [l.mixer for l in model.layers if l.mixer.spec.kind == "latent_attention"]
    assert latent[0]._tiled()
    toks = tokens_of(name, 260, 77)
    results = []
    for use_fast in (True, False):
        if not use_fast:
            for m in fast:
                m._fast_masks = lambda: False
            latent[0]._tiled = lambda: False
        try:
            eng = new_engine(name, "bfloat16", True)
            s = eng.open()
            out = [eng.step([entry(s, toks[:200], range(200))]).clone(), eng.step([entry(s, toks[200:230], range(30))]).clone()]
            out += [eng.step([entry(s, [t], [0])]).clone() for t in toks[230:]]
            results.append(torch.cat(out))
        finally:
            if not use_fast:
                for m in fast:
                    del m.__dict__["_fast_masks"]
                del latent[0].__dict__["_tiled"]
    ref = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 2e-2 * ref, f"{float((results[0] - results[1]).abs().max())} of {ref}"


# ------------------------------------------------------------ generation
def plain_greedy(name, prompt, max_tokens):
    cfg, w = CONFIGS[name], as_plain(weights(name))
    seq, out = list(prompt), []
    for _ in range(max_tokens):
        out.append(int(P.forward(cfg, w, seq)[-1].argmax()))
        seq.append(out[-1])
    return out


def test_greedy_generation_float32_equals_plain():
    from gguf_rs_cli_b200.api import generate
    prompts = [tokens_of("small", n, 50 + n) for n in (5, 1, 13, 66)]
    got = generate(llm("small", "float32"), prompts, max_tokens=10, temperature=0.0, stop_token_ids=[])
    assert got == [plain_greedy("small", p, 10) for p in prompts]
    # more requests than the batch holds: one batch after another through the same slots
    got2 = generate(llm("small", "float32"), prompts, max_tokens=10, temperature=0.0, stop_token_ids=[], max_batch=2)
    assert got2 == got


def test_bfloat16_greedy_follows_plain_until_a_near_tie():
    from gguf_rs_cli_b200.api import generate
    cfg, w = all_chosen(CONFIGS["wide"]), as_plain(weights("wide"))
    prompts = [tokens_of("wide", n, 80 + n) for n in (3, 40)]
    got = generate(llm("wide", "bfloat16", True), prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
    off = []
    for p, g in zip(prompts, got):
        seq = list(p)
        for tok in g:
            logits = P.forward(cfg, w, seq)[-1]
            off.append(float(logits[tok]) < float(logits.max()) - 0.1 * float(logits.abs().max()))
            seq.append(tok)
    assert sum(off) <= 1, "greedy tokens that the plain model ranks far below its best"


def test_decode_steps_run_as_captured_graphs():
    """The generation loop captures decode steps of this design as of the others: every part declares its class."""
    assert llm("wide", "bfloat16", True).model.capturable and llm("small", "float32").model.capturable


def test_command_line_with_random_weights(tmp_path, capsys):
    import json
    from gguf_rs_cli_b200.cli import main
    path = tmp_path / "config.json"
    path.write_text(json.dumps(config("small")))
    assert main(["--random", str(path), "-p", "1,2,3", "-p", "9", "-n", "5", "-t", "0", "--no-eos"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split(",")) == 5 for l in lines)


def test_trace_replay_of_a_model_folder(tmp_path):
    """bin/trace_run on a Fomodra folder: whole, then two requests together, then one by one."""
    import json
    from gguf_rs_cli_b200.weights import write_safetensors
    from tests.test_trace_run_gpu import Replay
    name = "small"
    cfg, w, V = config(name), weights(name), config(name)["vocab"]
    folder = tmp_path / "model"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(str(folder / "model.safetensors"), [(k, v.to(torch.bfloat16)) for k, v in w.items()])
    a, b = tokens_of(name, 40, 1), tokens_of(name, 23, 2)
    wa, wb = plain_logits(name, 40, 1), plain_logits(name, 23, 2)
    run = Replay(str(folder), "float32", str(tmp_path / "out"), 256)
    got = torch.from_numpy(run.step([("a", a[:30], [0, 29]), ("b", b[:20], [19])])).view(3, V)
    assert_model(got, torch.stack([wa[0], wa[29], wb[19]]), "float32", "two prompts together")
    for j in range(3):
        got = torch.from_numpy(run.step([("a", [a[30 + j]], [0]), ("b", [b[20 + j]], [0])], ["b"] if j == 2 else [])).view(2, V)
        assert_model(got, torch.stack([wa[30 + j], wb[20 + j]]), "float32", f"decoded together, step {j}")
    got = torch.from_numpy(run.step([("a", a[33:], [6])], ["a"])).view(1, V)
    assert_model(got, wa[39:40], "float32", "the rest alone")
    run.finish()
