"""Nazerax in the package against the plain implementation (tests/plain_nazerax.py), in 32-bit and in bfloat16: every
mechanism alone, whole prompts against token-by-token decoding, prompts cut into portions down to two tokens, unequal
batches against each request alone, slots and pages that are used again, keys far back, at page borders and just
inside and outside the window, the first tokens of a sequence, long decoding through a ring of pages that goes round,
and greedy generation through the package's entry point."""
import copy

import pytest
import torch

from tests import plain_nazerax as P
from tests.gpu_util import TOL
from tests.nazerax_util import CONFIGS, as_plain, build, config, llm, make_weights, new_engine, plain_logits, tokens_of, weights

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]
NAMES = ["small", "wide"]


def assert_close(got, want, dtype, what=""):
    """32-bit: the largest error against the largest value of the compared block, 1e-4 (the sharp test: a key left out,
    a state not carried or a wrong edge moves results by far more).  bfloat16, row by row: the root mean square of a
    row's error is held to 10% of the block's root mean square (the small model runs eleven layers' worth of bfloat16
    products, three passes of its looped stretch among them, and measures 8% on its worst rows)."""
    got, want = got.detach().float().cpu(), want.detach().float().cpu()
    assert got.shape == want.shape, f"{what}: shape {tuple(got.shape)} != {tuple(want.shape)}"
    assert torch.isfinite(got).all(), f"{what}: non-finite values"
    err, ref = float((got - want).abs().max()), max(float(want.abs().max()), 1e-6)
    if dtype == "float32":
        assert err <= TOL[dtype] * ref, f"{what}: max error {err:.3e} against max |ref| {ref:.3e} ({dtype})"
        return
    g2, w2 = got.reshape(-1, got.shape[-1]), want.reshape(-1, want.shape[-1])
    rms_ref = max(float(w2.pow(2).mean().sqrt()), 1e-6)
    worst = float((g2 - w2).pow(2).mean(-1).sqrt().max())
    assert worst <= 0.1 * rms_ref, f"{what}: a row is off by {worst:.3e}, more than 10% of {rms_ref:.3e} (max error {err:.3e}, {dtype})"


def entry(slot, tokens, want):
    from gguf_rs_cli_b200.engine.step import Entry
    return Entry(slot, tokens, want)


def tdtype(name):
    return {"float32": torch.float32, "bfloat16": torch.bfloat16}[name]


def plan_for(eng, lens, slots=None):
    slots = slots or [eng.open() for _ in lens]
    ctx, _, _ = eng.plan([entry(s, [1] * n, ()) for s, n in zip(slots, lens)])
    return ctx, slots


# ------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("out_dtype", DTYPES)
@pytest.mark.parametrize("E,terms,two", [(5, 0, True), (72, 3, True), (1000, 2, False), (256, 1, True), (12304, 2, True)])
def test_two_norms_of_one_row_with_pending_terms(E, terms, two, out_dtype):
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(E)
    T = 7
    x = torch.randn(T, E, generator=g)
    ds = [torch.randn(T, E, generator=g).to(torch.bfloat16 if i == 1 else torch.float32) for i in range(terms)]
    w1, w2 = (0.3 * torch.randn(E, generator=g)).to(tdtype(out_dtype)), (0.3 * torch.randn(E, generator=g)).to(tdtype(out_dtype))
    total = x.double() + sum(d.double() for d in ds)
    xd, o1 = x.to(DEV), torch.empty(T, E, dtype=tdtype(out_dtype), device=DEV)
    o2 = torch.empty_like(o1) if two else None
    kernels.add_rmsnorm_pair(xd, [d.to(DEV) for d in ds], w1.to(DEV), w2.to(DEV) if two else None, 1.0, 1e-5, o1, o2)
    assert_close(xd, total.float(), "float32", "the sum left in x")
    assert_close(o1, P.layer_norm_zero_centred(total, w1.double(), 1e-5).float(), out_dtype, "first norm")
    if two:
        assert_close(o2, P.layer_norm_zero_centred(total, w2.double(), 1e-5).float(), out_dtype, "second norm")
    # chosen rows only: x is left as it is
    rows = torch.tensor([5, 0, 5], dtype=torch.int32, device=DEV)
    xr, picked = x.to(DEV), torch.empty(3, E, dtype=tdtype(out_dtype), device=DEV)
    kernels.add_rmsnorm_pair(xr, [d.to(DEV) for d in ds], w1.to(DEV), None, 1.0, 1e-5, picked, None, rows=rows, write_x=False)
    assert torch.equal(xr.cpu(), x)
    assert_close(picked, P.layer_norm_zero_centred(total[[5, 0, 5]], w1.double(), 1e-5).float(), out_dtype, "chosen rows")


@pytest.mark.parametrize("name", NAMES)
def test_pair_embedding_carries_the_previous_token(name):
    """Two sequences in unequal pieces: the first token of a sequence takes the table's last row, the first token of a
    later piece the token that the piece before ended with; the copy holds the same rows."""
    cfg, w, model = config(name), weights(name), llm(name, "float32").model
    eng = new_engine(name, "float32")
    big = cfg["embedding"]["bigram"]
    seqs = [tokens_of(name, 30, 1), tokens_of(name, 12, 2)]
    slots, fed = [eng.open(), eng.open()], [0, 0]
    for cut in [(1, 3), (2, 1), (20, 7), (7, 1)]:
        pieces = [seqs[b][fed[b]:fed[b] + cut[b]] for b in range(2)]
        ctx, _, _ = eng.plan([entry(slots[b], pieces[b], ()) for b in range(2)])
        x0 = torch.empty(sum(cut), cfg["width"], device=DEV)
        stream = model.embedding.forward_stream(ctx.tokens, ctx, copy=x0)
        want = torch.cat([P.embedding(cfg, as_plain(w), pieces[b], seqs[b][fed[b] - 1] if fed[b] else None) for b in range(2)])
        assert_close(stream.x, want.float(), "float32", f"pieces {cut}")
        assert torch.equal(stream.x, x0)
        eng.cache.advance(slots, list(cut))
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    assert big["mul_prev"] * max(seqs[0]) > 2 ** 31 or name == "small"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("C,K,bias,act", [(5, 2, False, None), (72, 4, True, "silu"), (256, 3, True, None), (264, 16, False, "silu")])
def test_short_convolution_with_bias_and_without_activation(C, K, bias, act, dtype):
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32")
    g = torch.Generator().manual_seed(C + K)
    taps = (torch.rand(C, K, generator=g) - 0.5).to(torch.bfloat16).float()
    b = (torch.rand(C, generator=g) - 0.5).to(torch.bfloat16).float() if bias else None
    u = [torch.randn(40, C, generator=g).to(torch.bfloat16).float(), torch.randn(9, C, generator=g).to(torch.bfloat16).float()]
    want = []
    for s in u:
        y, _ = P.short_conv(s.double(), taps.double(), torch.zeros(K - 1, C, dtype=torch.float64), None if b is None else b.double())
        want.append(P.silu(y) if act else y)
    state = torch.zeros(eng.cache.n_slots, K - 1, C, device=DEV)
    slots, fed, got = [eng.open(), eng.open()], [0, 0], [[], []]
    td = tdtype(dtype)
    for cut in [(1, 2), (3, 1), (30, 5), (6, 1)]:
        ctx, _ = plan_for(eng, cut, slots)
        rows = torch.cat([u[i][fed[i]:fed[i] + cut[i]] for i in range(2)]).to(td).to(DEV)
        out = torch.empty_like(rows)
        kernels.short_conv(rows, taps.to(td).to(DEV), state, ctx, out, taps_t=taps.t().contiguous().to(td).to(DEV) if dtype == "bfloat16" else None,
                           bias=None if b is None else b.to(td).to(DEV), activation=act)
        eng.cache.advance(slots, list(cut))
        got[0].append(out[:cut[0]].cpu())
        got[1].append(out[cut[0]:].cpu())
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    for i in range(2):
        assert_close(torch.cat(got[i]), want[i].float(), dtype, f"convolution C={C} taps={K} sequence {i}")


@pytest.mark.parametrize("H,Dv,per_head,first", [(3, 20, True, False), (2, 36, False, True), (4, 64, True, True), (1, 300, True, True),
                                                 (1, 2048, True, True), (2, 1500, True, False), (3, 1024, False, True)])
def test_head_norm_with_rows_of_weights_and_gate_in_front(H, Dv, per_head, first):
    from gguf_rs_cli_b200 import kernels
    g = torch.Generator().manual_seed(H * Dv)
    T, eps = 6, 1e-5
    o, z = torch.randn(T, H * Dv, generator=g) * 3, torch.randn(T, H * Dv, generator=g)
    wt = 1.0 + 0.3 * torch.randn(H * Dv if per_head else Dv, generator=g)
    gate = P.silu(z.double())
    full = wt.double() if per_head else wt.double().repeat(H)
    if first:
        want = P.unit_rms((o.double() * gate).view(T, H, Dv), eps).reshape(T, -1) * full
    else:
        want = P.unit_rms(o.double().view(T, H, Dv), eps).reshape(T, -1) * full * gate
    out = torch.empty(T, H * Dv, device=DEV)
    kernels.gated_head_norm(o.to(DEV), z.to(DEV), wt.to(DEV), eps, out, H, Dv, gate_function="silu", gate_first=first)
    assert_close(out, want.float(), "float32", "head norm")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_mixer_alone_in_an_unequal_batch(name, dtype):
    """Every layer's mixer on rows of the test's own, for three sequences of unequal lengths in two steps, so that the
    second step starts from the first one's state, convolution inputs, last row and keys."""
    cfg, w, model = config(name), as_plain(weights(name)), llm(name, dtype).model
    eng = new_engine(name, dtype)
    runs = {run.layer: run for run in reversed(eng.runs)}             # a layer's first run
    slots = [eng.open() for _ in range(3)]
    g = torch.Generator().manual_seed(3)
    states = [[dict() for _ in slots] for _ in cfg["layers"]]
    for lens in ([70, 5, 1], [1, 290, 3]):
        ctx, _ = plan_for(eng, lens, slots)
        h = torch.randn(sum(lens), cfg["width"], generator=g).to(tdtype(dtype))
        for i, layer in enumerate(cfg["layers"]):
            got = model.layers[i].mixer.forward(h.to(DEV), ctx, runs[i])
            want, t0 = [], 0
            for b, n in enumerate(lens):
                want.append(P.MIXERS[layer["type"]](layer["mixer"], cfg["norm"]["eps"], w, f"l{i}.mix.", h[t0:t0 + n].double(), states[i][b]))
                t0 += n
            assert_close(got, torch.cat(want).float(), dtype, f"{name} layer {i} ({layer['type']}), step of {lens}")
        eng.cache.advance(slots, lens)


@pytest.mark.parametrize("D,H,cuts", [(8, 1, None), (20, 3, None), (64, 2, None), (100, 2, None), (128, 1, None), (200, 1, None),
                                      (20, 3, [(300, 2), (257, 400), (1, 129), (130, 157)]), (128, 2, [(640, 3), (1, 600), (47, 85)])])
def test_wkv_kernel_at_every_shape_of_its_walk(D, H, cuts):
    """The recurrence kernels alone: two sequences fed in unequal pieces give what the plain walk gives whole.  With
    pieces of more than 256 tokens the segments of a sequence are walked side by side, from states that earlier steps left."""
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32", n_tokens=4096)
    g = torch.Generator().manual_seed(D)
    cuts = cuts or [(1, 2), (2, 1), (3, 17), (1, 1), (30, 16)]
    n = max(sum(a for a, _ in cuts), sum(b for _, b in cuts))
    r, k, v, a = (torch.randn(2, n, H * D, generator=g) for _ in range(4))
    w0, u = -torch.rand(H * D, generator=g) * 4 - 1.5, torch.randn(H * D, generator=g) * 0.5
    decay = torch.exp(-torch.exp((0.3 * a + w0).double()))
    want = []
    for b in range(2):
        S, rows = torch.zeros(H, D, D, dtype=torch.float64), []
        for t in range(n):
            rt, kt, vt = (x[b, t].double().view(H, D) for x in (r, k, v))
            kv = kt[:, :, None] * vt[:, None, :]
            rows.append(torch.einsum("hij,hi->hj", S + u.double().view(H, D)[:, :, None] * kv, rt).reshape(-1))
            S = decay[b, t].view(H, D)[:, :, None] * S + kv
        want.append(torch.stack(rows))
    state = torch.full((eng.cache.n_slots, H, D, D), 7.0, device=DEV)     # slots of other sequences are not touched
    slots = [eng.open(), eng.open()]
    for s in slots:
        state[s] = 0.0
    fed, got = [0, 0], [[], []]
    for cut in cuts:
        ctx, _ = plan_for(eng, cut, slots)
        rows = [torch.cat([t[0, fed[0]:fed[0] + cut[0]], t[1, fed[1]:fed[1] + cut[1]]]).to(DEV) for t in (r, k, v, 0.3 * a)]
        out = torch.empty(sum(cut), H * D, device=DEV)
        kernels.wkv(rows[0], rows[1], rows[2], rows[3], w0.to(DEV), u.to(DEV), state, out, ctx, H, D)
        eng.cache.advance(slots, list(cut))
        got[0].append(out[:cut[0]].cpu())
        got[1].append(out[cut[0]:].cpu())
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    for b in range(2):
        assert_close(torch.cat(got[b]), want[b][:fed[b]].float(), "float32", f"wkv D={D} sequence {b}")
    others = [s for s in range(eng.cache.n_slots) if s not in slots]
    assert bool((state[others] == 7.0).all())


@pytest.mark.parametrize("N,Pv,H,G,cuts", [(4, 8, 2, 1, None), (20, 12, 6, 3, None), (64, 64, 4, 1, None), (128, 16, 8, 2, None), (16, 100, 2, 2, None),
                                           (20, 12, 6, 3, [(300, 2), (257, 400), (130, 157)])])
def test_state_space_kernel_at_every_shape_of_its_walk(N, Pv, H, G, cuts):
    from gguf_rs_cli_b200 import kernels
    eng = new_engine("small", "float32", n_tokens=4096)
    g = torch.Generator().manual_seed(N + Pv)
    cuts = cuts or [(1, 2), (2, 1), (3, 17), (1, 1), (30, 16)]
    n = max(sum(a for a, _ in cuts), sum(b for _, b in cuts))
    x, bm, cm, dt = (torch.randn(2, n, c, generator=g) for c in (H * Pv, G * N, G * N, H))
    dt_bias, a_log, skip = -torch.rand(H, generator=g) * 3 - 1, torch.rand(H, generator=g) * 2 - 1, 1 + 0.3 * torch.randn(H, generator=g)
    want = []
    for b in range(2):
        S, rows = torch.zeros(H, N, Pv, dtype=torch.float64), []
        step = P.softplus((dt[b] + dt_bias).double())
        decay = torch.exp(-torch.exp(a_log.double()) * step)
        for t in range(n):
            row = []
            for hh in range(H):
                gi = hh // (H // G)
                xt = x[b, t, hh * Pv:(hh + 1) * Pv].double()
                S[hh] = decay[t, hh] * S[hh] + step[t, hh] * bm[b, t, gi * N:(gi + 1) * N].double()[:, None] * xt[None, :]
                row.append(S[hh].T @ cm[b, t, gi * N:(gi + 1) * N].double() + skip[hh].double() * xt)
            rows.append(torch.cat(row))
        want.append(torch.stack(rows))
    state = torch.zeros(eng.cache.n_slots, H, N, Pv, device=DEV)
    slots = [eng.open(), eng.open()]
    fed, got = [0, 0], [[], []]
    for cut in cuts:
        ctx, _ = plan_for(eng, cut, slots)
        rows = [torch.cat([t[0, fed[0]:fed[0] + cut[0]], t[1, fed[1]:fed[1] + cut[1]]]) for t in (x, bm, cm, dt)]
        buf = torch.cat(rows[:3], dim=1).to(DEV)                       # x, B, C as column slices of one buffer
        out = torch.empty(sum(cut), H * Pv, device=DEV)
        kernels.ssd(buf[:, :H * Pv], buf[:, H * Pv:H * Pv + G * N], buf[:, H * Pv + G * N:], rows[3].to(DEV), dt_bias.to(DEV), a_log.to(DEV),
                    skip.to(DEV), state, out, ctx, H, G, N, Pv)
        eng.cache.advance(slots, list(cut))
        got[0].append(out[:cut[0]].cpu())
        got[1].append(out[cut[0]:].cpu())
        fed = [fed[0] + cut[0], fed[1] + cut[1]]
    for b in range(2):
        assert_close(torch.cat(got[b]), want[b][:fed[b]].float(), "float32", f"state space N={N} P={Pv} sequence {b}")


# ------------------------------------------------------------ whole models
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_request_alone(name, dtype):
    eng = new_engine(name, dtype)
    for n, seed in [(1, 1), (2, 2), (67, 3), (300, 4)]:
        toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
        s = eng.open()
        got = eng.step([entry(s, toks, range(n))])
        assert_close(got, want, dtype, f"{name} prompt of {n}")
        eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("n", [700, 1000])
def test_long_prompt_whose_wkv_projections_run_as_one_launch(n):
    """A prompt long enough for the grouped product of r, k, v and g (its blends padded to whole tiles of tokens), alone and
    beside a short one, and then cut so that the same positions come from products of their own."""
    eng = new_engine("wide", "bfloat16")
    toks, want = tokens_of("wide", n, 9), plain_logits("wide", n, 9)
    rows = list(range(0, n, 37)) + [n - 1]
    s, s2 = eng.open(), eng.open()
    got = eng.step([entry(s2, toks[:5], ()), entry(s, toks, rows)])
    assert_close(got, want[rows], "bfloat16", f"prompt of {n}")
    eng.close(s), eng.close(s2)
    s = eng.open()
    eng.step([entry(s, toks[:300], ())])
    cut = eng.step([entry(s, toks[300:], [r - 300 for r in rows if r >= 300])])
    assert_close(cut, want[[r for r in rows if r >= 300]], "bfloat16", f"prompt of {n} in two portions")
    eng.close(s)
    eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_stream_after_every_layer_run(name, dtype):
    """The residual stream behind every run of a layer (a looped layer counts each time), terms that still wait included."""
    from gguf_rs_cli_b200.parts.block import ParallelBlock
    cfg, w = config(name), as_plain(weights(name))
    toks = tokens_of(name, 33, 5)
    st = P.Stepper(cfg, w)
    st.feed(toks)
    eng, seen, orig = new_engine(name, dtype), [], ParallelBlock.forward

    def forward(self, stream, ctx, run):
        orig(self, stream, ctx, run)
        x = stream.x.clone()
        for t in ([stream.pending] if stream.pending is not None else []) + stream.more:
            x += t.float()
        seen.append(x.cpu())

    ParallelBlock.forward = forward
    try:
        s = eng.open()
        eng.step([entry(s, toks, [0])])
    finally:
        ParallelBlock.forward = orig
    assert len(seen) == len(st.trace)
    for r, (got, want) in enumerate(zip(seen, st.trace)):
        assert_close(got, want.float(), dtype, f"{name} stream behind run {r}")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_token_by_token_from_the_first(name, dtype):
    """Decoding from an empty sequence: the empty states, the token shift and the convolutions at a sequence's start,
    windows that are not yet full, and a page border on the way."""
    eng = new_engine(name, dtype)
    n, seed = 80, 8
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    s = eng.open()
    for i in range(n):
        got = eng.step([entry(s, [toks[i]], [0])])
        assert_close(got[0], want[i], dtype, f"{name} position {i} decoded alone")
    eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_in_portions(name, dtype):
    eng = new_engine(name, dtype)
    n, seed = 150, 9
    toks, want = tokens_of(name, n, seed), plain_logits(name, n, seed)
    for cuts in ([2, 3, 59, 1, 64, 21], [63, 2, 2, 83], [64, 64, 22], [1, 2, 147]):
        assert sum(cuts) == n
        s, at = eng.open(), 0
        for c in cuts:
            got = eng.step([entry(s, toks[at:at + c], range(c))])
            assert_close(got, want[at:at + c], dtype, f"{name} portion {at}..{at + c} of {cuts}")
            at += c
        eng.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_slots_and_pages_used_again(name, dtype):
    """Batches one after another in an engine with few slots and pages: what a finished request held (pages of keys,
    the recurrent states, the last token and row) goes to the next one, which must not see it."""
    eng = new_engine(name, dtype, n_tokens=64 * 7, n_slots=4)
    decode, seed = 6, 100
    for lens in ([5, 9, 13, 70], [1, 7, 20, 33], [64, 65, 2], [129, 3]):
        reqs = []
        for n in lens:
            seed += 1
            total = n + decode
            reqs.append(dict(toks=tokens_of(name, total, seed), want=plain_logits(name, total, seed), n=n,
                             keep=decode - (seed % 3), slot=eng.open(), fed=0))
        got = eng.step([entry(r["slot"], r["toks"][:r["n"]], [r["n"] - 1]) for r in reqs])
        for i, r in enumerate(reqs):
            assert_close(got[i], r["want"][r["n"] - 1], dtype, f"{name} prompt of {r['n']} in batch {lens}")
            r["fed"] = r["n"]
        live = list(reqs)
        for step in range(decode):
            live = [r for r in live if r["fed"] < r["n"] + r["keep"]]
            for r in reqs:
                if r not in live and r["slot"] is not None:
                    eng.close(r["slot"])
                    r["slot"] = None
            if not live:
                break
            got = eng.step([entry(r["slot"], [r["toks"][r["fed"]]], [0]) for r in live])
            for i, r in enumerate(live):
                assert_close(got[i], r["want"][r["fed"]], dtype, f"{name} step {step} of prompt {r['n']}")
                r["fed"] += 1
        for r in reqs:
            if r["slot"] is not None:
                eng.close(r["slot"])
        eng.cache.check()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_decoding_through_a_ring_that_goes_round(name, dtype):
    """A cache sized for steps of at most 16 tokens: the windowed layers keep a few pages that are written again and
    again.  A prompt in portions of 16, then 200 tokens one by one; the recurrent states still hold the first tokens."""
    eng = new_engine(name, dtype, n_tokens=1024, n_slots=2, max_step_tokens=16)
    assert any(g.ring_pages < 8 for g in eng.cache.groups)
    n_prompt, n = 160, 360
    toks, want = tokens_of(name, n, 21), plain_logits(name, n, 21)
    s = eng.open()
    for at in range(0, n_prompt, 16):
        got = eng.step([entry(s, toks[at:at + 16], [0, 15])])
        assert_close(got, want[[at, at + 15]], dtype, f"{name} portion at {at}")
    for i in range(n_prompt, n):
        got = eng.step([entry(s, [toks[i]], [0])])
        if i % 7 == 0 or i > n - 20:
            assert_close(got[0], want[i], dtype, f"{name} position {i}")
    eng.close(s)
    eng.cache.check()


ODD = {
    "architecture": "Nazerax", "vocab": 61, "width": 50, "norm": {"eps": 1e-4}, "logit_softcap": 4.0,
    "embedding": {"bigram": {"buckets": 7, "mul_prev": 3, "mul_cur": 1}}, "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        {"type": "wkv", "mixer": {"heads": 5, "dim": 7}, "mlp": {"kind": "dense", "ff": 33}},
        {"type": "attention", "mixer": {"heads": 4, "kv_heads": 2, "dim": 10, "vdim": 7, "conv": 5, "scale": 0.5, "mask": {"size": 1},
                                        "rot": {"base": 10.0, "dims": 2}}, "mlp": {"kind": "dense", "ff": 21}},
        {"type": "mamba2", "mixer": {"heads": 3, "vdim": 5, "state": 9, "groups": 3, "norm_groups": 5, "conv": 1}, "mlp": None},
    ],
}


@pytest.mark.parametrize("dtype", DTYPES)
def test_sizes_that_fit_no_fast_kernel(dtype):
    """Odd sizes everywhere (no multiple of 8, of 4 or even of 2 where the design allows it), a window of one position, a
    state-space layer without a convolution, a rank of one: a prompt, then single tokens, two requests together."""
    from gguf_rs_cli_b200.engine.step import Engine
    w = make_weights(ODD, {0: 1}, seed=5)
    seqs = [torch.randint(0, ODD["vocab"], (n,), generator=torch.Generator().manual_seed(n)).tolist() for n in (75, 12)]
    want = [P.forward(ODD, as_plain(w), s).float() for s in seqs]
    eng = Engine(build(ODD, w, dtype).model, n_tokens=512, n_slots=2)
    slots = [eng.open(), eng.open()]
    got = eng.step([entry(slots[0], seqs[0][:66], range(66)), entry(slots[1], seqs[1][:3], range(3))])
    assert_close(got, torch.cat([want[0][:66], want[1][:3]]), dtype, "two prompts of odd sizes")
    for i in range(9):
        got = eng.step([entry(slots[0], [seqs[0][66 + i]], [0]), entry(slots[1], [seqs[1][3 + i]], [0])])
        assert_close(got, torch.stack([want[0][66 + i], want[1][3 + i]]), dtype, f"single tokens, step {i}")


@pytest.mark.parametrize("kind", ["wkv", "mamba2", "attention", "bare"])
def test_models_of_one_kind_of_layer(kind):
    """A model whose layers are all recurrent keeps no keys at all (a cache without page groups); one of attention alone
    keeps only the convolutions' inputs beside its keys; `bare` has one attention layer with nothing optional (no window,
    no rotation, no convolution, as many key/value heads as heads, values as wide as keys, the default scale), no
    feed-forward, no pair table, no loop and no soft cap."""
    from gguf_rs_cli_b200.engine.step import Engine
    cfg = config("small")
    if kind == "bare":
        cfg = {"architecture": "Nazerax", "vocab": 50, "width": 40, "norm": {"eps": 1e-5},
               "layers": [{"type": "attention", "mixer": {"heads": 3, "dim": 24}, "mlp": None}]}
        ranks = {}
    else:
        keep = [i for i, l in enumerate(cfg["layers"]) if l["type"] == kind]
        cfg["layers"] = [cfg["layers"][i] for i in keep]
        cfg["loop"] = {"start": 0, "stop": 1, "times": 2}
        ranks = {j: 9 for j in range(len(keep))}
    w = make_weights(cfg, ranks, seed=4)
    n = 90
    toks = torch.randint(0, cfg["vocab"], (n,), generator=torch.Generator().manual_seed(9)).tolist()
    want = P.forward(cfg, as_plain(w), toks).float()
    model = build(cfg, w, "float32").model
    eng = Engine(model, n_tokens=512, n_slots=2)
    assert (len(eng.cache.groups) == 0) == (kind in ("wkv", "mamba2"))
    s = eng.open()
    got = [eng.step([entry(s, toks[:70], range(70))])]
    got += [eng.step([entry(s, [toks[i]], [0])]).clone() for i in range(70, n)]
    eng.close(s)
    assert_close(torch.cat(got), want, "float32", f"a model of {kind} layers")


# ------------------------------------------------- keys that stand out at every edge
SPIKE = {
    "architecture": "Nazerax", "vocab": 2048, "width": 48, "norm": {"eps": 1e-6},
    "layers": [{"type": "attention", "mixer": {"heads": 2, "kv_heads": 1, "dim": 24, "vdim": 16, "scale": 1.5, "mask": {"size": 70}}, "mlp": None}],
}


def spike_weights(cfg):
    """Token t + 1024 is the partner of token t: its query is the key of t (the query projection is the key projection
    behind an orthogonal map S of the rows, and the partner's row is S^T times the row of t).  A partner's score with
    its token's key is large, all other scores are a few units, so the partner's result is the value of t, if it may see
    t, and else mostly the sink's nothing."""
    g = torch.Generator().manual_seed(7)
    E, m = cfg["width"], cfg["layers"][0]["mixer"]
    k = torch.randn(m["dim"], E, generator=g) / E ** 0.5
    S, _ = torch.linalg.qr(torch.randn(E, E, generator=g))
    base = torch.randn(1024, E, generator=g)
    base = base / base.pow(2).mean(-1, keepdim=True).sqrt()
    w = {"embed": torch.cat([base, base @ S]), "l0.norm1": torch.zeros(E), "final.norm": torch.zeros(E),
         "head": torch.randn(cfg["vocab"], E, generator=g) / E ** 0.5, "l0.mix.k": k, "l0.mix.q": torch.cat([k @ S, k @ S]),
         "l0.mix.v": torch.randn(m["vdim"], E, generator=g) / E ** 0.5 * 3, "l0.mix.g": torch.zeros(2, E) ,
         "l0.mix.o": torch.randn(E, 2 * m["vdim"], generator=g) / 6}
    return {n: t.to(torch.bfloat16).float() for n, t in w.items()}


@pytest.mark.parametrize("dims", [(24, 16), (64, 64)])
@pytest.mark.parametrize("dtype", DTYPES)
def test_keys_that_stand_out_at_every_edge_in_prompt_and_decode(dtype, dims):
    """All tokens differ; for chosen pairs (i, j) position i holds the partner of the token at position j, whose key
    then takes all of i's attention if and only if i may see j.  Pairs: j just inside and just outside the window,
    across page borders, at the sequence's first positions, and hundreds of positions back."""
    cfg = copy.deepcopy(SPIKE)
    # keys and values of 64 entries reach the tiled kernel of prompts and the decode kernel in bfloat16
    cfg["layers"][0]["mixer"]["dim"], cfg["layers"][0]["mixer"]["vdim"] = dims
    cfg["layers"][0]["mixer"]["scale"] = 36.0 / dims[0]
    size = cfg["layers"][0]["mixer"]["mask"]["size"]
    w = spike_weights(cfg)
    n = 700
    toks = torch.randperm(1024, generator=torch.Generator().manual_seed(1))[:n].tolist()
    pairs = [(200, 200 - size + 1), (210, 210 - size), (size - 1, 0), (size, 0), (size + 2, 3), (64 + size - 1, 64), (64 + size + 3, 65),
             (128, 127), (129, 64), (650, 3), (660, 660 - size + 1), (670, 670 - size), (699, 699 - size + 1), (690, 690 - size), (5, 0), (1, 0)]
    for i, j in pairs:
        toks[i] = toks[j] + 1024
    pw = as_plain(w)
    want = P.forward(cfg, pw, toks).float()
    # the pairs do decide the logits: a window one longer moves them far
    longer = copy.deepcopy(cfg)
    longer["layers"][0]["mixer"]["mask"]["size"] = size + 1
    top = float(want.abs().max())
    assert float((P.forward(longer, pw, toks[:211]).float()[210] - want[210]).abs().max()) > 0.3 * top
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
                assert_close(got, want[[at + x for x in wanted]], dtype, f"portion {at}..{at + c} of {cuts}")
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
                assert_close(got[0], want[i], dtype, f"position {i} decoded alone")
        eng.close(s)


def test_a_sink_shows_when_nothing_matches():
    """A head whose scores are all far below 0 gives almost nothing; without the sink it would give a mean of values."""
    from gguf_rs_cli_b200.engine.step import Engine
    cfg = copy.deepcopy(SPIKE)
    cfg["layers"][0]["mixer"]["dim"], cfg["layers"][0]["mixer"]["vdim"] = 64, 64
    w = spike_weights(cfg)
    w["l0.mix.q"] = -w["l0.mix.q"].abs() * 4                       # queries and keys of opposite signs: scores far below 0
    w["l0.mix.k"] = w["l0.mix.k"].abs()
    w["embed"] = w["embed"].abs()
    toks = list(range(100, 180))
    want = P.forward(cfg, as_plain(w), toks).float()
    for dtype in DTYPES:
        model = build(cfg, w, dtype).model
        eng = Engine(model, n_tokens=512, n_slots=2)
        s = eng.open()
        got = [eng.step([entry(s, toks[:70], range(70))])] + [eng.step([entry(s, [t], [0])]).clone() for t in toks[70:]]
        assert_close(torch.cat(got), want, dtype, "scores far below the sink's")


@pytest.mark.parametrize("hd,window,conv", [(64, 70, 3), (128, 40, 2), (64, 200, 1), (128, 64, 4)])
def test_fast_attention_paths_agree_with_the_general_kernel(hd, window, conv):
    """One attention layer in bfloat16, fed the same rows twice: with the tiled kernel of prompts and the decode kernel
    of single tokens, and with the general kernel in their place.  Prompts in portions, then single tokens, two
    sequences of unequal lengths, in a cache whose ring goes round."""
    from gguf_rs_cli_b200.engine.step import Engine
    cfg = {"architecture": "Nazerax", "vocab": 32, "width": 128, "norm": {"eps": 1e-6},
           "layers": [{"type": "attention", "mlp": None,
                       "mixer": {"heads": 4, "kv_heads": 2, "dim": hd, "vdim": hd, "scale": 3.0 / hd, "conv": conv,
                                 "mask": {"size": window}, "rot": {"base": 100.0, "dims": hd // 2}}}]}
    w = make_weights(cfg, {}, seed=hd + window)
    model = build(cfg, w, "bfloat16").model
    mixer = model.layers[0].mixer
    assert mixer._exact_tiled() and mixer._exact_decode() and mixer.sink and mixer.gate_per_head
    g = torch.Generator().manual_seed(hd)
    steps = [(48, 33), (48, 1), (48, 48), (48, 7), (40, 48)] + [(1, 1)] * 40
    rows = [torch.randn(a + b, cfg["width"], generator=g).to(torch.bfloat16).to(DEV) for a, b in steps]
    results = []
    for fast in (True, False):
        eng = Engine(model, n_tokens=2048, n_slots=2, max_step_tokens=48)
        slots = [eng.open(), eng.open()]
        if not fast:
            mixer._exact_tiled = mixer._exact_decode = lambda: False
        outs = []
        for (a, b), h in zip(steps, rows):
            ctx, _, _ = eng.plan([entry(slots[0], [1] * a, ()), entry(slots[1], [1] * b, ())])
            outs.append(mixer.forward(h, ctx, eng.runs[0]).float().clone())
            eng.cache.advance(slots, [a, b])
        results.append(torch.cat(outs))
        if not fast:
            del mixer.__dict__["_exact_tiled"], mixer.__dict__["_exact_decode"]
    ref = float(results[1].abs().max())
    assert float((results[0] - results[1]).abs().max()) <= 2e-2 * ref, f"{float((results[0] - results[1]).abs().max())} of {ref}"


# ------------------------------------------------------------ generation
def plain_greedy(name, prompt, max_tokens):
    cfg, w = CONFIGS[name][0], as_plain(weights(name))
    st = P.Stepper(cfg, w)
    logits, out = st.feed(list(prompt)), []
    for _ in range(max_tokens):
        out.append(int(logits[-1].argmax()))
        logits = st.feed([out[-1]])
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
    cfg, w = CONFIGS["wide"][0], as_plain(weights("wide"))
    prompts = [tokens_of("wide", n, 80 + n) for n in (3, 40)]
    got = generate(llm("wide", "bfloat16"), prompts, max_tokens=12, temperature=0.0, stop_token_ids=[])
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
    assert llm("wide", "bfloat16").model.capturable and llm("small", "float32").model.capturable


def test_command_line_with_random_weights(tmp_path, capsys):
    import json
    from gguf_rs_cli_b200.cli import main
    path = tmp_path / "config.json"
    path.write_text(json.dumps(config("small")))
    assert main(["--random", str(path), "-p", "1,2,3", "-p", "9", "-n", "5", "-t", "0", "--no-eos"]) == 0
    lines = capsys.readouterr().out.strip().splitlines()
    assert len(lines) == 2 and all(len(l.split(",")) == 5 for l in lines)


def test_trace_replay_of_a_model_folder(tmp_path):
    """bin/trace_run on a Nazerax folder: whole, then two requests together, then one by one."""
    import json
    from gguf_rs_cli_b200.weights import write_safetensors
    from tests.test_trace_run_gpu import Replay
    for dtype in DTYPES:
        name = "small"
        cfg, w, V = config(name), weights(name), config(name)["vocab"]
        folder = tmp_path / f"model_{dtype}"
        folder.mkdir()
        (folder / "config.json").write_text(json.dumps(cfg))
        write_safetensors(str(folder / "model.safetensors"), [(n, t.to(torch.bfloat16)) for n, t in w.items()])
        a, b = tokens_of(name, 40, 1), tokens_of(name, 9, 2)
        wa, wb = plain_logits(name, 40, 1), plain_logits(name, 9, 2)
        r = Replay(str(folder), dtype, str(tmp_path / f"out_{dtype}"), max_tokens=49)

        def close(got, want, what):
            assert_close(torch.from_numpy(got.copy()).reshape(-1, V), want.reshape(-1, V), dtype, what)

        close(r.step([("a", a, range(40))], end=["a"]), wa, "whole")
        close(r.step([("a", a[:30], [29]), ("b", b[:5], [0, 4])]), torch.stack([wa[29], wb[0], wb[4]]), "two prompts")
        for i in range(4):
            close(r.step([("a", [a[30 + i]], [0]), ("b", [b[5 + i]], [0])], end=["b"] if i == 3 else []),
                  torch.stack([wa[30 + i], wb[5 + i]]), f"two requests, step {i}")
        close(r.step([("a", [a[34]], [0])], end=["a"]), wa[34], "the longer one alone")
        r.finish()
