"""Fogapel on the GPU against the plain implementation (tests/plain_fogapel.py): every mechanism
alone, whole prompts, decoding through cache and state, portions of prompts, unequal batches, slots,
pages and state used again, chunks' and pages' edges, far keys, long decoding, greedy generation and
the trace program.  Configurations and weights are the tests' own (tests/fogapel_util.py)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import fogapel_util as U
import gpu_util as G
import helpers
import plain_fogapel as plain

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
NAMES = ["mix", "lean", "ones", "sharp", "wide"]
F = torch.float64


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("fogapel")


_engines, _models = {}, {}


def engine_of(root, name, dtype, max_slots=None, use_graphs=None, edit=None, edit_weights=None):
    import moe_b200
    from moe_b200.engine import Engine

    d = U.model_folder(root, name, edit=edit, edit_weights=edit_weights)
    key = (d, dtype, max_slots, use_graphs)
    if key not in _engines:
        _engines[key] = Engine(moe_b200.load_model(d, dtype=dtype), max_tokens=2048, max_slots=max_slots,
                               use_graphs=use_graphs)
    return d, _engines[key]


def model_of(folder):
    if folder not in _models:
        _models[folder] = plain.read_model(folder)
    return _models[folder]


def tol_of(name, dtype):
    """Against the plain implementation.  In bfloat16 queries and keys are rounded to 8 bits before the
    score, whose error is the score's size times 2^-8 or so: with the peaked attention of "sharp" and
    "far" (scores of 10 and more) that is tenths, several times what ordinary scores give."""
    if dtype == "bfloat16" and name in ("sharp", "far"):
        return 3 * G.tol(dtype)
    return G.tol(dtype)


def check_schedule(folder, eng, requests, steps, tol, flip, cut_against=None, cut_tol=None):
    """Run ``steps`` (helpers.run_schedule) and compare every wanted place with the plain
    implementation run whole, with the engine's expert choices (a choice may differ from the plain
    implementation's own only where the two router logits are within ``flip`` of each other).
    Returns {request: [rows]} for comparisons between cuts."""
    cfg, w = model_of(folder)
    logits, picks = helpers.run_schedule(eng, steps)
    out, flips, total = {}, 0, 0
    for rid, toks in requests.items():
        forced = [[layer[(rid, i)] for i in range(len(toks))] for layer in picks]
        margins = []
        ref = plain.forward(cfg, w, toks, forced=forced, margins=margins)
        assert not margins or max(margins) < flip, f"{rid}: an expert choice differs at margin {max(margins):.3g}"
        flips, total = flips + len(margins), total + len(toks) * max(len(picks), 1)
        scale = float(ref.abs().max())
        rows = {pos: row for (r, pos), row in logits.items() if r == rid}
        assert rows, rid
        for pos, row in rows.items():
            err = float((row.double() - ref[pos]).abs().max()) / scale
            assert err < tol, f"{rid} at position {pos} of {len(toks)}: relative error {err:.3g}"
        out[rid] = rows
    assert flips <= 0.05 * total, f"expert choices differ too often: {flips} of {total}"
    return out


def portions_schedule(rid, toks, sizes):
    """One request in portions of the given sizes (the last size repeats), logits at every place."""
    steps, at, i = [], 0, 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        steps.append({"entries": [(rid, toks[at:at + n], list(range(n)))], "end": [rid] if at + n == len(toks) else []})
        at, i = at + n, i + 1
    return steps


def dev(t, dtype=torch.float32):
    return t.to(dtype).cuda().contiguous()


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("nh,nkv,d,dv,rot,taps,unit", [(4, 2, 32, 16, 16, 4, True), (2, 2, 16, 48, 16, 2, True), (3, 1, 24, 40, 0, 1, True),
                                                      (1, 1, 64, 64, 8, 3, False), (5, 5, 18, 6, 6, 0, True), (2, 1, 128, 64, 64, 3, True)])
def test_convolution_rotation_of_pairs_unit_norm_and_split_in_pieces(bf16, nh, nkv, d, dv, rot, taps, unit):
    """Two sequences of unequal lengths in three steps (the second one joins later and a step brings
    fewer tokens than the convolution has taps), so that earlier rows come from the step, from the
    state, and from before the sequence's start."""
    from moe_b200.ops import core
    from moe_b200.parts.attention import record_width

    g = torch.Generator().manual_seed(nh * 100 + d)
    D = record_width(d, dv, bf16)
    ch = (nh + nkv) * d + nkv * dv
    eps, base = 1e-5, 300.0
    lens = {0: 23, 1: 9}
    proj = {s: torch.randn(n, ch, generator=g) for s, n in lens.items()}
    taps_w = (0.5 + 0.6 * torch.randn(ch, max(taps, 1), generator=g)) if taps else None
    state = torch.zeros((3, max(taps - 1, 1) * ch), device="cuda")
    freq = dev(base ** (-2.0 * torch.arange(rot // 2, dtype=F) / max(rot, 1))) if rot else None
    cuts = [[(0, 0, 10)], [(0, 10, 12), (1, 0, 2)], [(0, 12, 23), (1, 2, 9)]]       # (sequence, from, to)
    dt = torch.bfloat16 if bf16 else torch.float32
    got = {s: [] for s in lens}
    status = core.new_status("cuda")
    for step in cuts:
        batch = G.make_batch("cuda", [s + 1 for s, _, _ in step], [a for _, a, _ in step], [b - a for _, a, b in step])
        rows = dev(torch.cat([proj[s][a:b] for s, a, b in step]))
        T = rows.shape[0]
        q, k, v = (torch.full((T, n, D), 7.0, dtype=dt, device="cuda") for n in (nh, nkv, nkv))
        core.conv_heads_prepare(rows, batch, nh=nh, nkv=nkv, d=d, dv=dv, width=D, q=q, k=k, v=v,
                                taps_w=dev(taps_w.t()) if taps else None, state=state if taps > 1 else None, eps=eps,
                                unit_norm=unit, freq=freq, rot=rot, status=status)
        if taps > 1:
            core.conv_state_update(rows, state, batch, taps=taps, channels=ch)
        o = 0
        for s, a, b in step:
            got[s].append((q[o:o + b - a].double().cpu(), k[o:o + b - a].double().cpu(), v[o:o + b - a].double().cpu()))
            o += b - a
    core.check_status(status)
    for s, n in lens.items():
        u = proj[s].double()
        if taps:
            u = plain.short_convolution(u, taps_w.double())
        rq, rk, rv = u[:, :nh * d].reshape(n, nh, d), u[:, nh * d:(nh + nkv) * d].reshape(n, nkv, d), u[:, (nh + nkv) * d:].reshape(n, nkv, dv)
        if rot:
            rq, rk = plain.rotate_pairs(rq, torch.arange(n), rot, base), plain.rotate_pairs(rk, torch.arange(n), rot, base)
        if unit:
            rq, rk = plain.unit_rms(rq, eps), plain.unit_rms(rk, eps)
        for i, (ref, w_) in enumerate(((rq, d), (rk, d), (rv, dv))):
            have = torch.cat([piece[i] for piece in got[s]])
            assert float(have[..., w_:].abs().max() if D > w_ else 0.0) == 0.0            # zero-filled beyond the head
            assert (have[..., :w_] - ref).abs().max() < (3e-2 if bf16 else 2e-5) * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("fused", [True, False])
@pytest.mark.parametrize("heads,d,W,rank", [(2, 32, 64, 5), (1, 40, 48, 3), (3, 8, 32, 1), (2, 64, 128, 8), (2, 128, 64, 32), (4, 20, 24, 2),
                                            (2, 16, 40, 40), (1, 200, 32, 4)])
def test_recurrent_mixer_kernels_in_pieces_with_the_state_carried(bf16, fused, heads, d, W, rank):
    """Blends, decay, scan and the normed, gated output, for two sequences cut into unequal pieces
    (one token, two, many), against the plain loop over whole sequences.  The decay is formed in the
    blends' launch (``fused``, a narrow projection of up to 32) or by kernels of its own."""
    if fused and rank > 32:
        pytest.skip("the blends' kernel forms the decay for a narrow projection of up to 32")
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(heads * 1000 + d)
    I = heads * d
    lens = {0: 31, 1: 12}
    h = {s: torch.randn(n, W, generator=g) for s, n in lens.items()}
    mu = torch.rand(5, W, generator=g)
    Wm = {s: torch.randn(I, W, generator=g) / math.sqrt(W) for s in "rkvg"}
    w1, w2 = torch.randn(rank, W, generator=g) / math.sqrt(W), torch.randn(I, rank, generator=g)
    w0, u, nw = -1.0 + torch.randn(I, generator=g), 0.5 * torch.randn(heads, d, generator=g), 1 + 0.2 * torch.randn(I, generator=g)
    eps = 1e-5
    state = torch.zeros((3, W + I * d), device="cuda")
    dt = torch.bfloat16 if bf16 else torch.float32
    cuts = [[(0, 0, 1)], [(0, 1, 3), (1, 0, 5)], [(0, 3, 20), (1, 5, 6)], [(1, 6, 12), (0, 20, 31)]]
    got = {s: [] for s in lens}
    for step in cuts:
        batch = G.make_batch("cuda", [s + 1 for s, _, _ in step], [a for _, a, _ in step], [b - a for _, a, b in step])
        x = dev(torch.cat([h[s][a:b] for s, a, b in step]))
        T = x.shape[0]
        mixed = torch.empty((4, T, W), dtype=dt, device="cuda")
        decay = torch.empty((T, I), device="cuda")
        if fused:
            core.wkv_shift_mix(x, dev(mu), state, batch, mixed, decay=(dev(w1), dev(w2.t()), dev(w0), decay))
        else:
            xw = torch.empty((T, W), device="cuda")
            core.wkv_shift_mix(x, dev(mu), state, batch, mixed, last32=xw)
            low = dev(xw.double().cpu() @ w1.double().T)
            core.wkv_decay(low, dev(w2.t()), dev(w0), decay)
        r, k, v, gl = (dev(mixed[i].double().cpu() @ Wm[s].double().T) for i, s in enumerate("rkvg"))
        o = torch.empty((T, I), device="cuda")
        core.wkv_scan(r, k, v, decay, dev(u), state[:, W:], batch, o, heads=heads, d=d)
        y = torch.empty((T, I), dtype=dt, device="cuda")
        core.wkv_finish(o, gl, dev(nw), eps, batch, y, heads=heads, d=d)
        at = 0
        for s, a, b in step:
            got[s].append(y[at:at + b - a].double().cpu())
            at += b - a
    w = {"p.mu." + s: mu[i].double() for i, s in enumerate("rkvgw")}
    w.update({"p." + s: Wm[s].double() for s in "rkvg"})
    w.update({"p.w1": w1.double(), "p.w2": w2.double(), "p.w0": w0.double(), "p.u": u.double(), "p.norm": nw.double(),
              "p.o": torch.eye(I, dtype=F)})
    for s, n in lens.items():
        final = []
        ref = plain.wkv_mixer(w, "p", {"heads": heads, "dim": d}, h[s].double(), eps, trace=final)
        have = torch.cat(got[s])
        assert (have - ref).abs().max() < (4e-2 if bf16 else 1e-4) * max(1.0, float(ref.abs().max())), s
        S = state[s + 1, W:].double().cpu().reshape(heads, d, d)
        assert (S - final[0]).abs().max() < (3e-2 if bf16 else 1e-4) * max(1.0, float(final[0].abs().max()))
        assert torch.equal(state[s + 1, :W].cpu(), h[s][-1])                   # the last token's input, kept exactly
    assert float(state[0].abs().max()) == 0.0                                  # a slot nobody used


@pytest.mark.parametrize("H", [64, 50, 192])
@pytest.mark.parametrize("bf16", [False, True])
def test_norm_with_two_scaled_sublayer_outputs_in_front(H, bf16):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(H)
    T = 9
    x, a, b = (torch.randn(T, H, generator=g) * 2 for _ in range(3))
    sa, sb, w = (0.8 + 0.3 * torch.randn(H, generator=g) for _ in range(3))
    rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
    status = core.new_status("cuda")
    for two, use_rows in [(True, False), (False, False), (True, True)]:
        xs = dev(x)
        n = 3 if use_rows else T
        out = torch.empty((n, H), dtype=torch.bfloat16 if bf16 else torch.float32, device="cuda")
        core.rmsnorm_scaled(xs, dev(a), dev(sa), dev(b) if two else None, dev(sb) if two else None, dev(w), 1e-5,
                            rows=rows if use_rows else None, status=status, **{"out16" if bf16 else "out32": out})
        s = x.double() + a.double() * sa.double() + (b.double() * sb.double() if two else 0.0)
        ref = plain.unit_rms(s, 1e-5) * w.double()
        if use_rows:
            ref = ref[rows.cpu().long()]
            assert torch.equal(xs.cpu(), x)                   # a selection of rows leaves the stream alone
        else:
            assert (xs.cpu().double() - s).abs().max() < 1e-5     # the sum went back into the stream
        assert (out.double().cpu() - ref).abs().max() < (3e-2 if bf16 else 5e-6)
    # the second output still as routed experts left it: three picks a token (one of them none), a shared expert
    y, shared, wt = torch.randn(3 * T, H, generator=g), torch.randn(T, H, generator=g), torch.rand(T, 3, generator=g)
    pos = torch.randperm(3 * T, generator=g).reshape(T, 3).to(torch.int32)
    pos[2, 1] = -1
    for with_shared in (True, False):
        xs = dev(x)
        out = torch.empty((T, H), dtype=torch.bfloat16 if bf16 else torch.float32, device="cuda")
        core.rmsnorm_scaled(xs, dev(a), dev(sa), None, dev(sb), dev(w), 1e-5, status=status,
                            combine=(dev(y), pos.cuda(), dev(wt), 3, dev(shared) if with_shared else None),
                            **{"out16" if bf16 else "out32": out})
        comb = sum(torch.where(pos[:, j:j + 1] >= 0, wt[:, j:j + 1].double() * y.double()[pos[:, j].clamp(min=0).long()], 0.0)
                   for j in range(3)) + (shared.double() if with_shared else 0.0)
        s = x.double() + a.double() * sa.double() + comb * sb.double()
        assert (xs.cpu().double() - s).abs().max() < 1e-5
        assert (out.double().cpu() - plain.unit_rms(s, 1e-5) * w.double()).abs().max() < (3e-2 if bf16 else 5e-6)
    core.check_status(status)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("limit", [0.5, 2.5])
def test_clamped_gated_feed_forward_in_both_products(dtype, limit):
    """The gated pair min(g, L) sigmoid(1.702 min(g, L)) (clamp(u, -L, L) + 1) in the plain kernel and
    in the tensor-core product's epilogue, for few rows and many; inputs large enough that every
    clamp acts for some elements."""
    from moe_b200.ops.linear import swiglu_linear
    from moe_b200.parts.base import Runtime

    rt = Runtime("cuda", torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    g = torch.Generator().manual_seed(5)
    K, I = 64, 96
    for M in (3, 300):
        x = (torch.randn(M, K, generator=g)).to(rt.compute_dtype)
        wgu = (2.0 * torch.randn(2 * I, K, generator=g) / math.sqrt(K)).to(rt.compute_dtype)
        got = swiglu_linear(rt, x.cuda(), wgu.cuda(), "clamped_sigmoid", limit).double().cpu()
        w = {"p.gate": wgu[:I].double(), "p.up": wgu[I:].double(), "p.down": torch.eye(I, dtype=F)}
        ref = plain.clamped_glu(w, "p", x.double(), limit)
        pre = x.double() @ wgu.double().T
        assert M < 100 or (float(pre[:, :I].max()) > limit and float(pre[:, I:].min()) < -limit < limit < float(pre[:, I:].max()))
        assert (got - ref).abs().max() < (3e-2 if dtype == "bfloat16" else 1e-5) * max(1.0, float(ref.abs().max()))
    rt.check()


@pytest.mark.parametrize("T", [1, 7, 70, 300])
@pytest.mark.parametrize("E,k", [(6, 3), (5, 1), (2, 2), (1, 1), (40, 4)])
def test_router_with_a_bias_picks_by_logit_and_weights_by_the_softmax_of_the_chosen(T, E, k):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(E * 10 + k)
    H = 48
    h, wr, b = torch.randn(T, H, generator=g), torch.randn(E, H, generator=g) / math.sqrt(H), 2.0 * torch.randn(E, generator=g)
    idx = torch.empty((T, k), dtype=torch.int32, device="cuda")
    wt = torch.empty((T, k), dtype=torch.float32, device="cuda")
    core.router(dev(h), dev(wr), k, True, 1.0, idx, wt, bias=dev(b))
    z = h.double() @ wr.double().T + b.double()
    top = torch.topk(z, k, dim=-1)
    assert torch.equal(idx.cpu().long().sort(dim=-1).values, top.indices.sort(dim=-1).values)
    ref = torch.softmax(torch.gather(z, 1, idx.cpu().long()), dim=-1)
    assert (wt.double().cpu() - ref).abs().max() < 1e-5
    # the bias matters: without it other experts would be chosen for some token
    if E > k and T > 1:
        assert not torch.equal(torch.topk(z - b.double(), k, dim=-1).indices.sort(dim=-1).values, top.indices.sort(dim=-1).values)


# ----------------------------------------------------------------------------- whole prompts, layer by layer
@pytest.mark.parametrize("name", NAMES)
def test_every_layer_of_a_whole_prompt_in_32_bit(root, name):
    d, eng = engine_of(root, name, "float32", use_graphs=False)
    cfg, w = model_of(d)
    toks = U.tokens(cfg["vocab"], 150, 1)
    ref_layers = []
    ref = plain.forward(cfg, w, toks, ref_layers)
    eng.model.stream_tap = []
    try:
        s = eng.new_sequence()
        got = eng.step([s], [toks], [list(range(len(toks)))]).cpu()
        eng.release(s)
        tap = eng.model.stream_tap
    finally:
        eng.model.stream_tap = None
    assert len(tap) == len(ref_layers) == len(cfg["layers"])
    for i, (a, b) in enumerate(zip(tap, ref_layers)):
        assert helpers.max_rel_err(a.cpu(), b) < 2e-5, f"layer {i}"
    assert helpers.max_rel_err(got, ref) < G.tol("float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_of_many_lengths(root, name, dtype):
    """Lengths around a page (64), around the chunks, one and two tokens, and past two pages."""
    d, eng = engine_of(root, name, dtype)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"w{n}": U.tokens(V, n, n) for n in (1, 2, 7, 24, 25, 63, 64, 65, 71, 129, 200)}
    check_schedule(d, eng, reqs, helpers.whole_schedule(reqs), tol_of(name, dtype), G.flip(dtype))


# ----------------------------------------------------------------------------- the same tokens cut differently
def rows_close(a, b, tol):
    scale = max(float(r.abs().max()) for r in b.values())
    return all(float((a[p].double() - b[p].double()).abs().max()) / scale < tol for p in b)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_decoding_token_by_token_from_the_first_token_and_long_after_the_rings_wrap(root, name, dtype):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 210, 3)
    reqs = {"r": toks}
    tol, flip = tol_of(name, dtype), G.flip(dtype)
    check_schedule(d, eng, reqs, portions_schedule("r", toks, [1]), tol, flip)        # every token alone, 210 steps
    check_schedule(d, eng, reqs, helpers.tail_schedule(reqs, tail=150), tol, flip)    # a prompt of 60, then 150 single steps


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("sizes", [[2], [3, 64, 1, 65, 2, 7], [64], [63, 2, 1, 70], [129, 5]])
def test_portions_of_a_prompt_of_several_sizes(root, name, dtype, sizes):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 150 if sizes == [2] else 200, 4)
    check_schedule(d, eng, {"r": toks}, portions_schedule("r", toks, sizes), tol_of(name, dtype), G.flip(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_few_slots_against_the_plain_implementation(root, name, dtype):
    """Seven requests of unequal lengths on three slots: a batch starts with half of each prompt in one
    step and decodes together, the shorter ones leave earlier, and the next batch takes over slots,
    pages and state that were given back (twice, so that everything has been used before)."""
    d, eng = engine_of(root, name, dtype, max_slots=3)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"b{i}": U.tokens(V, n, 20 + i) for i, n in enumerate([150, 3, 40, 1, 131, 66, 17])}
    steps = helpers.batches_schedule(reqs, 3, lambda r: len(reqs[r]) // 2)
    for _ in range(2):
        check_schedule(d, eng, reqs, steps, tol_of(name, dtype), G.flip(dtype))
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_portions_that_go_on_from_different_places(root, dtype):
    """Fresh and continued sequences mixed in one step, each bringing a different number of tokens."""
    d, eng = engine_of(root, "mix", dtype)
    V = U.CONFIGS["mix"]["vocab"]
    reqs = {f"m{i}": U.tokens(V, n, 40 + n) for i, n in enumerate((90, 130, 70))}
    cuts = {"m0": [60, 30], "m1": [5, 64, 61], "m2": [70]}
    at = {r: 0 for r in reqs}
    steps = []
    for step in range(3):
        entries, end = [], []
        for r in reqs:
            if step < len(cuts[r]):
                n = cuts[r][step]
                entries.append((r, reqs[r][at[r]:at[r] + n], list(range(n))))
                at[r] += n
                if at[r] == len(reqs[r]):
                    end.append(r)
        steps.append({"entries": entries, "end": end})
    check_schedule(d, eng, reqs, steps, G.tol(dtype), G.flip(dtype))


# ----------------------------------------------------------------------------- edges that random weights would hide
def with_chunk(delta):
    def edit(cfg):
        cfg["layers"][0]["mixer"]["mask"]["size"] += delta
    edit.__name__ = f"chunk{delta:+d}"
    return edit


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_just_inside_and_just_outside_a_chunk_in_prompts_and_in_decoding(root, dtype):
    """With peaked attention the result moves by far more than the tolerance when the chunks are one
    position longer or shorter (the plain implementation says by how much); the engine agrees with
    the chunks of the configuration, whole, decoded and in portions."""
    d, eng = engine_of(root, "sharp", dtype)
    cfg, w = model_of(d)
    toks = U.tokens(cfg["vocab"], 100, 6)
    ref = plain.forward(cfg, w, toks)
    scale = float(ref.abs().max())
    c = cfg["layers"][0]["mixer"]["mask"]["size"]
    for delta in (-1, +1):
        other = plain.forward(*model_of(U.model_folder(root, "sharp", edit=with_chunk(delta))), toks)
        moved = (other - ref).abs().amax(dim=1) / scale
        assert float(moved[: c - 1].max()) == 0.0                      # inside the first chunk nothing differs
        assert float(moved[c + 1:].median()) > max(1e-2, 5 * G.tol(dtype))   # afterwards nearly every place does
    reqs = {"r": toks}
    for steps in (helpers.whole_schedule(reqs), helpers.tail_schedule(reqs, tail=70), portions_schedule("r", toks, [5, 9, 10, 1, 64])):
        check_schedule(d, eng, reqs, steps, tol_of("sharp", dtype), G.flip(dtype))


SPIKE = 5


def spike(w, cfg):
    U.spike_token(w, cfg, SPIKE)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_among_hundreds_is_seen_and_the_sink_counts(root, dtype):
    """The layer of this configuration sees every earlier token, and its weights are made so that the
    key of one token, which stands at the very first place only, outweighs all others.  Without that
    key (another token in its place) the plain implementation's logits move by a large part of their
    size 300 and more places later.  The engine agrees with the plain implementation on the original:
    whole, decoded one by one across five pages, and in portions.  The same layer without the spike
    has flat scores near zero, where the sink's one in the denominator is felt: leaving it out moves
    the plain result for the first tokens by much more than the tolerance."""
    d, eng = engine_of(root, "far", dtype, edit_weights=spike)
    cfg, w = model_of(d)
    toks = [SPIKE] + [t if t != SPIKE else SPIKE + 1 for t in U.tokens(cfg["vocab"], 329, 7)]
    ref = plain.forward(cfg, w, toks)
    other = plain.forward(cfg, w, [SPIKE + 1] + toks[1:])
    assert float((other - ref)[300:].abs().amax(dim=1).min()) / float(ref.abs().max()) > 0.1
    reqs = {"r": toks}
    for steps in (helpers.whole_schedule(reqs), helpers.tail_schedule(reqs, tail=40), portions_schedule("r", toks, [100, 64, 3, 129])):
        check_schedule(d, eng, reqs, steps, tol_of("far", dtype), G.flip(dtype))
    # the sink: the first tokens of a sequence have few keys, so the one in the denominator is a large part of it
    d2, eng2 = engine_of(root, "far", dtype)
    cfg2, w2 = model_of(d2)
    short = U.tokens(cfg2["vocab"], 12, 8)
    orig = plain.chunked_sink_attention
    try:
        plain.chunked_sink_attention = lambda *a, **k: orig(*a, **dict(k, sink=False))
        without = plain.forward(cfg2, w2, short)
    finally:
        plain.chunked_sink_attention = orig
    with_sink = plain.forward(cfg2, w2, short)
    assert float((without - with_sink).abs().max()) / float(with_sink.abs().max()) > 10 * G.tol(dtype)
    check_schedule(d2, eng2, {"s": short}, helpers.whole_schedule({"s": short}), G.tol(dtype), G.flip(dtype))
    check_schedule(d2, eng2, {"s": short}, portions_schedule("s", short, [1]), G.tol(dtype), G.flip(dtype))


# ----------------------------------------------------------------------------- the library's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_generation_loop(root, dtype):
    import moe_b200

    d, eng = engine_of(root, "lean", dtype)
    cfg, w = model_of(d)
    prompts = [U.tokens(cfg["vocab"], n, 60 + n) for n in (5, 70, 1, 23)]
    outs = moe_b200.generate(eng, prompts, max_tokens=12, eos=())
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain.forward(cfg, w, p + o.tokens)[len(p) - 1:-1]
        top = ref.max(dim=-1).values
        margin = (2e-4 if dtype == "float32" else 4e-2) * float(ref.abs().max())
        for j, tok in enumerate(o.tokens):
            assert float(ref[j, tok]) >= float(top[j]) - margin, (p[:3], j, tok)
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_trace_program_replays_steps_on_a_model_folder(root, tmp_path, dtype):
    """bin/trace_run as a user drives it: two requests start together in one step, go on by one token
    each, the shorter one ends earlier; its files against the plain implementation."""
    d = U.model_folder(root, "lean")
    cfg, w = model_of(d)
    V = cfg["vocab"]
    a, b = U.tokens(V, 75, 70), U.tokens(V, 9, 71)
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:70], "want": [0, 63, 64, 69]},
                                      {"id": "b", "tokens": b[:7], "want": []}], "end": []},
             {"step": 1, "entries": [{"id": "a", "tokens": [a[70]], "want": [0]}, {"id": "b", "tokens": [b[7]], "want": [0]}], "end": []},
             {"step": 2, "entries": [{"id": "a", "tokens": [a[71]], "want": []}, {"id": "b", "tokens": [b[8]], "want": [0]}], "end": ["b"]},
             {"step": 3, "entries": [{"id": "a", "tokens": a[72:], "want": [2]}], "end": ["a"]}]
    out = str(tmp_path / "out")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", d, "--dtype", dtype, "--out", out,
                        "--max-tokens", "84"], input="".join(json.dumps(s) + "\n" for s in steps), capture_output=True,
                       text=True, timeout=900)
    assert r.returncode == 0, r.stderr[-2000:]
    assert [l for l in r.stdout.splitlines() if l.startswith("done")] == [f"done {i}" for i in range(4)]
    ra, rb = plain.forward(cfg, w, a), plain.forward(cfg, w, b)      # ("lean" takes every expert: nothing to choose)
    want = {0: ra[[0, 63, 64, 69]], 1: torch.stack([ra[70], rb[7]]), 2: rb[8:9], 3: ra[74:75]}
    import numpy as np

    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        assert got.shape == ref.shape and helpers.max_rel_err(got, ref) < G.tol(dtype), n


def test_model_summary_names_the_parts(root):
    import moe_b200

    d = U.model_folder(root, "mix")
    model = moe_b200.load_model(d, dtype="bfloat16")
    b = model.blocks
    assert b[0].kind == "parallel" and "RMSNorm" in b[0].norm1.describe()
    for word in ("convolution of 4 taps", "pairs (2i, 2i+1)", "chunks of 24", "capped at 8", "sink", "unit RMS"):
        assert word in b[0].mixer.describe(), word
    assert "clamped_sigmoid" in b[0].ffn.describe() and "wkv(2 heads of 32" in b[1].mixer.describe()
    assert "rank-5" in b[1].mixer.describe() and "with bias" in b[1].ffn.describe() and b[3].ffn is None
    assert model.blocks[0].mixer.width == 64 and model.blocks[2].mixer.width == 64
    # state of fixed size: the convolution's last rows, the recurrent mixer's last input and matrices
    reqs = model.state_requests()
    assert reqs[0].shape == (3 * ((4 + 2) * 32 + 2 * 16),) and reqs[1].shape == (64 + 2 * 32 * 32,)
