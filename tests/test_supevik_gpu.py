"""Supevik on the GPU against the plain implementation (tests/plain_supevik.py): every mechanism
alone, whole prompts, decoding through the cache, portions of prompts, unequal batches, slots and
pages used again, windows' and pages' edges, far keys, long decoding, greedy generation and the
trace program.  Configurations and weights are the tests' own (tests/supevik_util.py)."""
import json
import math
import os
import subprocess
import sys

import pytest
import torch

import gpu_util as G
import helpers
import plain_supevik as plain
import supevik_util as U

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]
NAMES = ["loop3", "odd", "ones", "plain", "sharp"]


@pytest.fixture(scope="module")
def root(tmp_path_factory):
    return tmp_path_factory.mktemp("supevik")


_engines, _plain = {}, {}


def engine_of(root, name, dtype, max_slots=None, use_graphs=None, edit=None, edit_weights=None):
    import moe_b200
    from moe_b200.engine import Engine

    d = U.model_folder(root, name, edit=edit, edit_weights=edit_weights)
    key = (d, dtype, max_slots, use_graphs)
    if key not in _engines:
        _engines[key] = Engine(moe_b200.load_model(d, dtype=dtype), max_tokens=2048, max_slots=max_slots,
                               use_graphs=use_graphs)
    return d, _engines[key]


def plain_of(folder, toks, layers_out=None):
    key = (folder, tuple(toks))
    if layers_out is not None:
        cfg, w = plain.read_model(folder)
        return plain.forward(cfg, w, toks, layers_out)
    if key not in _plain:
        cfg, w = plain.read_model(folder)
        _plain[key] = plain.forward(cfg, w, toks)
    return _plain[key]


def tol_of(name, dtype):
    """Against the plain implementation.  In bfloat16 queries and keys are rounded to 8 bits before the
    score, whose error is the score's size times 2^-8 or so: with the peaked attention of "sharp" and
    "far" (scores of 10 and more) that is tenths, several times what the ordinary scores of the other
    configurations give."""
    if dtype == "bfloat16" and name in ("sharp", "far"):
        return 3 * G.tol(dtype)
    return G.tol(dtype)


def dev(t, dtype=torch.float32):
    return t.to(dtype).cuda().contiguous()


# ----------------------------------------------------------------------------- mechanisms alone
@pytest.mark.parametrize("H", [64, 50])
@pytest.mark.parametrize("bf16", [False, True])
def test_dynamic_tanh_kernel_with_and_without_the_sum_in_front(H, bf16):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(H)
    T = 9
    x, delta = torch.randn(T, H, generator=g) * 2, torch.randn(T, H, generator=g) * 2
    w = {}
    for n in ("pre", "post"):
        w[n], w[n + ".b"], w[n + ".alpha"] = 1 + 0.3 * torch.randn(H, generator=g), 0.2 * torch.randn(H, generator=g), torch.tensor(0.6 if n == "pre" else 1.3)
    tri = lambda n: (w[n + ".alpha"].cuda(), dev(w[n]), dev(w[n + ".b"]))
    wd = {k: v.double() for k, v in w.items()}
    rows = torch.tensor([7, 0, 3], dtype=torch.int32).cuda()
    status = core.new_status("cuda")
    for post, use_delta, use_rows in [(False, False, False), (False, True, False), (True, True, False), (True, True, True)]:
        xs = dev(x)
        n = 3 if use_rows else T
        out = torch.empty((n, H), dtype=torch.bfloat16 if bf16 else torch.float32, device="cuda")
        core.dyt(xs, tri("pre"), delta=dev(delta) if use_delta else None, post=tri("post") if post else None,
                 rows=rows if use_rows else None, status=status, **{"out16" if bf16 else "out32": out})
        s = x.double()
        if use_delta:
            s = s + (plain.dynamic_tanh(delta.double(), wd, "post") if post else delta.double())
        ref = plain.dynamic_tanh(s, wd, "pre")
        if use_rows:
            ref = ref[rows.cpu().long()]
            assert torch.equal(xs.cpu(), x)                   # a selection of rows leaves the stream alone
        elif use_delta:
            assert (xs.cpu().double() - s).abs().max() < 1e-5     # the sum went back into the stream
        assert (out.double().cpu() - ref).abs().max() < (2e-2 if bf16 else 2e-6)
    # the identity in place of the norm, into one half of a wider buffer
    both = torch.zeros((T, 2 * H), device="cuda")
    core.dyt(dev(x), None, delta=dev(delta), post=tri("post"), out32=both[:, H:], write_back=False, status=status)
    ref = x.double() + plain.dynamic_tanh(delta.double(), wd, "post")
    assert (both[:, H:].double().cpu() - ref).abs().max() < 1e-5 and float(both[:, :H].abs().max()) == 0.0
    core.check_status(status)


@pytest.mark.parametrize("bf16", [False, True])
@pytest.mark.parametrize("extra", [5, 8])      # a row pitch that allows 16-byte accesses, and one that does not
@pytest.mark.parametrize("nh,nkv,d,dv,rot,scaling", [(3, 1, 24, 40, 8, U.YARN), (4, 2, 32, 16, 32, None), (2, 2, 16, 16, 0, None),
                                                      (5, 5, 40, 8, 16, dict(U.YARN, factor=1.5)), (2, 1, 20, 20, 12, None),
                                                      (9, 3, 128, 128, 64, U.YARN), (2, 1, 160, 96, 32, None)])
def test_heads_prepare_norm_rotation_split_and_zero_fill(bf16, extra, nh, nkv, d, dv, rot, scaling):
    from moe_b200.config.spec import PartSpec
    from moe_b200.ops import core
    from moe_b200.parts.attention import record_width
    from moe_b200.parts.base import make_part

    g = torch.Generator().manual_seed(d * dv)
    T = 11
    width = (nh + nkv) * d + nkv * dv + extra
    proj = torch.randn(T, width, generator=g) * 3
    pos = torch.tensor([0, 1, 2, 63, 64, 65, 500, 1000, 4095, 7, 7], dtype=torch.int32)
    qn, kn = 1 + 0.3 * torch.randn(d, generator=g), 1 + 0.3 * torch.randn(d, generator=g)
    eps = 1e-3
    D = record_width(d, dv, bf16)
    dt = torch.bfloat16 if bf16 else torch.float32
    q, k, v = (torch.full((T, n, D), 7.0, dtype=dt, device="cuda") for n in (nh, nkv, nkv))
    freq, mscale = None, 1.0
    rd = {"dims": rot, "base": 10000.0}
    if rot:
        if scaling:
            rd["scaling"] = scaling
            part = make_part("position", PartSpec("rotary_yarn", dict(theta=10000.0, rotary_dim=rot, **scaling)))
            freq, mscale = part.frequencies().cuda(), part.cos_sin_scale()
        else:
            freq = plain.yarn_frequencies(rd)[0].float().cuda()
    status = core.new_status("cuda")
    core.heads_prepare(dev(proj), pos.cuda(), torch.zeros(T, dtype=torch.int32).cuda(), nh=nh, nkv=nkv, d=d, dv=dv,
                       width=D, q=q, k=k, v=v, q_norm=dev(qn), k_norm=dev(kn), eps=eps, freq=freq, rot=rot, mscale=mscale,
                       status=status)
    P = proj.double()
    rq = plain.unit_rms(P[:, :nh * d].reshape(T, nh, d), qn.double(), eps)
    rk = plain.unit_rms(P[:, nh * d:(nh + nkv) * d].reshape(T, nkv, d), kn.double(), eps)
    if rot:
        rq, rk = plain.rotate(rq, pos, rd), plain.rotate(rk, pos, rd)
    rv = P[:, (nh + nkv) * d:(nh + nkv) * d + nkv * dv].reshape(T, nkv, dv)
    tol = 3e-2 if bf16 else 2e-4          # (float32 angles at positions in the thousands)
    for got, ref, n in ((q, rq, d), (k, rk, d), (v, rv, dv)):
        got = got.double().cpu()
        assert (got[..., :n] - ref).abs().max() < tol * max(1.0, float(ref.abs().max()))
        assert float(got[..., n:].abs().max() if n < D else 0.0) == 0.0
    core.check_status(status)


@pytest.mark.parametrize("bf16", [False, True])
def test_gate_and_packing(bf16):
    from moe_b200.ops import core

    g = torch.Generator().manual_seed(5)
    T, nh, dv, D = 6, 3, 24, 32
    dt = torch.bfloat16 if bf16 else torch.float32
    ctx = (torch.randn(T, nh, D, generator=g)).to(dt)
    proj = torch.randn(T, 100 + nh * dv, generator=g) * 2
    out = torch.empty((T, nh * dv), dtype=dt, device="cuda")
    pj = dev(proj)
    core.gate_pack(ctx.cuda(), out, nh=nh, dv=dv, width=D, gate=pj[:, 100:])
    ref = ctx.double()[..., :dv].reshape(T, nh * dv) * torch.sigmoid(proj.double()[:, 100:])
    assert (out.double().cpu() - ref).abs().max() < (2e-2 if bf16 else 1e-6)
    core.gate_pack(ctx.cuda(), out, nh=nh, dv=dv, width=D)
    assert torch.equal(out.cpu(), ctx[..., :dv].reshape(T, nh * dv))


def test_gelu_gated_product_on_both_paths():
    from moe_b200.ops import core, tc

    g = torch.Generator().manual_seed(8)
    M, K, I = 70, 64, 136
    a, wgu = torch.randn(M, K, generator=g), torch.randn(2 * I, K, generator=g) / 8
    gu = a.double() @ wgu.double().T
    out = torch.empty((M, I), device="cuda")
    core.swiglu(dev(gu), out, "gelu_tanh")
    ref = plain.gelu_tanh(gu[:, :I]) * gu[:, I:]
    assert (out.double().cpu() - ref).abs().max() < 1e-5 * float(ref.abs().max())
    a16, w16 = a.to(torch.bfloat16), wgu.to(torch.bfloat16)
    gu = a16.double() @ w16.double().T
    ref = plain.gelu_tanh(gu[:, :I]) * gu[:, I:]
    status = core.new_status("cuda")
    for rows in (M, 3):           # the persistent form's epilogue and the few-tokens one
        out = torch.empty((rows, I), dtype=torch.bfloat16, device="cuda")
        assert tc.gemm_tc(a16[:rows].cuda().contiguous(), w16.cuda(), out, swiglu=True, status=status, act="gelu_tanh")
        assert (out.double().cpu() - ref[:rows]).abs().max() < 1e-2 * float(ref.abs().max())
        silu = torch.empty_like(out)
        assert tc.gemm_tc(a16[:rows].cuda().contiguous(), w16.cuda(), silu, swiglu=True, status=status)
        rs = torch.nn.functional.silu(gu[:rows, :I]) * gu[:rows, I:]
        assert (silu.double().cpu() - rs).abs().max() < 1e-2 * float(rs.abs().max())
    core.check_status(status)


# ----------------------------------------------------------------------------- whole prompts, layer by layer
@pytest.mark.parametrize("name", NAMES)
def test_every_layer_run_of_a_whole_prompt_in_32_bit(root, name):
    d, eng = engine_of(root, name, "float32", use_graphs=False)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 150, 1)
    ref_layers = []
    ref = plain_of(d, toks, ref_layers)
    eng.model.stream_tap = []
    try:
        s = eng.new_sequence()
        got = eng.step([s], [toks], [list(range(len(toks)))]).cpu()
        eng.release(s)
        tap = eng.model.stream_tap
    finally:
        eng.model.stream_tap = None
    assert len(tap) == len(ref_layers) == len(plain.layer_order(U.config_dict(name)))
    for i, (a, b) in enumerate(zip(tap, ref_layers)):
        assert helpers.max_rel_err(a.cpu(), b) < 2e-5, f"layer run {i}"
    assert helpers.max_rel_err(got, ref) < G.tol("float32")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_whole_prompts_of_many_lengths(root, name, dtype):
    """Lengths around a page (64), around the windows, one and two tokens, and past two pages."""
    d, eng = engine_of(root, name, dtype)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"w{n}": U.tokens(V, n, n) for n in (1, 2, 7, 8, 63, 64, 65, 71, 129, 200)}
    got = helpers.replay_whole(eng, reqs)
    for rid, toks in reqs.items():
        assert helpers.max_rel_err(got[rid], plain_of(d, toks)) < tol_of(name, dtype), rid


# ----------------------------------------------------------------------------- the same tokens cut differently
def replay_portions(engine, toks, sizes):
    """One request in portions of the given sizes (the last size repeats), logits at every place."""
    s, at, rows, i = engine.new_sequence(), 0, [], 0
    while at < len(toks):
        n = min(sizes[min(i, len(sizes) - 1)], len(toks) - at)
        rows.append(engine.step([s], [toks[at:at + n]], [list(range(n))]).cpu())
        at, i = at + n, i + 1
    engine.release(s)
    return torch.cat(rows, dim=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_decoding_token_by_token_from_the_first_token_and_long_after_the_rings_wrap(root, name, dtype):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 210, 3)
    ref = plain_of(d, toks)
    whole = helpers.replay_whole(eng, {"r": toks})["r"]
    ones = replay_portions(eng, toks, [1])                       # every token decoded alone, 210 steps
    tail = helpers.replay_tail(eng, {"r": toks}, tail=150)["r"]    # a prompt of 60, then 150 single steps
    for got in (ones, tail):
        assert helpers.max_rel_err(got, whole) < G.tol_cut(dtype)
        assert helpers.max_rel_err(got, ref) < tol_of(name, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("sizes", [[2], [3, 64, 1, 65, 2, 7], [64], [63, 2, 1, 70], [129, 5]])
def test_portions_of_a_prompt_of_several_sizes(root, name, dtype, sizes):
    d, eng = engine_of(root, name, dtype)
    toks = U.tokens(U.CONFIGS[name]["vocab"], 150 if sizes == [2] else 200, 4)
    ref = plain_of(d, toks)
    got = replay_portions(eng, toks, sizes)
    assert helpers.max_rel_err(got, ref) < tol_of(name, dtype)
    assert helpers.max_rel_err(got, helpers.replay_whole(eng, {"r": toks})["r"]) < G.tol_cut(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_unequal_batches_on_few_slots_against_each_request_alone(root, name, dtype):
    """Seven requests of unequal lengths on three slots: a batch starts with half of each prompt in one
    step and decodes together, the shorter ones leave earlier, and the next batch takes over slots and
    pages that were given back."""
    d, eng = engine_of(root, name, dtype, max_slots=3)
    V = U.CONFIGS[name]["vocab"]
    reqs = {f"b{i}": U.tokens(V, n, 20 + i) for i, n in enumerate([150, 3, 40, 1, 131, 66, 17])}
    alone = helpers.replay_whole(eng, reqs)
    for rounds in range(2):                     # the second time every slot and page has been used before
        got = helpers.replay_batches(eng, reqs, 3)
        for rid, toks in reqs.items():
            assert helpers.max_rel_err(got[rid], alone[rid]) < G.tol_cut(dtype), rid
            assert helpers.max_rel_err(got[rid], plain_of(d, toks)) < tol_of(name, dtype), rid
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_batch_of_portions_that_go_on_from_different_places(root, dtype):
    """Fresh and continued sequences mixed in one step, each bringing a different number of tokens."""
    d, eng = engine_of(root, "loop3", dtype)
    V = U.CONFIGS["loop3"]["vocab"]
    reqs = [U.tokens(V, n, 40 + n) for n in (90, 130, 70)]
    cuts = [[60, 30], [5, 64, 61], [70]]
    slots = [eng.new_sequence() for _ in reqs]
    rows = [[] for _ in reqs]
    at = [0, 0, 0]
    for step in range(3):
        live = [i for i in range(3) if step < len(cuts[i])]
        lg = eng.step([slots[i] for i in live], [reqs[i][at[i]:at[i] + cuts[i][step]] for i in live],
                      [list(range(cuts[i][step])) for i in live]).cpu()
        o = 0
        for i in live:
            rows[i].append(lg[o:o + cuts[i][step]])
            o += cuts[i][step]
            at[i] += cuts[i][step]
    for i, s in enumerate(slots):
        eng.release(s)
        assert helpers.max_rel_err(torch.cat(rows[i]), plain_of(d, reqs[i])) < G.tol(dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_both_forms_of_the_single_token_step(root, dtype):
    """The fused decode kernel (append, attention, merge, gate and packing in one launch) and the
    default three launches give the same logits."""
    import moe_b200
    from moe_b200.engine import Engine

    d = U.model_folder(root, "loop3")
    toks = U.tokens(U.CONFIGS["loop3"]["vocab"], 120, 9)
    got = {}
    for fused in (False, True):
        model = moe_b200.load_model(d, dtype=dtype)
        for b in model.blocks:
            b.mixer._fused_decode = fused
        got[fused] = helpers.replay_tail(Engine(model, max_tokens=512), {"r": toks}, tail=90)["r"]
        # (records of 64 ... 512 bytes: all of this model's in bfloat16; in float32 the layer with heads of
        # 48 has records of 192 bytes, which the fused kernel declines, and goes back to three launches)
        took = [b.mixer._fused_decode for b in model.blocks]
        assert took == ([fused] * 4 if dtype == "bfloat16" else [fused, fused, False, fused])
        assert helpers.max_rel_err(got[fused], plain_of(d, toks)) < G.tol(dtype)
    assert helpers.max_rel_err(got[True], got[False]) < G.tol_cut(dtype)


# ----------------------------------------------------------------------------- edges that random weights would hide
def with_window(delta):
    def edit(cfg):
        cfg["layers"][0]["mixer"]["mask"]["size"] += delta
    edit.__name__ = f"window{delta:+d}"
    return edit


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_just_inside_and_just_outside_the_window_in_prompts_and_in_decoding(root, dtype):
    """With peaked attention the result moves by far more than the tolerance when the window is one
    key longer or shorter (the plain implementation says by how much); the engine agrees with the
    window of the configuration, whole, decoded and in portions."""
    d, eng = engine_of(root, "sharp", dtype)
    toks = U.tokens(U.CONFIGS["sharp"]["vocab"], 100, 6)
    ref = plain_of(d, toks)
    scale = float(ref.abs().max())
    for delta in (-1, +1):
        other = plain_of(U.model_folder(root, "sharp", edit=with_window(delta)), toks)
        moved = (other - ref).abs().amax(dim=1) / scale
        w = U.CONFIGS["sharp"]["layers"][0]["mixer"]["mask"]["size"]
        assert float(moved[: w - 1].max()) == 0.0                      # before the window is full nothing differs
        assert float(moved[w + 1:].median()) > max(1e-2, 5 * G.tol(dtype))   # afterwards nearly every place does
    for got in (helpers.replay_whole(eng, {"r": toks})["r"], helpers.replay_tail(eng, {"r": toks}, tail=70)["r"],
                replay_portions(eng, toks, [5, 9, 10, 1, 64])):
        assert helpers.max_rel_err(got, ref) < tol_of("sharp", dtype)


SPIKE = 5


def spike(w, cfg):
    U.spike_token(w, cfg, SPIKE)


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_key_far_back_among_hundreds_is_seen(root, dtype):
    """The layer of this configuration sees every earlier token, and its weights are made so that the
    key of one token, which stands at the very first place only, outweighs all others.  Without that
    key (another token in its place) the plain implementation's logits move by a large part of their
    size 300 and more places later.  The engine agrees with the plain implementation on the original:
    whole, decoded one by one across five pages, and in portions."""
    d, eng = engine_of(root, "far", dtype, edit_weights=spike)
    V = U.CONFIGS["far"]["vocab"]
    toks = [SPIKE] + [t if t != SPIKE else SPIKE + 1 for t in U.tokens(V, 329, 7)]
    ref = plain_of(d, toks)
    other = plain_of(d, [SPIKE + 1] + toks[1:])
    assert float((other - ref)[300:].abs().amax(dim=1).min()) / float(ref.abs().max()) > 0.1
    for got in (helpers.replay_whole(eng, {"r": toks})["r"], helpers.replay_tail(eng, {"r": toks}, tail=40)["r"],
                replay_portions(eng, toks, [100, 64, 3, 129])):
        assert helpers.max_rel_err(got, ref) < tol_of("far", dtype)


# ----------------------------------------------------------------------------- the library's entry points
@pytest.mark.parametrize("dtype", DTYPES)
def test_greedy_generation_through_the_generation_loop(root, dtype):
    import moe_b200

    d, eng = engine_of(root, "loop3", dtype)
    V = U.CONFIGS["loop3"]["vocab"]
    prompts = [U.tokens(V, n, 60 + n) for n in (5, 70, 1, 23)]
    outs = moe_b200.generate(eng, prompts, max_tokens=12, eos=())
    for p, o in zip(prompts, outs):
        assert len(o.tokens) == 12
        ref = plain_of(d, p + o.tokens)[len(p) - 1:-1]
        top = ref.max(dim=-1).values
        margin = (2e-4 if dtype == "float32" else 4e-2) * float(ref.abs().max())
        for j, tok in enumerate(o.tokens):
            assert float(ref[j, tok]) >= float(top[j]) - margin, (p[:3], j, tok)
    assert eng.cache.ledger.slots.num_held == 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_the_trace_program_replays_steps_on_a_model_folder(root, tmp_path, dtype):
    """bin/trace_run as a user drives it: two requests start together in one step, go on by one token
    each, the shorter one ends earlier; its files against the plain implementation."""
    d = U.model_folder(root, "plain")
    V = U.CONFIGS["plain"]["vocab"]
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
    ra, rb = plain_of(d, a), plain_of(d, b)
    want = {0: ra[[0, 63, 64, 69]], 1: torch.stack([ra[70], rb[7]]), 2: rb[8:9], 3: ra[74:75]}
    import numpy as np

    for n, ref in want.items():
        got = torch.from_numpy(np.fromfile(os.path.join(out, f"{n}.f32"), dtype="<f4").reshape(-1, V))
        assert got.shape == ref.shape and helpers.max_rel_err(got, ref) < G.tol(dtype), n


def test_model_summary_names_the_new_parts(root):
    import moe_b200

    d = U.model_folder(root, "loop3")
    model = moe_b200.load_model(d, dtype="bfloat16")
    b = model.blocks[0]
    assert "Dynamic Tanh" in b.norm1.describe() and "sigmoid output gate" in b.mixer.describe()
    assert "YaRN" in b.mixer.describe() and "gelu_tanh" in b.ffn.describe() and model.blocks[1].ffn is None
    assert model.blocks[0].mixer.width == 64 and model.blocks[2].mixer.width == 64
