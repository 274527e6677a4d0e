"""Chunks, capped scores and the softmax with a sink in every attention kernel that takes them (the
plain one, the tiled one, the tcgen05 one for prompts and for steps that go on from the cache, and the
one for single-token steps with its merge of the key splits) against the plain attention function of
tests/plain_fogapel.py: unequal pasts and unequal numbers of new tokens in one batch, fresh sequences
among them, grouped heads, chunks whose ring has wrapped and whose edge falls inside a page and inside
a tile.  Pages that no sequence has written hold huge numbers, so that a key that should be masked
shows."""
import math

import pytest
import torch

import gpu_util as G
import plain_fogapel as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


@pytest.fixture(scope="module")
def libs():
    from moe_b200.ops import core, tc

    core.lib(), tc.lib()
    return core, tc


def case(libs, kernel, dt, nh, nkv, hd, variant, before, new, seed=0, edit=None):
    """-> (output of the kernel, plain reference), rows of all sequences one after another."""
    from moe_b200.cache import KVCache, KVRequest

    core, tc = libs
    chunk, softcap, sink = variant
    torch.manual_seed(seed)
    B = len(new)
    cache = KVCache({0: KVRequest(nkv, hd, chunk)}, {0: None}, max_tokens=64 * 40, max_slots=B + 1, dtype=dt, device=DEV)
    cache.groups[0].storage.fill_(3e30)
    view = cache.view(0)
    slots = [cache.acquire() for _ in range(B)]
    st = torch.zeros(4, dtype=torch.int32, device=DEV)
    K = [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(before, new)]
    V = [torch.randn(a + b, nkv, hd, device=DEV).to(dt) for a, b in zip(before, new)]
    Q = [(2 * torch.randn(b, nh, hd, device=DEV)).to(dt) for b in new]
    if edit:
        edit(Q, K, V)
    live = [i for i in range(B) if before[i] > 0]
    if live:                                         # the past goes through the cache
        for i in live:
            G.give_pages(cache, slots[i], before[i])
        b0 = G.make_batch(DEV, [slots[i] for i in live], [0] * len(live), [before[i] for i in live])
        core.kv_commit(torch.cat([K[i][:before[i]] for i in live]).contiguous(),
                       torch.cat([V[i][:before[i]] for i in live]).contiguous(), view, b0, st)
    for i in range(B):
        G.give_pages(cache, slots[i], before[i] + new[i])
    b1 = G.make_batch(DEV, slots, before, new)
    q = torch.cat(Q).contiguous()
    kn = torch.cat([K[i][before[i]:] for i in range(B)]).contiguous()
    vn = torch.cat([V[i][before[i]:] for i in range(B)]).contiguous()
    out = torch.full((q.shape[0], nh * hd), float("nan"), device=DEV, dtype=dt)
    scale = 1.0 / math.sqrt(hd)
    kw = dict(nh=nh, window=None, scale=scale, status=st, chunk=chunk or 0, softcap=softcap, sink=sink)
    if kernel == "generic":
        core.attention_generic(q, kn, vn, view, b1, out, use_local=True, **kw)
    elif kernel == "tiled":
        assert core.attention_tiled(q, kn, vn, view, b1, out, use_local=True, **kw)
    elif kernel == "tc":
        assert tc.attention_cached(q, kn, vn, view, b1, out, **kw)
    elif kernel == "tc_prompt":
        assert not any(before)
        assert tc.attention_prefill(q, kn, vn, b1, out, nkv=nkv, hd=hd, **kw)
    else:                                            # one new token each: appended first, then read from the cache
        assert all(n == 1 for n in new)
        core.kv_commit(kn, vn, view, b1, st)
        core.attention_decode(q, view, b1, out, **kw)
    torch.cuda.synchronize()
    assert st[:2].tolist() == [0, 0], st.tolist()
    refs = []
    for i in range(B):
        full_q = torch.zeros(before[i] + new[i], nh, hd, dtype=torch.float64)
        full_q[before[i]:] = Q[i].double().cpu()
        refs.append(plain.chunked_sink_attention(full_q, K[i].double().cpu(), V[i].double().cpu(), scale, softcap, chunk or 0,
                                                 sink=sink)[before[i]:].reshape(new[i], nh * hd))
    return out.double().cpu(), torch.cat(refs)


PASTS = [([0, 0, 0], [5, 70, 131]),                       # fresh sequences only: nothing from the cache
         ([10, 100], [7, 30]),
         ([130, 64, 0], [70, 129, 200]),                  # past a page's and a tile's edge; a fresh one among them
         ([700, 128, 127, 129, 1], [300, 1, 5, 257, 128]),
         ([63, 64, 65, 191, 192, 193], [1, 2, 64, 65, 3, 130])]
ONES = [([0, 1, 63, 64, 65, 199, 200, 201, 700], [1] * 9), ([299, 300, 301, 7, 8, 9, 127, 128], [1] * 8)]
# (chunk, cap, sink)
VARIANTS = [(None, 0.0, True), (1, 0.0, True), (8, 5.0, True), (64, 0.0, True), (70, 3.0, False), (100, 0.0, True),
            (200, 20.0, True), (300, 5.0, False), (None, 2.0, False)]


def check(out, ref, before, new, tol):
    assert torch.isfinite(out).all(), (before, new)
    o = 0
    for a, b in zip(before, new):
        err = float((out[o:o + b] - ref[o:o + b]).abs().max())
        assert err < tol * max(float(ref[o:o + b].abs().max()), 0.1), (before, new, a, b, err)
        o += b


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("kernel,dt,nh,nkv,hd", [("generic", torch.float32, 3, 1, 48), ("tiled", torch.float32, 4, 2, 96),
                                                 ("tiled", torch.bfloat16, 2, 2, 80), ("tc", torch.bfloat16, 6, 3, 64),
                                                 ("tc", torch.bfloat16, 5, 1, 128)])
def test_steps_of_several_tokens_against_plain(libs, kernel, dt, nh, nkv, hd, variant):
    for n, (before, new) in enumerate(PASTS):
        out, ref = case(libs, kernel, dt, nh, nkv, hd, variant, before, new, seed=n + hd)
        check(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("hd", [64, 128])
def test_whole_prompts_on_the_tensor_cores_against_plain(libs, hd, variant):
    before, new = [0, 0, 0, 0], [5, 70, 131, 400]
    out, ref = case(libs, "tc_prompt", torch.bfloat16, 4, 2, hd, variant, before, new, seed=hd)
    check(out, ref, before, new, 2e-2)


@pytest.mark.parametrize("variant", VARIANTS)
@pytest.mark.parametrize("dt,nh,nkv,hd", [(torch.float32, 3, 1, 48), (torch.float32, 4, 2, 64), (torch.bfloat16, 6, 1, 128),
                                          (torch.bfloat16, 2, 2, 64), (torch.bfloat16, 4, 2, 80)])
def test_single_token_steps_against_plain(libs, dt, nh, nkv, hd, variant):
    for n, (before, new) in enumerate(ONES):
        out, ref = case(libs, "decode", dt, nh, nkv, hd, variant, before, new, seed=n + hd)
        check(out, ref, before, new, 2e-5 if dt == torch.float32 else 2e-2)


@pytest.mark.parametrize("kernel,dt,hd", [("tiled", torch.float32, 64), ("tc", torch.bfloat16, 64), ("tc", torch.bfloat16, 128)])
def test_a_far_key_in_the_cache_counts_exactly_while_its_chunk_lasts(libs, kernel, dt, hd):
    """One key of the past is made to stand out (query and key scaled).  Without chunks every new query
    returns that key's value (nearly: the sink takes its share).  With chunks of 650 the key at 610
    counts for the queries at 620 ... 649 and for none from 650 on."""
    past, new, far = 620, 100, 610

    def edit(Q, K, V):
        d = torch.zeros(hd, device=DEV)
        d[3] = 1.0
        K[0][far, 0] = (40 * d).to(dt)
        Q[0][:, :] = (40 * d).to(dt)

    tol = 2e-5 if dt == torch.float32 else 2e-2
    out, ref = case(libs, kernel, dt, 2, 1, hd, (None, 0.0, True), [past], [new], edit=edit)
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())
    assert float((out - out[0]).abs().max()) < 1e-2
    out, ref = case(libs, kernel, dt, 2, 1, hd, (650, 0.0, True), [past], [new], edit=edit)
    assert float((out - ref).abs().max()) < tol * float(ref.abs().max())
    assert float((out[:30] - out[0]).abs().max()) < 1e-2          # positions 620 ... 649 all return its value
    assert float((out[30] - out[0]).abs().max()) > 0.1            # position 650 starts a chunk of its own
