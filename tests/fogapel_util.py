"""Small Fogapel configurations and weights of the tests' own making.

The weights are drawn here (not by the library's random mode) so that every constant is away from
its neutral value: norm weights, the per-channel factors on the sublayers' outputs, biases, the
convolutions' taps, the recurrent mixer's blends, decay and bonus, the router's bias.  Values are
rounded to bfloat16 and stored so, as a checkpoint is: the float32 engine, the bfloat16 engine and
the plain implementation read the same numbers.
"""
import json
import math
import os

import torch


def attention(heads=4, kv_heads=2, dim=32, vdim=32, chunk=None, rot=16, base=10000.0, scale=None, softcap=None, conv=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if chunk is not None:
        m["mask"] = {"size": chunk}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
    if softcap is not None:
        m["softcap"] = softcap
    if conv is not None:
        m["conv"] = conv
    return {"type": "attention", "mixer": m}


def wkv(heads=2, dim=32):
    return {"type": "wkv", "mixer": {"heads": heads, "dim": dim}}


def dense(ff=96, limit=1.0):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(experts=6, top=2, ff=40, shared=48):
    d = {"kind": "moe", "router": {"experts": experts, "top": top}, "expert": {"ff": ff}}
    if shared:
        d["shared"] = {"ff": shared}
    return d


def layer(mixer, mlp):
    return dict(mixer, mlp=mlp)


# Sizes differ from layer to layer and from one configuration to the next; where one configuration
# has values that coincide or are 1, another has not.
CONFIGS = {
    # both mixers and all three kinds of feed-forward; value heads smaller and larger than key heads;
    # chunks shorter than a page and longer than one (a ring of two pages); convolutions of 4 and 2 taps;
    # part of the head and the whole head rotated; three of six experts and one of five; a layer
    # without a feed-forward; a decay projection 5 wide
    "mix": dict(vocab=131, width=64, scale=2.0, eps=1e-5, rank=5, layers=[
        layer(attention(4, 2, 32, 16, chunk=24, rot=16, base=500.0, scale=0.25, softcap=8.0, conv=4), dense(96, 1.25)),
        layer(wkv(2, 32), moe(6, 3, 40, 48)),
        layer(attention(2, 2, 16, 48, chunk=70, rot=16, scale=0.3, softcap=30.0, conv=2), moe(5, 1, 32, 0)),
        layer(wkv(4, 16), None)]),
    # what may be absent is absent: no convolution, no cap, no chunks, no rotation; as many kv heads as
    # heads; heads of 24 and 40 (no multiples of 16); one recurrent head; every expert chosen (2 of 2)
    "lean": dict(vocab=97, width=48, scale=1.0, eps=1e-6, rank=3, layers=[
        layer(attention(3, 3, 24, 24, chunk=None, rot=0, scale=0.2), dense(64, 0.5)),
        layer(wkv(1, 40), moe(2, 2, 24, 16))]),
    # ones: one head on one kv head, a chunk of one position (a token sees itself only) and of exactly a
    # page, a convolution of one tap (a factor per channel), one expert of one
    "ones": dict(vocab=64, width=32, scale=0.5, eps=1e-5, rank=1, layers=[
        layer(attention(1, 1, 64, 64, chunk=64, rot=8, conv=1, softcap=5.0), moe(1, 1, 16, 8)),
        layer(attention(1, 1, 24, 40, chunk=1, rot=24, conv=3), dense(48, 2.0)),
        layer(wkv(3, 8), dense(40, 1.0))]),
    # peaked attention (a large score scale, no cap), so that one key more or less in sight changes the result
    "sharp": dict(vocab=80, width=64, scale=1.5, eps=1e-5, rank=4, layers=[
        layer(attention(4, 2, 32, 32, chunk=9, rot=16, scale=1.5, conv=2), dense(64, 1.0)),
        layer(attention(4, 1, 32, 32, chunk=None, rot=32, scale=1.5), dense(64, 1.0))]),
    # heads of 128 and 64 (records the tensor-core kernels take), a wider model, chunks of several pages
    "wide": dict(vocab=203, width=128, scale=1.0, eps=1e-5, rank=8, layers=[
        layer(attention(2, 1, 128, 64, chunk=150, rot=64, base=250.0, scale=0.09, softcap=15.0, conv=3), moe(4, 2, 64, 64)),
        layer(wkv(2, 64), dense(160, 1.5)),
        layer(attention(4, 4, 64, 64, chunk=None, rot=32, scale=0.125, conv=2), None)]),
    # one layer that sees everything, without rotation or convolution: the tests make one far key stand out in it
    "far": dict(vocab=70, width=32, scale=3.0, eps=1e-5, rank=2, layers=[
        layer(attention(2, 1, 16, 16, chunk=None, rot=0, scale=1.0), dense(48, 1.0))]),
}


def spike_token(w, cfg, token):
    """Change drawn weights of a model whose first layer is attention without rotation or convolution
    so that every query looks at the key of ``token`` wherever it stands: only that token has a
    component along feature 0, which alone feeds key dimension 0, and every query has a large
    constant along dimension 0.  After the unit norms the score of that key exceeds all others by
    about 16 x scale."""
    s = cfg["embedding"]["scale"]
    w["embed"][:, 0] = 0.0
    w["embed"][token, 0] = 3.0 / s
    w["l0.norm1"][0] = 1.0
    w["l0.mix.k"][0, :], w["l0.mix.k.b"][0] = 0.0, 0.0
    w["l0.mix.k"][0, 0] = 40.0
    d = cfg["layers"][0]["mixer"]["dim"]
    for h in range(cfg["layers"][0]["mixer"]["heads"]):
        w["l0.mix.q.b"][h * d] = 40.0


def config_dict(name):
    c = CONFIGS[name]
    return {"architecture": "Fogapel", "vocab": c["vocab"], "width": c["width"], "embedding": {"scale": c["scale"]},
            "norm": {"eps": c["eps"]}, "layers": json.loads(json.dumps(c["layers"]))}


def draw_weights(cfg, seed, rank=4):
    """name -> bfloat16 tensor for every tensor of the configuration."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}

    def mat(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(name, n, mean, std):
        out[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def glu(p, ff):
        mat(p + ".gate", ff, W, gain=1.5), mat(p + ".up", ff, W, gain=1.5), mat(p + ".down", W, ff, gain=1.5)

    out["embed"] = (torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"]).to(torch.bfloat16)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        vec(p + "norm1", W, 1.0, 0.2)
        vec(p + "ls1", W, 0.8, 0.2)
        if L["type"] == "attention":
            H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
            mat(p + "mix.q", H * d, W), vec(p + "mix.q.b", H * d, 0.0, 0.3)
            mat(p + "mix.k", G * d, W), vec(p + "mix.k.b", G * d, 0.0, 0.3)
            mat(p + "mix.v", G * dv, W, gain=1.5), vec(p + "mix.v.b", G * dv, 0.0, 0.3)
            mat(p + "mix.o", W, H * dv, gain=1.5), vec(p + "mix.o.b", W, 0.0, 0.2)
            if m.get("conv"):
                for s, ch in (("q", H * d), ("k", G * d), ("v", G * dv)):
                    out[p + f"mix.{s}.conv"] = (0.6 * torch.randn(ch, m["conv"], generator=g) + 0.5).to(torch.bfloat16)
        else:
            H, d = m["heads"], m["dim"]
            for s in "rkvgw":
                out[p + "mix.mu." + s] = torch.rand(W, generator=g).to(torch.bfloat16)
            for s in "rkvg":
                mat(p + "mix." + s, H * d, W, gain=1.3)
            mat(p + "mix.w1", rank, W, gain=1.5), mat(p + "mix.w2", H * d, rank, gain=1.5)
            vec(p + "mix.w0", H * d, -1.0, 0.8)
            out[p + "mix.u"] = (0.5 * torch.randn(H, d, generator=g)).to(torch.bfloat16)
            vec(p + "mix.norm", H * d, 1.0, 0.2)
            mat(p + "mix.o", W, H * d, gain=1.5)
        ml = L["mlp"]
        if ml:
            vec(p + "ls2", W, 0.8, 0.2)
            if ml["kind"] == "dense":
                glu(p + "mlp", ml["ff"])
            else:
                E = ml["router"]["experts"]
                mat(p + "mlp.router", E, W, gain=2.0), vec(p + "mlp.router.b", E, 0.0, 0.5)
                for e in range(E):
                    glu(p + f"mlp.e{e}", ml["expert"]["ff"])
                if ml.get("shared"):
                    glu(p + "mlp.shared", ml["shared"]["ff"])
    vec("final.norm", W, 1.0, 0.2)
    mat("head", cfg["vocab"], W)
    return out


_folders = {}


def model_folder(root, name, seed=11, edit=None, edit_weights=None):
    """Write (once) config.json and model.safetensors of configuration ``name``; ``edit(cfg)`` may
    change the configuration dict first and ``edit_weights(weights, cfg)`` the drawn weights (their
    ``__name__`` tells the folders apart)."""
    from moe_b200.weights.safetensors_io import write_safetensors

    key = (str(root), name, seed, getattr(edit, "__name__", None), getattr(edit_weights, "__name__", None))
    if key not in _folders:
        cfg = config_dict(name)
        if edit is not None:
            edit(cfg)
        d = os.path.join(str(root), "_".join(str(k) for k in key[1:]))
        os.makedirs(d, exist_ok=True)
        with open(os.path.join(d, "config.json"), "w") as f:
            json.dump(cfg, f)
        w = draw_weights(cfg, seed, CONFIGS[name]["rank"])
        if edit_weights is not None:
            edit_weights(w, cfg)
        write_safetensors(os.path.join(d, "model.safetensors"), w)
        _folders[key] = d
    return _folders[key]


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
