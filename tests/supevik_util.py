"""Small Supevik configurations and weights of the tests' own making.

The weights are drawn here (not by the library's random mode) so that every constant is away from
its neutral value: norm weights and shifts, the norms' alpha, the head norms' weights and the
biases.  Values are rounded to bfloat16 and stored so, as a checkpoint is: the float32 engine, the
bfloat16 engine and the plain implementation read the same numbers.
"""
import json
import math
import os

import torch


def mixer(heads=4, kv_heads=2, dim=32, vdim=32, window=8, rot=16, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim,
         "scale": float(scale if scale is not None else 1.0 / math.sqrt(dim))}
    if window is not None:
        m["mask"] = {"size": window}
    if rot:
        m["rot"] = {"dims": rot, "base": base}
        if scaling is not None:
            m["rot"]["scaling"] = dict(scaling)
    return m


def layer(mix, ff=96):
    return {"type": "attention", "mixer": mix, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


YARN = {"factor": 4.0, "original": 64, "fast": 16.0, "slow": 2.0}

# Sizes differ from layer to layer, and from one configuration to the next; where one configuration
# has values that coincide or are 1, another has not.
CONFIGS = {
    # looped middle stretch run three times, a layer without a feed-forward, value heads smaller than
    # key heads, a window shorter than a page, YaRN on part of the head
    "loop3": dict(vocab=131, width=64, scale=5.0, eps=1e-5, loop=(1, 3, 3), layers=[
        layer(mixer(4, 2, 32, 16, window=7, rot=16, scaling=YARN), ff=96),
        layer(mixer(4, 1, 32, 16, window=7, rot=16, scaling=YARN), ff=None),
        layer(mixer(2, 2, 48, 16, window=21, rot=48, base=500.0), ff=80),
        layer(mixer(4, 2, 32, 16, window=7, rot=16, scaling=YARN), ff=96)]),
    # no loop at all; value heads larger than key heads; as many kv heads as heads; a window larger
    # than a page (a ring of two pages); every dimension rotated, no scaling; one layer sees everything
    "plain": dict(vocab=97, width=48, scale=1.0, eps=1e-6, loop=None, layers=[
        layer(mixer(3, 3, 16, 48, window=70, rot=16), ff=64),
        layer(mixer(3, 1, 16, 48, window=None, rot=0), ff=64)]),
    # ones: one head, one pass, a window of one (a token sees itself only) and of exactly a page
    "ones": dict(vocab=64, width=32, scale=2.0, eps=1e-5, loop=(0, 2, 1), layers=[
        layer(mixer(1, 1, 64, 64, window=64, rot=8, scaling=dict(YARN, factor=1.5)), ff=48),
        layer(mixer(1, 1, 24, 40, window=1, rot=24), ff=48)]),
    # peaked attention (a large score scale), so that one key more or less in sight changes the result
    "sharp": dict(vocab=80, width=64, scale=4.0, eps=1e-5, loop=(0, 1, 2), layers=[
        layer(mixer(4, 2, 32, 32, window=9, rot=16, scaling=YARN, scale=1.5), ff=64),
        layer(mixer(4, 2, 32, 32, window=None, rot=32, scale=1.5), ff=64)]),
    # sizes that are multiples of little: heads of 40 and 80 (records are filled up), a rotated width of
    # 20 (not a multiple of 8), widths that no 16-byte access fits, four passes over a single layer
    "odd": dict(vocab=203, width=72, scale=0.5, eps=1e-4, loop=(0, 1, 4), layers=[
        layer(mixer(6, 3, 40, 24, window=100, rot=20, scaling=dict(YARN, factor=2.5, original=32)), ff=100),
        layer(mixer(3, 1, 80, 96, window=33, rot=80, base=123.0), ff=52),
        layer(mixer(5, 5, 18, 6, window=5, rot=6, scaling=dict(YARN, factor=16.0)), ff=None)]),
    # one layer that sees everything, without rotation: the tests make one far key stand out in it
    "far": dict(vocab=70, width=32, scale=3.0, eps=1e-5, loop=None, layers=[
        layer(mixer(2, 1, 16, 16, window=None, rot=0, scale=1.0), ff=48)]),
}


def spike_token(w, cfg, token):
    """Change drawn weights of a one-layer model so that every query looks at the key of ``token``
    wherever it stands: only that token has a component along feature 0, which alone feeds key
    dimension 0, and every query has a large constant along dimension 0.  After the head norms the
    score of that key exceeds all others by about 16 x scale."""
    s = cfg["embedding"]["scale"]
    w["embed"][:, 0] = 0.0
    w["embed"][token, 0] = 3.0 / s
    w["l0.norm1"][0], w["l0.norm1.b"][0] = 1.0, 0.0
    w["l0.mix.k"][0, :], w["l0.mix.k.b"][0] = 0.0, 0.0
    w["l0.mix.k"][0, 0] = 40.0
    d = cfg["layers"][0]["mixer"]["dim"]
    for h in range(cfg["layers"][0]["mixer"]["heads"]):
        w["l0.mix.q.b"][h * d] = 40.0
    w["l0.mix.q.norm"][0] = w["l0.mix.k.norm"][0] = 1.0


def config_dict(name):
    c = CONFIGS[name]
    d = {"architecture": "Supevik", "vocab": c["vocab"], "width": c["width"], "embedding": {"scale": c["scale"]},
         "norm": {"eps": c["eps"]}, "layers": json.loads(json.dumps(c["layers"]))}
    if c["loop"] is not None:
        d["loop"] = {"start": c["loop"][0], "stop": c["loop"][1], "times": c["loop"][2]}
    return d


def draw_weights(cfg, seed):
    """name -> bfloat16 tensor for every tensor of the configuration."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]
    out = {}

    def mat(name, rows, cols, gain=1.0):
        out[name] = (torch.randn(rows, cols, generator=g) * gain / math.sqrt(cols)).to(torch.bfloat16)

    def vec(name, n, mean, std):
        out[name] = (mean + std * torch.randn(n, generator=g)).to(torch.bfloat16)

    def norm(name):
        vec(name, W, 1.0, 0.2)
        vec(name + ".b", W, 0.0, 0.1)
        out[name + ".alpha"] = (0.7 + 0.3 * torch.rand((), generator=g)).to(torch.bfloat16)

    out["embed"] = (torch.randn(cfg["vocab"], W, generator=g) / cfg["embedding"]["scale"]).to(torch.bfloat16)
    if cfg.get("loop"):
        mat("loop.in", W, 2 * W, gain=1.2)
    for i, L in enumerate(cfg["layers"]):
        p, m = f"l{i}.", L["mixer"]
        H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
        norm(p + "norm1"), norm(p + "norm1b")
        mat(p + "mix.q", H * d, W), vec(p + "mix.q.b", H * d, 0.0, 0.3)
        mat(p + "mix.k", G * d, W), vec(p + "mix.k.b", G * d, 0.0, 0.3)
        mat(p + "mix.v", G * dv, W, gain=1.5), vec(p + "mix.v.b", G * dv, 0.0, 0.3)
        vec(p + "mix.q.norm", d, 1.0, 0.3), vec(p + "mix.k.norm", d, 1.0, 0.3)
        mat(p + "mix.g", H * dv, W, gain=1.5)
        mat(p + "mix.o", W, H * dv, gain=1.5)
        if L["mlp"]:
            ff = L["mlp"]["ff"]
            norm(p + "norm2"), norm(p + "norm2b")
            mat(p + "mlp.gate", ff, W, gain=1.5), mat(p + "mlp.up", ff, W, gain=1.5), mat(p + "mlp.down", W, ff, gain=1.5)
    norm("final.norm")
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
        w = draw_weights(cfg, seed)
        if edit_weights is not None:
            edit_weights(w, cfg)
        write_safetensors(os.path.join(d, "model.safetensors"), w)
        _folders[key] = d
    return _folders[key]


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()
