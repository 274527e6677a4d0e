"""A plain, slow restatement of the Supevik design in float64 PyTorch on the CPU: one function per
mechanism, whole sequences, no cache.  It shares no code with the library; the tests compare the
library's kernels, cache and step function with it.

Notation: W weights stored [out, in] and applied as W n; n the input of a sublayer; p a position
counted from 0; d the per-head query/key size, dv the value size, r the rotated width.
"""
import json
import math
import os
import struct

import torch

F = torch.float64


# --------------------------------------------------------------------------- files
def read_safetensors(path):
    """name -> tensor (float tensors widened to float64, integer tables kept)."""
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        head = json.loads(f.read(n))
        data = f.read()
    kinds = {"BF16": torch.bfloat16, "F32": torch.float32, "F16": torch.float16, "I32": torch.int32, "F64": torch.float64}
    out = {}
    for name, rec in head.items():
        if name == "__metadata__":
            continue
        a, b = rec["data_offsets"]
        t = torch.frombuffer(bytearray(data[a:b]), dtype=kinds[rec["dtype"]]).reshape(rec["shape"])
        out[name] = t.to(F) if t.is_floating_point() else t
    return out


def read_model(folder):
    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    return cfg, read_safetensors(os.path.join(folder, "model.safetensors"))


# --------------------------------------------------------------------------- mechanisms
def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dynamic_tanh(x, w, name):
    """tanh(alpha x) * weight + shift; no statistic of x enters."""
    return torch.tanh(w[name + ".alpha"] * x) * w[name] + w[name + ".b"]


def unit_rms(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def yarn_frequencies(rot):
    """(frequency per pair [r/2], factor on cos and sin) of a rotation with optional YaRN scaling."""
    r, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(r // 2, dtype=F)
    f = base ** (-2.0 * i / r)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn(t):                      # the (fractional) pair that makes t turns over the original length
        return r * math.log(orig / (2.0 * math.pi * t)) / (2.0 * math.log(base))

    lo = max(math.floor(turn(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn(float(sc["slow"]))), r - 1)
    ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot):
    """x: [T, heads, d]; the first r dims of each head turn, pair (i, i + r/2); the rest pass."""
    r = int(rot["dims"])
    f, m = yarn_frequencies(rot)
    a = positions.to(F)[:, None] * f[None, :]
    cos, sin = (torch.cos(a) * m)[:, None, :], (torch.sin(a) * m)[:, None, :]
    u, v = x[..., : r // 2], x[..., r // 2: r]
    return torch.cat([u * cos - v * sin, v * cos + u * sin, x[..., r:]], dim=-1)


def windowed_softmax_attention(q, k, v, scale, window, start=0):
    """q: [T, H, d], k: [S, G, d], v: [S, G, dv]; query t stands at position start + t and sees key j
    with 0 <= (start + t) - j < window (every earlier key without a window)."""
    T, H, _ = q.shape
    S, G, dv = v.shape
    out = torch.zeros(T, H, dv, dtype=F)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        i = torch.arange(T)[:, None] + start
        j = torch.arange(S)[None, :]
        seen = (i - j >= 0)
        if window:
            seen &= (i - j < window)
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, g]
    return out


def attention_mixer(w, p, m, n, eps):
    """The attention mixer on the sublayer input n [T, width]; p is the tensor prefix '<layer>.mix'."""
    T = n.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = (n @ w[p + ".q"].T + w[p + ".q.b"]).reshape(T, H, d)
    k = (n @ w[p + ".k"].T + w[p + ".k.b"]).reshape(T, G, d)
    v = (n @ w[p + ".v"].T + w[p + ".v.b"]).reshape(T, G, dv)
    q, k = unit_rms(q, w[p + ".q.norm"], eps), unit_rms(k, w[p + ".k.norm"], eps)
    pos = torch.arange(T)
    if m.get("rot"):
        q, k = rotate(q, pos, m["rot"]), rotate(k, pos, m["rot"])
    window = int(m["mask"]["size"]) if m.get("mask") else None
    ctx = windowed_softmax_attention(q, k, v, float(m["scale"]), window).reshape(T, H * dv)
    ctx = ctx * torch.sigmoid(n @ w[p + ".g"].T)
    return ctx @ w[p + ".o"].T


def gated_mlp(w, p, n):
    return (gelu_tanh(n @ w[p + ".gate"].T) * (n @ w[p + ".up"].T)) @ w[p + ".down"].T


def layer_order(cfg):
    """[(layer, first of a pass?)] in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(l, False) for l in range(n)]
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    order = [(l, False) for l in range(a)]
    for _ in range(times):
        order += [(l, l == a) for l in range(a, b)]
    return order + [(l, False) for l in range(b, n)]


def forward(cfg, w, tokens, layers_out=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after every layer run."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    x0 = x.clone()
    for l, first in layer_order(cfg):
        L, p = cfg["layers"][l], f"l{l}"
        if first:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        assert L["type"] == "attention"
        x = x + dynamic_tanh(attention_mixer(w, p + ".mix", L["mixer"], dynamic_tanh(x, w, p + ".norm1"), eps), w, p + ".norm1b")
        if L.get("mlp"):
            assert L["mlp"]["kind"] == "dense"
            x = x + dynamic_tanh(gated_mlp(w, p + ".mlp", dynamic_tanh(x, w, p + ".norm2")), w, p + ".norm2b")
        if layers_out is not None:
            layers_out.append(x.clone())
    return dynamic_tanh(x, w, "final.norm") @ w["head"].T
