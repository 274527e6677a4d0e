"""A plain, slow restatement of the Fogapel design in float64 PyTorch on the CPU: one function per
mechanism, whole sequences, no cache and no state carried between calls.  It shares no code with
the library; the tests compare the library's kernels, cache, state and step function with it.

Notation: W weights stored [out, in] and applied as W n; n the input of both sublayers of a layer;
p a position counted from 0; H query heads on G key/value heads; d the per-head query/key size, dv
the value size, r the rotated width, C the size of an attention chunk; in the recurrent mixer S is
a head's state [d, d], w its decay per key channel and u its bonus for the current token.
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


# --------------------------------------------------------------------------- small functions
def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def silu(z):
    return z * torch.sigmoid(z)


# --------------------------------------------------------------------------- attention mixer
def short_convolution(u, taps_w):
    """u: [T, channels]; taps_w: [channels, taps].  y_t = sum_j taps_w[:, j] * u_(t - taps + 1 + j),
    with zeros before the first row."""
    T, _ = u.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, u.shape[1], dtype=F), u], dim=0)
    y = torch.zeros_like(u)
    for j in range(taps):
        y = y + padded[j:j + T] * taps_w[:, j]
    return y


def rotate_pairs(x, positions, r, base):
    """x: [T, heads, d]; dims (2i, 2i + 1), i < r/2, turn by the angle p * base^(-2i/r); the rest pass."""
    i = torch.arange(r // 2, dtype=F)
    a = positions.to(F)[:, None] * (base ** (-2.0 * i / r))[None, :]
    cos, sin = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    even, odd = x[..., 0:r:2], x[..., 1:r:2]
    out = x.clone()
    out[..., 0:r:2] = even * cos - odd * sin
    out[..., 1:r:2] = odd * cos + even * sin
    return out


def chunked_sink_attention(q, k, v, scale, softcap, chunk, sink=True):
    """q: [T, H, d], k: [T, G, d], v: [T, G, dv].  Query i sees key j <= i of its own chunk
    (i // chunk == j // chunk; every earlier key without chunks).  The scores pass
    cap * tanh(s / cap) if a cap is given; the weights are exp(s_j) / (1 + sum_j exp(s_j)) (the 1
    is the sink; ``sink=False`` leaves it out, to show how much it matters)."""
    T, H, _ = q.shape
    _, G, dv = v.shape
    out = torch.zeros(T, H, dv, dtype=F)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    seen = j <= i
    if chunk:
        seen &= (i // chunk) == (j // chunk)
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h] @ k[:, g].T) * scale
        if softcap:
            s = softcap * torch.tanh(s / softcap)
        e = torch.exp(s).masked_fill(~seen, 0.0)
        out[:, h] = (e / ((1.0 if sink else 0.0) + e.sum(-1, keepdim=True))) @ v[:, g]
    return out


def attention_mixer(w, p, m, n, eps):
    """The attention mixer on n [T, width]; p is the tensor prefix '<layer>.mix'."""
    T = n.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = n @ w[p + ".q"].T + w[p + ".q.b"]
    k = n @ w[p + ".k"].T + w[p + ".k.b"]
    v = n @ w[p + ".v"].T + w[p + ".v.b"]
    if m.get("conv"):
        q, k, v = (short_convolution(t, w[p + "." + s + ".conv"]) for t, s in ((q, "q"), (k, "k"), (v, "v")))
    q, k, v = q.reshape(T, H, d), k.reshape(T, G, d), v.reshape(T, G, dv)
    pos = torch.arange(T)
    if m.get("rot"):
        r, base = int(m["rot"]["dims"]), float(m["rot"]["base"])
        q, k = rotate_pairs(q, pos, r, base), rotate_pairs(k, pos, r, base)
    q, k = unit_rms(q, eps), unit_rms(k, eps)
    chunk = int(m["mask"]["size"]) if m.get("mask") else 0
    ctx = chunked_sink_attention(q, k, v, float(m["scale"]), float(m.get("softcap") or 0.0), chunk)
    return ctx.reshape(T, H * dv) @ w[p + ".o"].T + w[p + ".o.b"]


# --------------------------------------------------------------------------- recurrent mixer
def wkv_mixer(w, p, m, n, eps, trace=None):
    """The recurrent mixer on n [T, width].  Every projection reads its own blend of the token's
    input and the previous token's; per head o_t = (S + diag(u) k_t v_t^T)^T r_t and then
    S <- diag(w_t) S + k_t v_t^T."""
    T, _ = n.shape
    H, d = int(m["heads"]), int(m["dim"])
    prev = torch.cat([torch.zeros(1, n.shape[1], dtype=F), n[:-1]], dim=0)

    def blend(s):
        return n + (prev - n) * w[p + ".mu." + s]

    r = (blend("r") @ w[p + ".r"].T).reshape(T, H, d)
    k = (blend("k") @ w[p + ".k"].T).reshape(T, H, d)
    v = (blend("v") @ w[p + ".v"].T).reshape(T, H, d)
    gate = silu(blend("g") @ w[p + ".g"].T)
    decay = torch.exp(-torch.exp(torch.tanh(blend("w") @ w[p + ".w1"].T) @ w[p + ".w2"].T + w[p + ".w0"])).reshape(T, H, d)
    u = w[p + ".u"]
    out = torch.zeros(T, H, d, dtype=F)
    S = torch.zeros(H, d, d, dtype=F)
    for t in range(T):
        kv = k[t][:, :, None] * v[t][:, None, :]
        out[t] = torch.einsum("hi,hij->hj", r[t], S + u[:, :, None] * kv)
        S = decay[t][:, :, None] * S + kv
    if trace is not None:
        trace.append(S.clone())
    out = unit_rms(out, eps).reshape(T, H * d) * w[p + ".norm"] * gate
    return out @ w[p + ".o"].T


# --------------------------------------------------------------------------- feed-forwards
def clamped_glu(w, p, n, limit):
    """g = min(Wg n, limit), u = clamp(Wu n, -limit, limit); Wd (g sigmoid(1.702 g) (u + 1))."""
    g = (n @ w[p + ".gate"].T).clamp(max=limit)
    u = (n @ w[p + ".up"].T).clamp(min=-limit, max=limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + ".down"].T


def silu_glu(w, p, n):
    return (silu(n @ w[p + ".gate"].T) * (n @ w[p + ".up"].T)) @ w[p + ".down"].T


def routed_experts(w, p, mlp, n, picks=None, forced=None, margins=None):
    """Every token takes the ``top`` experts of largest router logit, weighted by the softmax over
    those logits alone; a shared expert, if any, is added for every token.  ``picks`` (a list)
    receives the chosen experts [T, top]; ``forced`` replaces the choice (the weights still come from
    the logits), for comparisons with an implementation whose near-ties fall the other way;
    ``margins`` (a list) then receives, for every token whose forced choice differs from the free one,
    the gap between the logits that were swapped as a fraction of the logits' root mean square."""
    E, top = int(mlp["router"]["experts"]), int(mlp["router"]["top"])
    z = n @ w[p + ".router"].T + w[p + ".router.b"]
    free = torch.topk(z, top, dim=-1).indices
    idx = free if forced is None else torch.as_tensor(forced, dtype=torch.long)
    if forced is not None and margins is not None:
        rms = float(z.pow(2).mean().sqrt().clamp(min=1e-30))
        for t in range(z.shape[0]):
            a, b = set(free[t].tolist()), set(idx[t].tolist())
            if a != b:
                margins.append((max(float(z[t, e]) for e in a - b) - min(float(z[t, e]) for e in b - a)) / rms)
    if picks is not None:
        picks.append(idx.clone())
    weight = torch.softmax(torch.gather(z, 1, idx), dim=-1)
    out = torch.zeros_like(n)
    for e in range(E):
        rows, slot = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            out[rows] += weight[rows, slot][:, None] * silu_glu(w, f"{p}.e{e}", n[rows])
    if mlp.get("shared"):
        out = out + silu_glu(w, p + ".shared", n)
    return out


# --------------------------------------------------------------------------- the model
def forward(cfg, w, tokens, layers_out=None, picks=None, forced=None, margins=None):
    """Logits [T, vocab] of one whole sequence; ``layers_out`` (a list) receives the stream after
    every layer; ``picks`` / ``forced`` / ``margins``: the routed layers' choices, in layer order
    (see ``routed_experts``)."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)] * float(cfg["embedding"]["scale"])
    forced = list(forced) if forced is not None else None
    for l, L in enumerate(cfg["layers"]):
        p = f"l{l}"
        n = unit_rms(x, eps) * w[p + ".norm1"]
        if L["type"] == "attention":
            a = attention_mixer(w, p + ".mix", L["mixer"], n, eps)
        elif L["type"] == "wkv":
            a = wkv_mixer(w, p + ".mix", L["mixer"], n, eps)
        else:
            raise ValueError(L["type"])
        delta = a * w[p + ".ls1"]
        mlp = L.get("mlp")
        if mlp:
            if mlp["kind"] == "dense":
                b = clamped_glu(w, p + ".mlp", n, float(mlp["limit"]))
            elif mlp["kind"] == "moe":
                b = routed_experts(w, p + ".mlp", mlp, n, picks, forced.pop(0) if forced is not None else None, margins)
            else:
                raise ValueError(mlp["kind"])
            delta = delta + b * w[p + ".ls2"]
        x = x + delta
        if layers_out is not None:
            layers_out.append(x.clone())
    return (unit_rms(x, eps) * w["final.norm"]) @ w["head"].T
