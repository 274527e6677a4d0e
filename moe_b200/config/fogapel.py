"""Typed configuration of the Fogapel design, read from its own config.json keys.

A small decoder whose config.json lists its layers one by one: each entry names its mixer
(``type``: "attention" or "wkv"), the mixer's sizes (``mixer``) and its feed-forward (``mlp``: a
dense gated one, routed experts with an optional shared expert, or null for none).  Every layer is
"parallel": one RMS norm whose output both sublayers read, each sublayer's output multiplied by a
per-channel factor (``ls1`` / ``ls2``) before the one residual sum.  The attention mixer has biases,
an optional short causal convolution on q, k and v, a rotation of pairs (2i, 2i + 1) on part of each
head, a weightless RMS norm of query and key heads after it, a given score scale, optionally
capped scores and chunks, and a softmax with a sink.  The recurrent mixer ("wkv") carries a
matrix-valued state per head.  Tensors of layer i start with ``l<i>.``.

Every size and every constant that may differ between models comes from config.json (or, for the
width of the recurrent mixer's decay projection, from the tensor's shape); nothing is derived from
one model's values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple, Union

from .registry import Architecture, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Fogapel"


def _fail(msg: str):
    raise ConfigError(f"{ARCHITECTURE}: {msg}")


def _obj(cfg, key, where="config.json") -> Dict[str, Any]:
    v = cfg.get(key)
    if not isinstance(v, dict):
        _fail(f"{where} lacks the object '{key}'")
    return v


def _int(cfg, key, where, low=1) -> int:
    v = cfg.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)) or int(v) != v:
        _fail(f"{where}: '{key}' must be an integer, got {v!r}")
    if int(v) < low:
        _fail(f"{where}: '{key}' must be at least {low}, got {v}")
    return int(v)


def _num(cfg, key, where, positive=True) -> float:
    v = cfg.get(key)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        _fail(f"{where}: '{key}' must be a number, got {v!r}")
    if positive and not float(v) > 0:
        _fail(f"{where}: '{key}' must be positive, got {v}")
    return float(v)


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int                          # per-head query/key size
    vdim: int                         # per-head value size
    scale: float                      # factor on q . k
    softcap: float                    # scores pass cap * tanh(s / cap); 0: no cap
    chunk: int                        # position i sees j <= i with i // chunk == j // chunk; 0: every earlier one
    taps: int                         # of the convolution on q, k, v; 0: none
    rot_dims: int                     # rotated dimensions of each head (0: none)
    rot_base: float


@dataclass(frozen=True)
class WkvMixer:
    heads: int
    dim: int


@dataclass(frozen=True)
class DenseMlp:
    ff: int
    limit: float


@dataclass(frozen=True)
class MoeMlp:
    experts: int
    top: int
    expert_ff: int
    shared_ff: int                    # 0: no shared expert


@dataclass(frozen=True)
class FogapelLayer:
    type: str
    mixer: Union[AttentionMixer, WkvMixer]
    mlp: Union[DenseMlp, MoeMlp, None]


@dataclass(frozen=True)
class FogapelConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[FogapelLayer, ...]
    raw: Tuple[Tuple[str, Any], ...] = ()      # config.json as it was read, for writing it out again

    @staticmethod
    def from_dict(cfg: Dict[str, Any]) -> "FogapelConfig":
        vocab, width = _int(cfg, "vocab", "config.json"), _int(cfg, "width", "config.json")
        scale = _num(_obj(cfg, "embedding"), "scale", "embedding", positive=False)
        eps = _num(_obj(cfg, "norm"), "eps", "norm")
        entries = cfg.get("layers")
        if not isinstance(entries, list) or not entries:
            _fail("'layers' must be a non-empty list")
        layers = []
        for i, e in enumerate(entries):
            where = f"layers[{i}]"
            if not isinstance(e, dict):
                _fail(f"{where} must be an object")
            kind = e.get("type")
            m = _obj(e, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                heads = _int(m, "heads", mw)
                kv = _int(m, "kv_heads", mw) if m.get("kv_heads") is not None else heads
                if heads % kv:
                    _fail(f"{mw}: heads {heads} is not a multiple of kv_heads {kv}")
                dim = _int(m, "dim", mw)
                vdim = _int(m, "vdim", mw) if m.get("vdim") is not None else dim
                chunk = _int(_obj(m, "mask", mw), "size", mw + ".mask") if m.get("mask") is not None else 0
                softcap = _num(m, "softcap", mw) if m.get("softcap") is not None else 0.0
                taps = _int(m, "conv", mw) if m.get("conv") is not None else 0
                rot_dims, rot_base = 0, 10000.0
                if m.get("rot") is not None:
                    r = _obj(m, "rot", mw)
                    rot_dims, rot_base = _int(r, "dims", mw + ".rot", low=0), _num(r, "base", mw + ".rot")
                    if rot_dims % 2 or rot_dims > dim:
                        _fail(f"{mw}.rot: dims {rot_dims} must be even and at most dim {dim}")
                mixer: Union[AttentionMixer, WkvMixer] = AttentionMixer(
                    heads, kv, dim, vdim, _num(m, "scale", mw, positive=False), softcap, chunk, taps, rot_dims, rot_base)
            elif kind == "wkv":
                mixer = WkvMixer(_int(m, "heads", mw), _int(m, "dim", mw))
            else:
                _fail(f"{where}: unknown mixer type {kind!r}; known: attention, wkv")
            mlp: Union[DenseMlp, MoeMlp, None] = None
            if e.get("mlp") is not None:
                ml, lw = _obj(e, "mlp", where), where + ".mlp"
                if ml.get("kind") == "dense":
                    mlp = DenseMlp(_int(ml, "ff", lw), _num(ml, "limit", lw))
                elif ml.get("kind") == "moe":
                    rt = _obj(ml, "router", lw)
                    experts, top = _int(rt, "experts", lw + ".router"), _int(rt, "top", lw + ".router")
                    if top > experts:
                        _fail(f"{lw}.router: top {top} exceeds experts {experts}")
                    shared = _int(_obj(ml, "shared", lw), "ff", lw + ".shared") if ml.get("shared") is not None else 0
                    mlp = MoeMlp(experts, top, _int(_obj(ml, "expert", lw), "ff", lw + ".expert"), shared)
                else:
                    _fail(f"{lw}: unknown kind {ml.get('kind')!r}; known: dense, moe")
            layers.append(FogapelLayer(kind, mixer, mlp))
        return FogapelConfig(vocab, width, scale, eps, tuple(layers), tuple(cfg.items()))

    def to_dict(self) -> Dict[str, Any]:
        if self.raw:
            return dict(self.raw)

        def mixer(m):
            if isinstance(m, WkvMixer):
                return {"heads": m.heads, "dim": m.dim}
            d: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.softcap:
                d["softcap"] = m.softcap
            if m.chunk:
                d["mask"] = {"size": m.chunk}
            if m.taps:
                d["conv"] = m.taps
            if m.rot_dims:
                d["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
            return d

        def mlp(f):
            if f is None:
                return None
            if isinstance(f, DenseMlp):
                return {"kind": "dense", "ff": f.ff, "limit": f.limit}
            d = {"kind": "moe", "router": {"experts": f.experts, "top": f.top}, "expert": {"ff": f.expert_ff}}
            if f.shared_ff:
                d["shared"] = {"ff": f.shared_ff}
            return d

        return {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer), "mlp": mlp(l.mlp)} for l in self.layers],
        }


def model_spec(c: FogapelConfig) -> ModelSpec:
    """Layer by layer into parts; tensor names are the checkpoint's."""
    W = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": W, "eps": c.norm_eps, "names": {"weight": ""}}, name)

    def scale(name: str) -> PartSpec:
        return PartSpec("channel_scale", {"size": W, "names": {"weight": ""}}, name)

    layers = []
    for i, L in enumerate(c.layers):
        p, m = f"l{i}.", L.mixer
        if isinstance(m, AttentionMixer):
            position: Dict[str, Any] = {"kind": "none"}
            if m.rot_dims:
                position = {"kind": "rotary", "theta": m.rot_base, "rotary_dim": m.rot_dims,
                            "partial": m.rot_dims < m.dim, "interleaved": True}
            mixer = PartSpec(
                "gqa_attention",
                {
                    "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                    "value_dim": m.vdim, "qkv_bias": True, "o_bias": True, "window": None, "chunk": m.chunk,
                    "scale": m.scale, "softcap": m.softcap, "sink": True, "unit_norm": {"eps": c.norm_eps},
                    "conv": {"taps": m.taps} if m.taps else None, "position": position,
                    "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                              "o_bias": "o.b", "q_conv": "q.conv", "k_conv": "k.conv", "v_conv": "v.conv"},
                },
                p + "mix.",
            )
        else:
            mixer = PartSpec("wkv", {"hidden_size": W, "num_heads": m.heads, "head_dim": m.dim, "eps": c.norm_eps},
                             p + "mix.")
        ffn = None
        if isinstance(L.mlp, DenseMlp):
            ffn = PartSpec("dense_swiglu", {"hidden_size": W, "size": L.mlp.ff, "activation": "clamped_sigmoid",
                                            "limit": L.mlp.limit, "names": {"gate": "gate", "up": "up", "down": "down"}},
                           p + "mlp.")
        elif isinstance(L.mlp, MoeMlp):
            f = L.mlp
            ffn = PartSpec("routed_experts",
                           {"hidden_size": W, "num_experts": f.experts, "top_k": f.top, "expert_size": f.expert_ff,
                            # the softmax over the chosen logits alone = the softmax over all, renormalised
                            "norm_topk_prob": True, "shared_size": f.shared_ff, "shared_gate": False, "router_bias": True,
                            "names": {"router": "router", "router_bias": "router.b", "expert_gate": "e{e}.gate",
                                      "expert_up": "e{e}.up", "expert_down": "e{e}.down", "shared_gate_proj": "shared.gate",
                                      "shared_up": "shared.up", "shared_down": "shared.down"}},
                           p + "mlp.")
        layers.append(LayerSpec("parallel", norm(p + "norm1"), mixer, None, ffn, scale1=scale(p + "ls1"),
                                scale2=scale(p + "ls2") if ffn is not None else None))
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=W,
        vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "scale": c.embedding_scale,
                                               "names": {"weight": ""}}, "embed"),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(l, l, True) for l in range(len(layers))),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False, "names": {"weight": ""}}, "head"),
        # a layer without a feed-forward may still carry the factor of one
        ignorable=tuple(f"l{i}.ls2" for i, L in enumerate(c.layers) if L.mlp is None),
    )


register_architecture(Architecture(ARCHITECTURE, FogapelConfig.from_dict, model_spec, FogapelConfig.to_dict))
