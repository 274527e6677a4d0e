"""Typed configuration of the Supevik design, read from its own config.json keys.

A small decoder whose config.json lists its layers one by one: each entry names its mixer
(``type``), the mixer's sizes (``mixer``) and its feed-forward (``mlp``, or null for none).  A
stretch of the layers (``loop``: start, stop, times) may run several times in a row with the same
weights; every pass has cache entries of its own and starts by joining the stream with the
embedding output (tensor ``loop.in``).  Every layer is a "sandwich": Dynamic Tanh norms before and
after each sublayer.  Tensors of layer i start with ``l<i>.``.

Every size and every constant that may differ between models comes from config.json; nothing is
derived from one model's values.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .registry import Architecture, ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

ARCHITECTURE = "Supevik"


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
class RotScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class AttentionMixer:
    heads: int
    kv_heads: int
    dim: int                          # per-head query/key size
    vdim: int                         # per-head value size
    scale: float                      # factor on q . k
    window: Optional[int]             # position i sees j with 0 <= i - j < window; None: every earlier one
    rot_dims: int                     # rotated dimensions of each head (0: none)
    rot_base: float
    rot_scaling: Optional[RotScaling]


@dataclass(frozen=True)
class DenseMlp:
    ff: int


@dataclass(frozen=True)
class SupevikLayer:
    type: str
    mixer: AttentionMixer
    mlp: Optional[DenseMlp]


@dataclass(frozen=True)
class SupevikLoop:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class SupevikConfig:
    vocab: int
    width: int
    embedding_scale: float
    norm_eps: float
    layers: Tuple[SupevikLayer, ...]
    loop: Optional[SupevikLoop]
    raw: Tuple[Tuple[str, Any], ...] = ()      # config.json as it was read, for writing it out again

    @staticmethod
    def from_dict(cfg: Dict[str, Any]) -> "SupevikConfig":
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
            if kind != "attention":
                _fail(f"{where}: unknown mixer type {kind!r}; known: attention")
            m = _obj(e, "mixer", where)
            mw = where + ".mixer"
            heads, kv = _int(m, "heads", mw), _int(m, "kv_heads", mw)
            if heads % kv:
                _fail(f"{mw}: heads {heads} is not a multiple of kv_heads {kv}")
            dim, vdim = _int(m, "dim", mw), _int(m, "vdim", mw)
            window = None
            if m.get("mask") is not None:
                window = _int(_obj(m, "mask", mw), "size", mw + ".mask")
            rot_dims, rot_base, scaling = 0, 10000.0, None
            if m.get("rot") is not None:
                r = _obj(m, "rot", mw)
                rot_dims, rot_base = _int(r, "dims", mw + ".rot", low=0), _num(r, "base", mw + ".rot")
                if rot_dims % 2 or rot_dims > dim:
                    _fail(f"{mw}.rot: dims {rot_dims} must be even and at most dim {dim}")
                if r.get("scaling") is not None:
                    sc, sw = _obj(r, "scaling", mw + ".rot"), mw + ".rot.scaling"
                    scaling = RotScaling(_num(sc, "factor", sw), _num(sc, "original", sw), _num(sc, "fast", sw),
                                         _num(sc, "slow", sw))
            mixer = AttentionMixer(heads, kv, dim, vdim, _num(m, "scale", mw, positive=False), window, rot_dims,
                                   rot_base, scaling)
            mlp = None
            if e.get("mlp") is not None:
                ml = _obj(e, "mlp", where)
                if ml.get("kind") != "dense":
                    _fail(f"{where}.mlp: unknown kind {ml.get('kind')!r}; known: dense")
                mlp = DenseMlp(_int(ml, "ff", where + ".mlp"))
            layers.append(SupevikLayer(kind, mixer, mlp))
        loop = None
        if cfg.get("loop") is not None:
            lp = _obj(cfg, "loop")
            loop = SupevikLoop(_int(lp, "start", "loop", low=0), _int(lp, "stop", "loop", low=0), _int(lp, "times", "loop"))
            if not loop.start < loop.stop <= len(layers):
                _fail(f"loop: start {loop.start} and stop {loop.stop} must delimit layers of the {len(layers)}")
        return SupevikConfig(vocab, width, scale, eps, tuple(layers), loop, tuple(cfg.items()))

    def to_dict(self) -> Dict[str, Any]:
        if self.raw:
            return dict(self.raw)

        def mixer(m: AttentionMixer):
            d: Dict[str, Any] = {"heads": m.heads, "kv_heads": m.kv_heads, "dim": m.dim, "vdim": m.vdim, "scale": m.scale}
            if m.window is not None:
                d["mask"] = {"size": m.window}
            if m.rot_dims:
                d["rot"] = {"dims": m.rot_dims, "base": m.rot_base}
                if m.rot_scaling is not None:
                    s = m.rot_scaling
                    d["rot"]["scaling"] = {"factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            return d

        d: Dict[str, Any] = {
            "architecture": ARCHITECTURE, "vocab": self.vocab, "width": self.width,
            "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
            "layers": [{"type": l.type, "mixer": mixer(l.mixer),
                        "mlp": None if l.mlp is None else {"kind": "dense", "ff": l.mlp.ff}} for l in self.layers],
        }
        if self.loop is not None:
            d["loop"] = {"start": self.loop.start, "stop": self.loop.stop, "times": self.loop.times}
        return d

    def run_order(self):
        """[(layer, starts a pass?)] in the order the layers run: the layers before the loop, the
        looped stretch ``times`` times, the layers after it."""
        n = len(self.layers)
        if self.loop is None:
            return [(l, False) for l in range(n)]
        a, b = self.loop.start, self.loop.stop
        order = [(l, False) for l in range(a)]
        for _ in range(self.loop.times):
            order += [(l, l == a) for l in range(a, b)]
        return order + [(l, False) for l in range(b, n)]


def model_spec(c: SupevikConfig) -> ModelSpec:
    """Layer by layer into parts; tensor names are the checkpoint's."""
    W = c.width

    def norm(name: str) -> PartSpec:
        return PartSpec("dyt", {"size": W, "names": {"weight": "", "shift": ".b", "alpha": ".alpha"}}, name)

    layers, ignorable = [], []
    for i, L in enumerate(c.layers):
        p, m = f"l{i}.", L.mixer
        position: Dict[str, Any] = {"kind": "none"}
        if m.rot_dims:
            position = {"kind": "rotary", "theta": m.rot_base, "rotary_dim": m.rot_dims, "partial": m.rot_dims < m.dim}
            if m.rot_scaling is not None:
                s = m.rot_scaling
                position.update(kind="rotary_yarn", factor=s.factor, original=s.original, fast=s.fast, slow=s.slow)
        mixer = PartSpec(
            "gqa_attention",
            {
                "hidden_size": W, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                "value_dim": m.vdim, "qkv_bias": True, "window": m.window, "scale": m.scale,
                "qk_norm": {"eps": c.norm_eps}, "out_gate": True, "position": position,
                "names": {"q": "q", "k": "k", "v": "v", "o": "o", "q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b",
                          "q_norm": "q.norm", "k_norm": "k.norm", "gate": "g"},
            },
            p + "mix.",
        )
        if L.mlp is not None:
            ffn = PartSpec("dense_swiglu", {"hidden_size": W, "size": L.mlp.ff, "activation": "gelu_tanh",
                                            "names": {"gate": "gate", "up": "up", "down": "down"}}, p + "mlp.")
            layers.append(LayerSpec("sandwich", norm(p + "norm1"), mixer, norm(p + "norm2"), ffn,
                                    post1=norm(p + "norm1b"), post2=norm(p + "norm2b")))
        else:
            layers.append(LayerSpec("sandwich", norm(p + "norm1"), mixer, None, None, post1=norm(p + "norm1b")))
            ignorable += [p + "norm2", p + "norm2.*", p + "norm2b", p + "norm2b.*"]
    schedule = tuple(ScheduleEntry(l, run, True, join=0 if first else None)
                     for run, (l, first) in enumerate(c.run_order()))
    joins = ()
    if c.loop is not None:
        joins = (PartSpec("concat_linear", {"hidden_size": W, "names": {"weight": ""}}, "loop.in"),)
    return ModelSpec(
        architecture=ARCHITECTURE,
        hidden_size=W,
        vocab_size=c.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": W, "scale": c.embedding_scale,
                                               "names": {"weight": ""}}, "embed"),
        layers=tuple(layers),
        schedule=schedule,
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": c.vocab, "hidden_size": W, "tied": False, "names": {"weight": ""}}, "head"),
        ignorable=tuple(ignorable),
        joins=joins,
    )


register_architecture(Architecture(ARCHITECTURE, SupevikConfig.from_dict, model_spec, SupevikConfig.to_dict))
