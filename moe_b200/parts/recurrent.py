"""A recurrent mixer with a matrix-valued state per head and data-dependent decay (RWKV-style
time mixing).

With n_t the layer's normed input, n_(t-1) the previous token's (zeros before the first token)
and a blend x_s = n_t + (n_(t-1) - n_t) * mu_s for each of s in (r, k, v, g, w):
    r = Wr x_r, k = Wk x_k, v = Wv x_v           (heads x dim each)
    gate = silu(Wg x_g)
    w = exp(-exp(W2 tanh(W1 x_w) + w0))          (the decay, per head and key channel, in (0, 1))
per head, with a state S [dim, dim] that starts at zero:
    o_t = (S + diag(u) k_t v_t^T)^T r_t          (the bonus u acts on the current token only)
    S  <- diag(w_t) S + k_t v_t^T
and out = Wo ((o_t / rms(o_t over each head)) * norm_weight * gate).

What a sequence carries from step to step is of fixed size: n of its last token and S of every
head, both 32-bit (``state_request``).  The blends, the decay (its projections included), the scan
and the head norm are 32-bit arithmetic in both dtypes; the bfloat16 path rounds the blends that
feed the r, k, v and gate projections and the normed, gated output that feeds Wo.
"""
from __future__ import annotations

import os

import torch

from ..cache.kv import StateRequest
from ..ops import core
from ..ops.linear import grouped_linear, linear
from .base import Part, TensorSpec, register_part

_STREAMS = ("r", "k", "v", "g", "w")


class WKVMixer(Part):
    category, kind = "mixer", "wkv"
    graph_safe = True
    wants32 = True          # the blends are formed from the 32-bit normed input
    default_names = {"mu_r": "mu.r", "mu_k": "mu.k", "mu_v": "mu.v", "mu_g": "mu.g", "mu_w": "mu.w",
                     "r": "r", "k": "k", "v": "v", "g": "g", "w1": "w1", "w2": "w2", "w0": "w0", "u": "u",
                     "norm": "norm", "o": "o"}

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.hidden = int(p["hidden_size"])
        self.nh = int(p["num_heads"])
        self.hd = int(p["head_dim"])
        self.eps = float(p["eps"])                     # of the per-head norm of the output
        self.rank = p.get("decay_rank")                # None: read from the tensor's shape when bound
        if not (self.nh > 0 and 0 < self.hd <= 256):
            raise ValueError(f"wkv: {self.nh} heads of {self.hd}; the scan takes heads of up to 256")
        self.inner = self.nh * self.hd
        # up to this many tokens a step the blends' kernel forms the decay itself
        self.fused_decay_tokens = int(os.environ.get("MOE_B200_WKV_FUSED_DECAY_MAX", "64"))

    def tensors(self):
        n, W, I = self.names, self.hidden, self.inner
        rank = int(self.rank) if self.rank else 16
        t = {n["mu_" + s]: TensorSpec((W,), vector=True) for s in _STREAMS}
        for s in ("r", "k", "v", "g"):
            t[n[s]] = TensorSpec((I, W))
        t[n["w1"]] = TensorSpec((rank, W))
        t[n["w2"]] = TensorSpec((I, rank))
        t[n["w0"]] = TensorSpec((I,), vector=True)
        t[n["u"]] = TensorSpec((self.nh, self.hd), vector=True)
        t[n["norm"]] = TensorSpec((I,), init="ones", vector=True)
        t[n["o"]] = TensorSpec((W, I))
        return t

    def tensors_in(self, has):
        """The width of the decay's narrow projection is given by its tensors alone (unless the part
        was told ``decay_rank``): any extent is accepted there, and ``bind`` checks that the two agree."""
        t = self.tensors()
        if not self.rank:
            n = self.names
            t[n["w1"]] = TensorSpec((-1, self.hidden))
            t[n["w2"]] = TensorSpec((self.inner, -1))
        return t

    def describe(self):
        return f"wkv({self.nh} heads of {self.hd}, state {self.hd}x{self.hd} a head, decay by a rank-{self.rank or '?'} projection)"

    def kv_request(self):
        return None

    def state_request(self):
        # [the last token's normed input | S of every head]
        return StateRequest((self.hidden + self.nh * self.hd * self.hd,), torch.float32)

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        n = self.names
        self.mu = torch.stack([tensors[n["mu_" + s]].to(torch.float32) for s in _STREAMS]).contiguous()
        ws = [tensors[n[s]] for s in ("r", "k", "v", "g")]
        dt = ws[0].dtype if all(w.dtype == ws[0].dtype for w in ws) else torch.float32
        self.w_rkvg = torch.stack([w.to(dt) for w in ws]).contiguous()          # [4, inner, hidden]
        # the decay's two small projections stay 32-bit arithmetic in both dtypes
        w1 = tensors[n["w1"]]
        self.w1 = w1.to(torch.float32).contiguous()
        self.w1_3 = None
        if rt.is_bf16 and w1.dtype == torch.bfloat16 and self.hidden % 8 == 0:
            self.w1_3 = torch.cat([w1, w1, w1], dim=1).contiguous()
        w2 = tensors[n["w2"]].to(torch.float32)
        if self.w1.shape[0] != w2.shape[1]:
            raise ValueError(f"wkv: the decay's projections disagree on their inner width ({self.w1.shape[0]} and {w2.shape[1]})")
        self.w2t = w2.t().contiguous()                 # [rank, inner]: the decay kernel reads it by columns
        self.rank = int(self.w1.shape[0])
        self.w0 = tensors[n["w0"]].to(torch.float32).contiguous()
        self.u = tensors[n["u"]].to(torch.float32).contiguous()
        self.norm_w = tensors[n["norm"]].to(torch.float32).contiguous()
        self.wo = tensors[n["o"]].contiguous()
        self._offsets = {}

    def _group_offsets(self, T, device):
        """Row offsets [0, T, 2T, 3T, 4T] of the four blends in the grouped product."""
        o = self._offsets.get(T)
        if o is None:
            o = self._offsets[T] = torch.arange(0, 5 * T, T, dtype=torch.int32, device=device)[:5].contiguous()
        return o

    def forward(self, rt, h, batch, cache_view, state):
        T, W, I = batch.num_tokens, self.hidden, self.inner
        dev = h.f32.device
        # ---- the five blends (and the state's last-token row) -----------------------------------
        decay = torch.empty((T, I), dtype=torch.float32, device=dev)
        if self.rank <= core.WKV_FUSED_RANK and T <= self.fused_decay_tokens:
            # few tokens: the decay exp(-exp(W2 tanh(W1 x_w) + w0)) in the same launch, its blend in registers
            mixed = rt.empty((4, T, W))
            core.wkv_shift_mix(h.f32, self.mu, state, batch, mixed, decay=(self.w1, self.w2t, self.w0, decay))
        else:
            # many tokens: every block of the fused form would read both projections from L2 (measured
            # 833 us against 104 + 40 + 84 at 8,192 tokens of width 2,048).  The blend stays 32-bit; in
            # bfloat16 its narrow projection runs on the tensor cores without leaving 32-bit accuracy: the
            # blend as three bfloat16 terms (exact) against the (bfloat16, hence exact) rows, three times
            # side by side, accumulated in float32
            mixed = rt.empty((4, T, W))
            xw = torch.empty((T, W), dtype=torch.float32, device=dev)
            core.wkv_shift_mix(h.f32, self.mu, state, batch, mixed, last32=xw)
            low = torch.empty((T, self.rank), dtype=torch.float32, device=dev)
            done = False
            if self.w1_3 is not None:
                from ..ops import tc

                done = tc.gemm_tc(core.split3(xw), self.w1_3, low, bn=64, splits=8, status=rt.status)
            if not done:
                core.gemm_generic(xw, self.w1, low, status=rt.status)
            core.wkv_decay(low, self.w2t, self.w0, decay)
        # ---- r, k, v and the gate: one grouped product, a group a blend ---------------------------
        rkvg = grouped_linear(rt, mixed.view(4 * T, W), self.w_rkvg, self._group_offsets(T, dev), 4 * T)
        # ---- the scan over each sequence's tokens -----------------------------------------------
        o = torch.empty((T, I), dtype=torch.float32, device=dev)
        core.wkv_scan(rkvg[:T], rkvg[T:2 * T], rkvg[2 * T:3 * T], decay, self.u, state[:, W:], batch, o,
                      heads=self.nh, d=self.hd)
        y = rt.empty((T, I))
        core.wkv_finish(o, rkvg[3 * T:], self.norm_w, self.eps, batch, y, heads=self.nh, d=self.hd)
        return linear(rt, y, self.wo)


register_part("mixer", "wkv", WKVMixer)
