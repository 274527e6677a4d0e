"""Rotary position encoding.

inv_freq[i] = theta^(-2 i / dim) for i < dim/2, computed in float32 as the
reference does (src/spec.rs:89-96); the angle of position p is float32(p) *
inv_freq[i] (src/model.rs:326-328).  Pairs are half-split, (i, i + dim/2), unless the
part is given ``interleaved``: then pair i is (2i, 2i + 1).
"""
from __future__ import annotations

import math

import torch

from .base import Part, register_part


def rotary_inv_freq(theta: float, dim: int) -> torch.Tensor:
    # float32 exponent as in the reference, the power itself correctly rounded to float32
    i = torch.arange(dim // 2, dtype=torch.float32)
    expo = ((-2.0 * i) / torch.tensor(float(dim), dtype=torch.float32)).to(torch.float64)
    theta32 = torch.tensor(float(theta), dtype=torch.float32).to(torch.float64)
    return torch.pow(theta32, expo).to(torch.float32)


class RotaryEncoding(Part):
    category, kind = "position", "rotary"

    def __init__(self, spec):
        super().__init__(spec)
        self.theta = float(self.params["theta"])
        self.rotary_dim = int(self.params["rotary_dim"])
        if self.rotary_dim % 2:
            raise ValueError("rotary_dim must be even")
        self.interleaved = bool(self.params.get("interleaved", False))

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.inv_freq = rotary_inv_freq(self.theta, self.rotary_dim).to(rt.device)

    def describe(self):
        return (f"rope theta {self.theta:.0f}" + (f" on {self.rotary_dim} dims" if self.params.get("partial") else "")
                + (", pairs (2i, 2i+1)" if self.interleaved else ""))

    def rotary_table(self):
        """(inv_freq, rotary_dim): lets the mixer rotate inside its own kernel."""
        return self.inv_freq, self.rotary_dim

    def attention_scale(self) -> float:
        """Extra factor on 1/sqrt(head_dim); 1 without context extension (src/spec.rs:148-151)."""
        return 1.0

    def cos_sin_scale(self) -> float:
        """Factor on both cos and sin; 1 without context extension."""
        return 1.0


class YarnRotary(RotaryEncoding):
    """Rotary encoding with YaRN context extension.  With r rotated dimensions, base theta and
    f_i = theta^(-2i/r), let turn(t) = r ln(original / (2 pi t)) / (2 ln theta) be the (fractional)
    pair that makes t turns over the original context, lo = max(floor(turn(fast)), 0),
    hi = min(ceil(turn(slow)), r - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1).  Pair i
    turns at f_i / factor * ramp_i + f_i (1 - ramp_i): fast pairs keep their frequency, slow ones are
    interpolated.  cos and sin are multiplied by 0.1 ln(factor) + 1.  The table is formed in float64
    and rounded to float32 once."""

    kind = "rotary_yarn"

    def __init__(self, spec):
        super().__init__(spec)
        p = self.params
        self.factor, self.original = float(p["factor"]), float(p["original"])
        self.fast, self.slow = float(p["fast"]), float(p["slow"])
        if self.factor <= 0 or self.original <= 0 or self.fast <= 0 or self.slow <= 0 or self.theta <= 1:
            raise ValueError("rotary_yarn: factor, original, fast and slow must be positive and theta > 1")

    def frequencies(self) -> torch.Tensor:
        r = self.rotary_dim
        i = torch.arange(r // 2, dtype=torch.float64)
        f = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * i / r)

        def turn(t):
            return r * math.log(self.original / (2.0 * math.pi * t)) / (2.0 * math.log(self.theta))

        lo = max(math.floor(turn(self.fast)), 0)
        hi = min(math.ceil(turn(self.slow)), r - 1)
        ramp = ((i - lo) / max(hi - lo, 0.001)).clamp(0.0, 1.0)
        return (f / self.factor * ramp + f * (1.0 - ramp)).to(torch.float32)

    def bind(self, tensors, rt):
        Part.bind(self, tensors, rt)
        self.inv_freq = self.frequencies().to(rt.device)

    def describe(self):
        return f"rope theta {self.theta:.0f} on {self.rotary_dim} dims, YaRN x{self.factor:g} from {self.original:g}"

    def cos_sin_scale(self) -> float:
        return 0.1 * math.log(self.factor) + 1.0


class NoPositionEncoding(Part):
    category, kind = "position", "none"

    def describe(self):
        return "no position encoding"

    def rotary_table(self):
        return None, 0

    def attention_scale(self) -> float:
        return 1.0

    def cos_sin_scale(self) -> float:
        return 1.0


register_part("position", "rotary", RotaryEncoding)
register_part("position", "rotary_yarn", YarnRotary)
register_part("position", "none", NoPositionEncoding)
