"""Position encodings as tables that the attention kernels read by position.

Rotary: inv_freq[j] = theta^(-2j/rd), angle = pos * inv_freq[j] in float
(qwen_triton/modules/rotary.py:14-26).  The table keeps float cos and sin; the reference rounds
them to the model dtype before use, this library does not.
"""
from __future__ import annotations

import torch

from .base import Runtime, register_position


@register_position("rope")
class RotaryTable:
    def __init__(self, params, runtime: Runtime) -> None:
        self.theta = float(params["theta"])
        self.rotary_dim = int(params["rotary_dim"])
        # which elements turn together: (i, i + rotary_dim / 2) as in the reference (kernels/rope.py:59-69), or
        # neighbours (2i, 2i + 1) with pairing = "interleaved"
        pairing = params.get("pairing", "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing {pairing!r} is neither 'half' nor 'interleaved'")
        self.interleaved = pairing == "interleaved"
        if self.rotary_dim % 2 or self.rotary_dim <= 0 or self.rotary_dim > int(params["head_dim"]):
            raise ValueError(f"rotary_dim={self.rotary_dim} must be even and within head_dim={params['head_dim']}")
        # "float64": frequencies and angles are formed in float64 and only cos and sin are rounded to float, so that an
        # angle of thousands of radians is not off by its float rounding; the default forms them in float as the
        # reference does
        self.angles = str(params.get("angles", "float32"))
        if self.angles not in ("float32", "float64"):
            raise ValueError(f"rotary angles in {self.angles!r} (float32 or float64)")
        self.runtime = runtime

    def key(self) -> tuple:
        return ("rope", self.theta, self.rotary_dim, self.angles)          # the table does not depend on the pairing

    def table(self, max_positions: int) -> torch.Tensor:
        """float32 [max_positions, rotary_dim]: cos in the first half of each row, sin in the second."""
        work = torch.float64 if self.angles == "float64" else torch.float32
        exponent = torch.arange(0, self.rotary_dim, 2, dtype=work) / self.rotary_dim
        inv_freq = 1.0 / (self.theta ** exponent)
        angles = torch.arange(max_positions, dtype=work)[:, None] * inv_freq[None, :]
        return torch.cat((angles.cos(), angles.sin()), dim=-1).to(torch.float32).contiguous().to(self.runtime.device)


@register_position("none")
class NoPosition:
    def __init__(self, params, runtime: Runtime) -> None:
        self.runtime = runtime

    def key(self) -> tuple:
        return ("none",)

    def table(self, max_positions: int):
        return None
