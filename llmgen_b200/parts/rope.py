"""Rotary position encoding: the cos/sin tables its mixer's kernel reads."""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from .base import Part
from .registry import register_position
from .spec import RopeSpec

_TABLES: Dict[Tuple, Tuple[torch.Tensor, torch.Tensor]] = {}


class Rope(Part):
    """cos/sin of pos / theta^(2i / rotary_dim), i in [0, rotary_dim/2), for every position:
    computed once on the host in float64 and kept as float32 [max_positions, rotary_dim/2]
    (the reference computes inverse frequencies and angles in f64 and stores f32 rows whose two
    halves are equal, src/backend/cpu/rope.zig:47-75; only one half is kept here).  Layers
    with the same spec share one pair of tables."""

    def __init__(self, spec: RopeSpec, weights, dtype, device):
        self.spec = spec
        key = (spec.rotary_dim, float(spec.theta), spec.max_positions, str(device))
        if key not in _TABLES:
            half = spec.rotary_dim // 2
            inv = 1.0 / torch.pow(torch.tensor(float(spec.theta), dtype=torch.float64),
                                  torch.arange(0, half, dtype=torch.float64) * 2.0 / spec.rotary_dim)
            ang = torch.arange(spec.max_positions, dtype=torch.float64)[:, None] * inv[None, :]
            _TABLES[key] = (ang.cos().to(torch.float32).to(device).contiguous(),
                            ang.sin().to(torch.float32).to(device).contiguous())
        self.cos, self.sin = _TABLES[key]
        self.rotary_dim = spec.rotary_dim
        self.pairing = spec.pairing
        self.max_positions = spec.max_positions

    def tables(self):
        return self.cos, self.sin


register_position("rope", Rope)
