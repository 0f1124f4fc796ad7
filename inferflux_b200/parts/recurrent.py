"""Recurrent mixers.  ``mingru``: a gated recurrence whose gates read only the
current token,

    z_t = sigmoid(W_z x_t + b_z)            u_t = W_x x_t + b_x
    c_t = u_t + 1/2 where u_t >= 0,  sigmoid(u_t) where u_t < 0
    S_t = (1 - z_t) S_{t-1} + z_t c_t       element by element, float32, zero at the start of a sequence
    y_t = W_o (S_t * silu(W_g x_t))

The three input projections are stacked at load into one product whose sums
stay float32; gates, candidate and state are float32 in one scan kernel that
cuts long portions into segments (the recurrence is linear in S).  The state
lives in the request's state slot.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import Part, RunInfo, StateNeed
from .linear import Linear


@dataclass
class ScanStep:
    """The step cut into segments for the scan kernels: int32 device tensors."""

    seg_entry: torch.Tensor                   # [S] entry of each segment
    seg_t0: torch.Tensor                      # [S] its first token within the entry
    entry_first_seg: torch.Tensor             # [R] index of each entry's first segment
    n_segments: int
    multi: bool                               # some entry has more than one segment


class MinGRU(Part):
    """params: ``hidden``, ``width`` (of the state), ``name`` (tensors
    ``<prefix>.<name>.{z,z.b,x,x.b,g,o}``).  State: ``gru`` float32 [width]."""

    family = "mixer"
    describe_key = "mingru"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden, self.width = int(params["hidden"]), int(params["width"])
        self.zxg: Linear = None
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, w = int(params["hidden"]), int(params["width"])
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("z"), (w, h), MATRIX), WeightSpec(n("z.b"), (w,), VECTOR),
                WeightSpec(n("x"), (w, h), MATRIX), WeightSpec(n("x.b"), (w,), VECTOR),
                WeightSpec(n("g"), (w, h), MATRIX), WeightSpec(n("o"), (h, w), MATRIX)]

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        return [StateNeed("gru", (int(params["width"]),), torch.float32)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        mats = [tensors.pop(n(x)) for x in ("z", "x", "g")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.bias = torch.cat([tensors.pop(n("z.b")).float(), tensors.pop(n("x.b")).float()]).contiguous()   # added by the scan
        self.zxg = Linear(torch.cat(mats, dim=0))
        del mats
        self.o = Linear(tensors.pop(n("o")))

    def describe_step(self, layout, put) -> ScanStep:
        seg = ops.mingru_segment() if torch.device(self.device).type == "cuda" else 64
        seg_entry, seg_t0, first = [], [], []
        for i in range(layout.n_entries):
            first.append(len(seg_entry))
            for t0 in range(0, int(layout.q_len[i]), seg):
                seg_entry.append(i), seg_t0.append(t0)
        return ScanStep(put(seg_entry), put(seg_t0), put(first), len(seg_entry), len(seg_entry) > layout.n_entries)

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The gated states ``S_t * silu(g_t)``, ``[N, width]``, that the output projection takes."""
        step: ScanStep = ctx.extras[self.describe_key]
        proj = self.zxg.forward(x, out_dtype=torch.float32)
        if out is None:
            out = torch.empty((x.shape[0], self.width), dtype=x.dtype, device=x.device)
        return ops.mingru_scan(proj, self.bias, run.states["gru"], out, step.seg_entry, step.seg_t0, step.n_segments,
                               step.entry_first_seg, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries,
                               step.multi)

    @property
    def inner_width(self) -> int:
        return self.width

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position) -> torch.Tensor:
        return self.o.forward(self.inner(x, ctx, run), out_dtype=torch.float32)


register_part("mixer", "mingru", MinGRU)
