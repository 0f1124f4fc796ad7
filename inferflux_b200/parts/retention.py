"""``retention``: linear attention with a fixed decay per head, no softmax and no denominator,

    S_t = decay_h S_{t-1} + k_t v_t^T        S: [dim x vdim] per head, float32, zero at the start of a sequence
    o_t = S_t^T q_t

with q and k rotated by the layer's position table (first ``rot_dims`` dimensions, pairs in ``half``s or
``interleaved``), k then scaled by ``dim^-1/2``; each head's o is brought to unit root mean square (no weight),
the heads side by side are multiplied by silu(g) and projected.  q, k, v and g are one stacked projection whose
sums stay float32; rotation, state, scores and the norm are float32 in either engine type.  The state lives in
the request's state slot; portions are cut into segments that run side by side (the recurrence is linear in S).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, WeightSpec
from .base import Part, RunInfo, StateNeed
from .linear import Linear


@dataclass
class RetentionStep:
    """The step cut into segments for the scan kernels: int32 device tensors."""

    seg_entry: torch.Tensor
    seg_t0: torch.Tensor
    entry_first_seg: torch.Tensor
    n_segments: int
    multi: bool                               # some entry has more than one segment


class Retention(Part):
    """params: ``hidden``, ``heads``, ``dim``, ``vdim``, ``decay`` (one number per head), ``rot_dims``,
    ``rot_layout``, ``eps`` (of the per-head norm), ``name`` (tensors ``<prefix>.<name>.{q,k,v,g,o}``).
    State: ``retention`` float32 ``[heads, dim, vdim]``.
    Position: a pair ``(cos, sin)`` of float32 ``[N, rot_dims / 2]`` tensors."""

    family = "mixer"
    describe_key = "retention_segments"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.rot_dims = int(p.get("rot_dims") or 0)
        self.layout = ops.ROT_INTERLEAVED if p.get("rot_layout", "half") == "interleaved" else ops.ROT_HALF
        self.eps = float(p["eps"])
        decay = [float(d) for d in p["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"retention: {len(decay)} decays for {self.heads} heads")
        if self.rot_dims % 2 or self.rot_dims > self.dim:
            raise ValueError(f"rot_dims {self.rot_dims} must be even and at most dim {self.dim}")
        if not 1 <= self.dim <= 256:
            raise ValueError("retention: dim must be within 1..256")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=device)
        self.qkvg: Linear = None
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, d, vd = (int(params[k]) for k in ("hidden", "heads", "dim", "vdim"))
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("q"), (nh * d, h), MATRIX), WeightSpec(n("k"), (nh * d, h), MATRIX),
                WeightSpec(n("v"), (nh * vd, h), MATRIX), WeightSpec(n("g"), (nh * vd, h), MATRIX),
                WeightSpec(n("o"), (h, nh * vd), MATRIX)]

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        return [StateNeed("retention", (int(params["heads"]), int(params["dim"]), int(params["vdim"])), torch.float32)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        mats = [tensors.pop(n(x)) for x in ("q", "k", "v", "g")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.qkvg = Linear(torch.cat(mats, dim=0))
        del mats
        self.o = Linear(tensors.pop(n("o")))

    def describe_step(self, layout, put) -> RetentionStep:
        seg = ops.retention_segment() if torch.device(self.device).type == "cuda" else 32
        seg_entry, seg_t0, first = [], [], []
        for i in range(layout.n_entries):
            first.append(len(seg_entry))
            for t0 in range(0, int(layout.q_len[i]), seg):
                seg_entry.append(i), seg_t0.append(t0)
        return RetentionStep(put(seg_entry), put(seg_t0), put(first), len(seg_entry), len(seg_entry) > layout.n_entries)

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position, out: torch.Tensor = None) -> torch.Tensor:
        """The normed, gated heads ``[N, heads * vdim]`` that the output projection takes."""
        n = x.shape[0]
        step: RetentionStep = ctx.extras[self.describe_key]
        proj = self.qkvg.forward(x, out_dtype=torch.float32)
        hd, hv = self.heads * self.dim, self.heads * self.vdim
        if self.rot_dims:
            if not (isinstance(position, (tuple, list)) and len(position) == 2 and 2 * position[0].shape[1] == self.rot_dims):
                raise TypeError("retention takes its position as a pair (cos, sin) of [N, rot_dims / 2] float32 tensors; "
                                "the layer's position encoding gave something else")
            ops.rotate_heads(proj, 0, 2 * self.heads, self.dim, position[0], position[1], self.layout)   # q and k heads
        o = torch.empty((n, hv), dtype=torch.float32, device=x.device)
        ops.retention_scan(proj, 0, hd, 2 * hd, self.heads, self.dim, self.vdim, self.decay, float(self.dim) ** -0.5,
                           run.states["retention"], step.seg_entry, step.seg_t0, step.n_segments, step.entry_first_seg,
                           ctx.entry_q_start, ctx.entry_q_len, ctx.entry_slot, ctx.n_entries, step.multi, o)
        if out is None:
            out = torch.empty((n, hv), dtype=x.dtype, device=x.device)
        return ops.retention_finish(o, proj[:, 2 * hd + hv:], out, self.heads, self.vdim, self.eps)

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position):
        return self.o.forward(self.inner(x, ctx, run, position), allow_partials=True, f32_sums=True, out_dtype=torch.float32)


register_part("mixer", "retention", Retention)
