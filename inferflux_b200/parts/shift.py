"""Token shift: what a mixer reads is mixed with the token before it,

    s_t = h_t + (h_{t-1} - h_t) * mu        element by element, mu a weight of the layer

where ``h`` are the normed rows as they were before the mixing and ``h_{-1}``
is zero at the start of a sequence.  The last ``h`` of a step stays in the
request's state slot (float32), so a portion, or a single decoded token,
goes on from where the step before stopped.
"""
from __future__ import annotations

from typing import Any, Dict, List

import numpy as np
import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import VECTOR, WeightSpec
from .base import Part, RunInfo, StateNeed


class TokenShift(Part):
    """params: ``hidden``, ``weight_name`` (the leaf: weight is ``<prefix>.<weight_name>``).
    State: ``shift_prev`` float32 [hidden]."""

    family = "shift"
    describe_key = "token_rows"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        self.hidden = int(params["hidden"])
        self.mu: torch.Tensor = None

    @classmethod
    def _weight_name(cls, prefix, params) -> str:
        return ".".join(p for p in (prefix, params.get("weight_name", "shift")) if p)

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        return [WeightSpec(cls._weight_name(prefix, params), (int(params["hidden"]),), VECTOR, std=0.3)]

    @classmethod
    def state_needs(cls, params: Dict[str, Any]) -> List[StateNeed]:
        return [StateNeed("shift_prev", (int(params["hidden"]),), torch.float32)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.mu = tensors[self._weight_name(self.prefix, self.params)].to(torch.float32).contiguous()

    def describe_step(self, layout, put) -> torch.Tensor:
        """The entry of every row of the step."""
        return put(np.repeat(np.arange(layout.n_entries), layout.q_len[:layout.n_entries]))

    def forward(self, h32: torch.Tensor, ctx, run: RunInfo) -> torch.Tensor:
        """h32 float32 [N, hidden] -> the shifted rows in the engine's type; the
        run's state slot of every entry takes that entry's last row."""
        out = h32.new_empty(h32.shape, dtype=self.dtype)
        return ops.token_shift(h32, self.mu, run.states["shift_prev"], ctx.extras[self.describe_key], ctx.entry_q_start,
                               ctx.entry_q_len, ctx.entry_slot, out)


register_part("shift", "token_shift", TokenShift)
