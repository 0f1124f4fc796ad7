"""``latent_attention``: causal attention whose keys and values follow from one
cached latent vector per token, without positions.

    c_q = unit_rms(W_dq x) * w_q            q_h = (W_uq c_q)_h                 per head h, ``dim`` wide
    c   = unit_rms(W_dkv x) * w_kv          k_h = (W_uk c)_h,  v_h = (W_uv c)_h   (``dim`` and ``vdim`` wide)
    p_h(i, .) = softmax_j<=i( (q_h(i) . k_h(j)) * scale )
    o_h(i) = sigmoid(W_g x_i)_h * sum_j p_h(i, j) v_h(j)          y = W_o [o_1 .. o_H]

Only ``c`` is cached (one stream of ``kv_rank`` elements a token).  Keys and
values are never formed: the key projection is moved to the query,
``q_h . (Uk_h c) = (Uk_h^T q_h) . c``, and the value projection behind the
sum, ``sum_j p_j (Uv_h c_j) = Uv_h (sum_j p_j c_j)``, so the attention kernel
works on latents alone and all heads of a token read the same cached rows.
The three projections of x are stacked at load into one product whose sums
stay float32; both unit-rms norms, the cache write and the gates' sigmoid are
one kernel; scores, softmax and the weighted sums are float32.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional

import torch

from ..config.registry import register_part
from ..kernels import ops
from ..weights.loader import MATRIX, VECTOR, WeightSpec
from .base import CacheStream, KVNeed, Part, RunInfo
from .linear import Linear

QUERY_TILE = 16     # tokens per query tile of the latent attention kernel


@dataclass
class LatentStep:
    """The step's query tiles: int32 device tensors.  For the float32 kernel
    tiles of QUERY_TILE tokens; for the tensor-core kernel tiles of ``bm``
    (token, head) rows, which depend on the number of heads."""

    tile_entry: torch.Tensor
    tile_q0: torch.Tensor
    n_tiles: int
    bm: int
    row_tile_entry: torch.Tensor
    row_tile_row0: torch.Tensor
    n_row_tiles: int


class LatentAttention(Part):
    """params: ``hidden``, ``heads``, ``dim`` (of queries and keys), ``vdim``,
    ``kv_rank``, ``q_rank``, ``scale``, ``eps`` (of the two unit-rms norms),
    ``name`` (tensors ``<prefix>.<name>.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,g,o}``)."""

    family = "mixer"

    def __init__(self, params, prefix, dtype, device):
        super().__init__(params, prefix, dtype, device)
        p = params
        self.hidden, self.heads = int(p["hidden"]), int(p["heads"])
        self.describe_key = f"latent_attention/{self.heads}"     # layers with as many heads share a step's description
        self.dim, self.vdim = int(p["dim"]), int(p["vdim"])
        self.kv_rank, self.q_rank = int(p["kv_rank"]), int(p["q_rank"])
        self.scale, self.eps = float(p["scale"]), float(p["eps"])
        if not 1 <= self.kv_rank <= 1024:
            raise ValueError(f"kv_rank {self.kv_rank} is outside 1..1024")
        self.down: Linear = None            # [dq; dkv; g]
        self.uq: Linear = None
        self.uk_t: torch.Tensor = None      # [heads, kv_rank, dim]: a head's key projection, transposed
        self.uv: torch.Tensor = None        # [heads, vdim, kv_rank]
        self.o: Linear = None

    @classmethod
    def weight_specs(cls, params: Dict[str, Any], prefix: str) -> List[WeightSpec]:
        h, nh, d, vd, r, qr = (int(params[k]) for k in ("hidden", "heads", "dim", "vdim", "kv_rank", "q_rank"))
        n = lambda leaf: cls.full_name(prefix, params, leaf)
        return [WeightSpec(n("dq"), (qr, h), MATRIX), WeightSpec(n("dq.norm"), (qr,), VECTOR, init="one_plus_normal"),
                WeightSpec(n("uq"), (nh * d, qr), MATRIX),
                WeightSpec(n("dkv"), (r, h), MATRIX), WeightSpec(n("dkv.norm"), (r,), VECTOR, init="one_plus_normal"),
                WeightSpec(n("uk"), (nh * d, r), MATRIX), WeightSpec(n("uv"), (nh * vd, r), MATRIX),
                WeightSpec(n("g"), (nh, h), MATRIX), WeightSpec(n("o"), (h, nh * vd), MATRIX)]

    @classmethod
    def kv_need(cls, params: Dict[str, Any]) -> Optional[KVNeed]:
        return KVNeed((CacheStream("latent", 1, int(params["kv_rank"])),), None)

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = lambda leaf: self.full_name(self.prefix, self.params, leaf)
        mats = [tensors.pop(n(x)) for x in ("dq", "dkv", "g")]
        if len({m.dtype for m in mats}) > 1:
            mats = [m.float() for m in mats]
        self.down = Linear(torch.cat(mats, dim=0))
        del mats
        self.wq = tensors.pop(n("dq.norm")).to(torch.float32).contiguous()
        self.wkv = tensors.pop(n("dkv.norm")).to(torch.float32).contiguous()
        self.uq = Linear(tensors.pop(n("uq")))
        self.uk_t = tensors.pop(n("uk")).view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.uv = tensors.pop(n("uv")).view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.o = Linear(tensors.pop(n("o")))

    def describe_step(self, layout, put) -> LatentStep:
        tile_entry, tile_q0 = [], []
        for i in range(layout.n_entries):
            for q0 in range(0, int(layout.q_len[i]), QUERY_TILE):
                tile_entry.append(i), tile_q0.append(q0)
        small, large = ops.LATENT_MMA_TILES
        rows = [int(n) * self.heads for n in layout.q_len[:layout.n_entries]]
        bm = small if max(rows) <= small else large
        row_entry, row0 = [], []
        for i, n in enumerate(rows):
            for r in range(0, n, bm):
                row_entry.append(i), row0.append(r)
        return LatentStep(put(tile_entry), put(tile_q0), len(tile_entry), bm, put(row_entry), put(row0), len(row_entry))

    def _per_head(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        """x ``[N, heads, a]`` (a view), w ``[heads, b, a]`` -> float32 ``[N, heads, b]``
        (a view): head h's vectors times ``w[h]^T``."""
        n, width_out = x.shape[0], w.shape[1]
        if w.dtype == torch.float32:
            out = torch.empty((n, self.heads, width_out), dtype=torch.float32, device=x.device)
            for h in range(self.heads):
                ops.gemm_f32(x[:, h], w[h], None, out[:, h])
            return out
        # bfloat16 weights: one batched library product over the heads, float32 sums
        return torch.bmm(x.transpose(0, 1), w.transpose(1, 2), out_dtype=torch.float32).transpose(0, 1)

    def inner(self, x: torch.Tensor, ctx, run: RunInfo, position=None, out: torch.Tensor = None) -> torch.Tensor:
        """The gated heads ``[N, heads * vdim]`` that the output projection takes;
        writes this step's latents into the run's cache and attends over it."""
        n = x.shape[0]
        step: LatentStep = ctx.extras[self.describe_key]
        g = run.kv_group
        views, page_stride = ctx.kv.stream_views(g, run.kv_index)
        cache = views["latent"]
        p = self.down.forward(x, out_dtype=torch.float32)
        cq = torch.empty((n, self.q_rank), dtype=x.dtype, device=x.device)
        gate = torch.empty((n, self.heads), dtype=torch.float32, device=x.device)
        ops.latent_prep(p, self.wq, self.wkv, self.eps, self.q_rank, self.kv_rank, self.heads, cq, cache, page_stride,
                        ctx.page_size, ctx.slot_maps[g], gate)
        q = self.uq.forward(cq, out_dtype=x.dtype).view(n, self.heads, self.dim)
        q_lat = self._per_head(q, self.uk_t)                                   # float32 [N, heads, kv_rank]
        o_lat = torch.empty((self.heads, n, self.kv_rank), dtype=x.dtype, device=x.device).transpose(0, 1)
        if ops.attn_latent_mma_ok(self.kv_rank, cache):
            splits = ops.attn_latent_mma_splits(step.n_row_tiles, step.bm, self.kv_rank, ctx.max_ctx_len)
            ops.attn_latent_mma(q_lat, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.row_tile_entry,
                                step.row_tile_row0, step.n_row_tiles, step.bm, ctx.entry_q_start, ctx.entry_q_len,
                                ctx.entry_ctx_start, self.scale, splits)
        else:
            ops.attn_latent_paged(q_lat, o_lat, cache, page_stride, ctx.page_size, ctx.block_tables[g], step.tile_entry,
                                  step.tile_q0, step.n_tiles, ctx.entry_q_start, ctx.entry_q_len, ctx.entry_ctx_start,
                                  self.scale)
        heads = self._per_head(o_lat, self.uv)                                 # float32 [N, heads, vdim]
        if out is None:
            out = torch.empty((n, self.heads * self.vdim), dtype=x.dtype, device=x.device)
        return ops.gate_heads(heads, gate, out)

    @property
    def inner_width(self) -> int:
        return self.heads * self.vdim

    def forward(self, x: torch.Tensor, ctx, run: RunInfo, position) -> torch.Tensor:
        return self.o.forward(self.inner(x, ctx, run), out_dtype=torch.float32)


register_part("mixer", "latent_attention", LatentAttention)
