"""Feed-forward parts: experts chosen by a router, and a dense gated unit.

Routed experts (src/minimax.rs:88-126): router logits z = act W_r^T in float32;
score s = sigmoid(z); choice c = s + bias (the bias decides only who is picked);
the ``top_k`` largest c, ties to the lower id; weights s / sum of the picked s;
each picked expert computes silu(x W1^T) * (x W3^T) then W2; the outputs are
summed with their weights in rank order.  The experts' matrices are stacked:
``w13`` [E, 2I, d] holds each expert's gate rows then its up rows, ``w2`` [E, d, I].
Rows are grouped by expert with a counting sort on the device, so no step of the
feed-forward waits for the host.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import FeedForward, WeightedRows, register_part
from .linear import linear

TILE_ROWS = 32        # rows of one expert that a block of the expert kernels takes
# Above this many rows per expert (on average) a step's expert products run on tcgen05: tiles of 32 rows and more
# read an expert's weights once however its rows are spread, at the speed of the memory.  Measured on a B200 at
# MiniMax-M2's sizes: the streaming kernel with tiles of 8 rows is as fast while no expert gets more than 8 rows
# (a decode step of 64 sequences, two rows per expert on average: 1,087 against 1,094 us a layer), but a prompt's
# tokens crowd on fewer experts, and every tile beyond an expert's first reads its weights again (a prompt of 64
# tokens: 525 against 419 us a layer, of 256: 1,400 against 617).
TENSOR_CORE_ROWS_PER_EXPERT = {"decode": 4.0, "prompt": 1.0}


class RoutedExperts(FeedForward):
    wants_float32_input = True          # the router reads the normed rows before they are rounded
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_experts = int(a["num_experts"])
        self.top_k = int(a["top_k"])
        self.expert_width = int(a["expert_width"])
        if a.get("score", "sigmoid") != "sigmoid":
            raise ValueError(f"router score {a.get('score')!r}: only 'sigmoid' is built")
        self.choice_bias = bool(a.get("choice_bias", False))
        self.renormalize = bool(a.get("renormalize", True))
        self.routed_scale = float(a.get("routed_scale", 1.0))
        if not 1 <= self.top_k <= self.num_experts:
            raise ValueError(f"top_k {self.top_k} is outside 1..{self.num_experts} experts")
        self.router: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self.w13: Optional[torch.Tensor] = None
        self.w2: Optional[torch.Tensor] = None
        self.on_route = None              # called with the picked ids [T, k] of every step (for measurements)
        # int32 [rows >= T, k] on the device, or None: when set, every step copies its picked ids into the first
        # T rows.  The copy is a device operation, so unlike ``on_route`` it also happens in a recorded step.
        self.route_log: Optional[torch.Tensor] = None

    def _expert_needs(self, e: int) -> tuple[TensorNeed, TensorNeed, TensorNeed]:
        d, i = self.hidden_size, self.expert_width
        return (TensorNeed(self.name_of("w_gate").format(e=e), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_up").format(e=e), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_down").format(e=e), (d, i), MATRIX, "normal"))

    def tensor_needs(self):
        needs = [TensorNeed(self.name_of("router"), (self.num_experts, self.hidden_size), VECTOR, "normal")]
        if self.choice_bias:
            needs.append(TensorNeed(self.name_of("choice_bias"), (self.num_experts,), VECTOR, "bias"))
        for e in range(self.num_experts):
            needs.extend(self._expert_needs(e))
        return needs

    def load(self, source: TensorSource) -> None:
        d, i, n = self.hidden_size, self.expert_width, self.num_experts
        self.router = source.fetch(TensorNeed(self.name_of("router"), (n, d), VECTOR, "normal"))
        if self.choice_bias:
            self.bias = source.fetch(TensorNeed(self.name_of("choice_bias"), (n,), VECTOR, "bias"))
        for e in range(n):
            gate, up, down = (source.fetch(need) for need in self._expert_needs(e))
            if self.w13 is None:
                self.w13 = torch.empty((n, 2 * i, d), dtype=gate.dtype, device=gate.device)
                self.w2 = torch.empty((n, d, i), dtype=gate.dtype, device=gate.device)
            self.w13[e, :i].copy_(gate)
            self.w13[e, i:].copy_(up)
            self.w2[e].copy_(down)

    # -- one step --------------------------------------------------------------------------------------
    def logits(self, ctx, act32: torch.Tensor) -> torch.Tensor:
        """Router logits: float32 rows, float32 weight, no rounding.  Few rows: this library's kernel (the
        library's float32 product is slow on a handful of rows); many: the library."""
        tokens = act32.shape[0]
        if tokens <= ops.ROUTER_LOGITS_TOKENS and self.hidden_size % 4 == 0:
            out = ctx.buffer("experts.logits", (tokens, self.num_experts), torch.float32)
            ops.router_logits(act32, self.router, out)
            return out
        return linear(act32, self.router)

    def route(self, ctx, act32: torch.Tensor):
        tokens = act32.shape[0]
        logits = self.logits(ctx, act32)
        ids = ctx.buffer("experts.ids", (tokens, self.top_k), torch.int32)
        weights = ctx.buffer("experts.weights", (tokens, self.top_k), torch.float32)
        ops.router_topk(logits, self.bias, self.top_k, self.renormalize, self.routed_scale, ids, weights)
        return ids, weights

    def streams(self) -> bool:
        """Whether the tensor-core streaming kernel takes this part's sizes (bfloat16, sizes in steps of 32)."""
        return (self.dtype == torch.bfloat16 and self.hidden_size % 32 == 0 and self.expert_width % 32 == 0)

    def on_tensor_cores(self, assignments: int, decode: bool = False) -> bool:
        """Whether the tcgen05 kernel runs the step: bfloat16, sizes in steps of 128, and enough rows per
        expert that the products, not the weights alone, are the work."""
        return (self.dtype == torch.bfloat16 and self.hidden_size % 128 == 0 and self.expert_width % 128 == 0
                and assignments > TENSOR_CORE_ROWS_PER_EXPERT["decode" if decode else "prompt"] * self.num_experts)

    def tile_rows(self, assignments: int, decode: bool = False) -> int:
        """Rows of one expert that one block takes: few when experts get few rows each, so that no block
        carries accumulators it does not need; enough that most experts fit one tile when they get many."""
        per_expert = assignments / self.num_experts
        if self.on_tensor_cores(assignments, decode):
            return next((t for t in (32, 64, 128, 256) if t >= 1.3 * per_expert), 256)
        if not self.streams():
            return TILE_ROWS
        return 8 if per_expert <= 4 else 16 if per_expert <= 12 else 32

    def plan(self, ctx, ids: torch.Tensor):
        tokens = ids.shape[0]
        n = tokens * self.top_k
        chunks = (n + 1023) // 1024
        tile_rows = self.tile_rows(n, ctx.is_decode)
        max_tiles = (n + tile_rows - 1) // tile_rows + min(self.num_experts, n)
        p = {
            "counts": ctx.buffer("experts.counts", (chunks * self.num_experts,), torch.int32),
            "offsets": ctx.buffer("experts.offsets", (self.num_experts + 1,), torch.int32),
            "sorted_token": ctx.buffer("experts.sorted_token", (n,), torch.int32),
            "row_of_assign": ctx.buffer("experts.row_of_assign", (n,), torch.int32),
            "tile_expert": ctx.buffer("experts.tile_expert", (max_tiles,), torch.int32),
            "tile_row0": ctx.buffer("experts.tile_row0", (max_tiles,), torch.int32),
            "num_tiles": ctx.buffer("experts.num_tiles", (1,), torch.int32),
            "max_tiles": max_tiles,
            "rows": n,
            "tile_rows": tile_rows,
        }
        ops.expert_plan(ids, self.num_experts, tile_rows, p["counts"], p["offsets"], p["sorted_token"],
                        p["row_of_assign"], p["tile_expert"], p["tile_row0"], p["num_tiles"])
        return p

    def experts(self, ctx, act: torch.Tensor, p) -> torch.Tensor:
        """y [N, d] float32: the output of its expert for every (token, rank), in expert-sorted order."""
        hidden = ctx.buffer("experts.hidden", (p["rows"], self.expert_width), self.dtype)
        y = ctx.buffer("experts.y", (p["rows"], self.hidden_size), torch.float32)
        if self.on_tensor_cores(p["rows"], ctx.is_decode):
            gathered = ctx.buffer("experts.gathered", (p["rows"], self.hidden_size), self.dtype)
            ops.gather_rows(act, p["sorted_token"], gathered)
            ops.expert_gemm_tc(self.w13, gathered, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                               p["max_tiles"], p["tile_rows"], hidden, paired=True)
            ops.expert_gemm_tc(self.w2, hidden, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                               p["max_tiles"], p["tile_rows"], y, paired=False)
            return y
        if self.streams() and ops.weight_stream_takes(self.expert_width, self.hidden_size, paired=True) \
                and ops.weight_stream_takes(self.hidden_size, self.expert_width, paired=False):
            ops.weight_stream(self.w13, act, p["sorted_token"], p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                              p["max_tiles"], p["tile_rows"], hidden, paired=True)
            # the second product's lists are the first one's: its weights may be on their way while the first still runs
            ops.weight_stream(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                              p["max_tiles"], p["tile_rows"], y, paired=False, lists_final=True)
            return y
        if self.streams():
            tiles = min(p["rows"], self.num_experts)           # about as many tiles as experts that got rows
            ops.expert_gemm_mma(self.w13, act, p["sorted_token"], p["tile_expert"], p["tile_row0"], p["num_tiles"],
                                p["offsets"], p["max_tiles"], p["tile_rows"], hidden, paired=True,
                                **ops.stream_shape(tiles, self.expert_width, self.hidden_size, p["tile_rows"], paired=True))
            ops.expert_gemm_mma(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                                p["max_tiles"], p["tile_rows"], y, paired=False,
                                **ops.stream_shape(tiles, self.hidden_size, self.expert_width, p["tile_rows"]))
            return y
        ops.expert_gemm_generic(self.w13, act, p["sorted_token"], p["tile_expert"], p["tile_row0"], p["num_tiles"],
                                p["offsets"], p["max_tiles"], hidden, paired=True)
        ops.expert_gemm_generic(self.w2, hidden, None, p["tile_expert"], p["tile_row0"], p["num_tiles"], p["offsets"],
                                p["max_tiles"], y, paired=False)
        return y

    def route_and_plan(self, ctx, act32: torch.Tensor):
        """For steps of few tokens: choice and lists in one launch."""
        tokens = act32.shape[0]
        n = tokens * self.top_k
        tile_rows = self.tile_rows(n, ctx.is_decode)
        max_tiles = (n + tile_rows - 1) // tile_rows + min(self.num_experts, n)
        ids = ctx.buffer("experts.ids", (tokens, self.top_k), torch.int32)
        weights = ctx.buffer("experts.weights", (tokens, self.top_k), torch.float32)
        p = {
            "offsets": ctx.buffer("experts.offsets", (self.num_experts + 1,), torch.int32),
            "sorted_token": ctx.buffer("experts.sorted_token", (n,), torch.int32),
            "row_of_assign": ctx.buffer("experts.row_of_assign", (n,), torch.int32),
            "tile_expert": ctx.buffer("experts.tile_expert", (max_tiles,), torch.int32),
            "tile_row0": ctx.buffer("experts.tile_row0", (max_tiles,), torch.int32),
            "num_tiles": ctx.buffer("experts.num_tiles", (1,), torch.int32),
            "max_tiles": max_tiles, "rows": n, "tile_rows": tile_rows,
        }
        if self.hidden_size % 4 == 0 and tokens <= ops.ROUTER_SMALL_TOKENS:
            logits = ctx.buffer("experts.logits", (tokens, self.num_experts), torch.float32)
            ops.router_small(act32, self.router, logits, self.bias, self.top_k, self.renormalize, self.routed_scale, tile_rows,
                             ids, weights, p["offsets"], p["sorted_token"], p["row_of_assign"], p["tile_expert"],
                             p["tile_row0"], p["num_tiles"])
        else:
            logits = self.logits(ctx, act32)
            ops.route_plan_small(logits, self.bias, self.top_k, self.renormalize, self.routed_scale, tile_rows, ids, weights,
                                 p["offsets"], p["sorted_token"], p["row_of_assign"], p["tile_expert"], p["tile_row0"],
                                 p["num_tiles"])
        return ids, weights, p

    def _tell_route(self, ids: torch.Tensor) -> None:
        if self.on_route is not None:
            self.on_route(ids)
        if self.route_log is not None:
            self.route_log[:ids.shape[0]].copy_(ids)

    def forward(self, ctx, act, act32):
        return self.forward_deferred(ctx, act, act32).materialize(ctx)

    def forward_deferred(self, ctx, act, act32):
        if act32 is None:
            raise ValueError("routed experts need the normed rows in float32 for the router")
        if (act.shape[0] <= ops.SMALL_ROUTE_TOKENS and act.shape[0] * self.top_k <= ops.SMALL_ROUTE_ASSIGNMENTS
                and self.num_experts <= 1024):
            ids, weights, p = self.route_and_plan(ctx, act32)
            self._tell_route(ids)
        else:
            ids, weights = self.route(ctx, act32)
            self._tell_route(ids)
            p = self.plan(ctx, ids)
        y = self.experts(ctx, act, p)
        # each token's expert outputs, not yet summed: the norm after this layer adds them in rank order
        return WeightedRows(y, weights, p["row_of_assign"])


class DenseGatedUnit(FeedForward):
    """silu(x W_gate^T) * (x W_up^T), then W_down: one expert's formula for every row (src/minimax.rs:116-120)."""

    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        self.hidden_size = int(spec.args["hidden_size"])
        self.width = int(spec.args["width"])
        self.w_gate_up: Optional[torch.Tensor] = None
        self.w_down: Optional[torch.Tensor] = None

    def _needs(self):
        d, i = self.hidden_size, self.width
        return (TensorNeed(self.name_of("w_gate"), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_up"), (i, d), MATRIX, "normal"),
                TensorNeed(self.name_of("w_down"), (d, i), MATRIX, "normal"))

    def tensor_needs(self):
        return list(self._needs())

    def load(self, source: TensorSource) -> None:
        gate, up, down = (source.fetch(n) for n in self._needs())
        self.w_gate_up = torch.cat([gate, up], dim=0).contiguous()
        self.w_down = down

    def forward(self, ctx, act, act32):
        both = linear(act, self.w_gate_up)                         # float32 [T, 2I]
        hidden = ctx.buffer("dense.hidden", (act.shape[0], self.width), self.dtype)
        ops.gated_unit(both, hidden)
        return linear(hidden, self.w_down)


register_part("feed_forward", "routed_experts", RoutedExperts, replace=True)
register_part("feed_forward", "dense_gated", DenseGatedUnit, replace=True)
