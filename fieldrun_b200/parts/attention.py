"""Grouped-query attention over the paged cache.

q, k, v = act W^T without bias; optionally an RMSNorm of q and of k before the
rotary: "full_width", one statistic over the whole Q row and one over the whole
K row with weights as wide as the rows (before the head split,
src/minimax.rs:136-138), or "per_head", a statistic per head with one weight
vector of the head's size for all heads; rotary on the first ``rotary_dim`` dims of each head at
the token's absolute position; K (normed, rotated) and V written to the cache
line; every query head h attends, with keys of head h // (heads / kv_heads), over
the keys it may see; output projection without bias (src/minimax.rs:253-282).
The three projections are held as one matrix so that one product makes q|k|v.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..cache import CacheNeed, LineView
from ..csrc import ops
from ..weights.loader import MATRIX, VECTOR, TensorNeed, TensorSource
from .base import Mixer, build_position, register_part
from .linear import linear


TC_ATTENTION_MIN_QUERIES = 64       # a step whose longest run of new tokens is shorter uses tiles of 16 queries


class GQAAttention(Mixer):
    replayable = True

    def __init__(self, spec, dtype):
        super().__init__(spec, dtype)
        a = spec.args
        self.hidden_size = int(a["hidden_size"])
        self.num_heads = int(a["num_heads"])
        self.num_kv_heads = int(a["num_kv_heads"])
        self.head_dim = int(a["head_dim"])
        self.qk_norm = a.get("qk_norm", "none")
        if self.qk_norm not in ("none", "full_width", "per_head"):
            raise ValueError(f"qk_norm {self.qk_norm!r} is none of 'none', 'full_width', 'per_head'")
        self.qk_norm_eps = float(a.get("qk_norm_eps", 1e-6))
        self.softmax_scale = float(a.get("softmax_scale", self.head_dim ** -0.5))
        self.window = a.get("window")
        if self.window is not None and int(self.window) <= 0:
            raise ValueError(f"an attention window of {self.window} keys")
        if self.num_heads % self.num_kv_heads:
            raise ValueError(f"{self.num_heads} heads are not a multiple of {self.num_kv_heads} kv heads")
        if not 1 <= self.head_dim <= 256:
            raise ValueError(f"head_dim {self.head_dim} is outside the kernels' range 1..256")
        self.position = build_position(a.get("position"))
        if self.position is not None and self.position.rotary_dim > self.head_dim:
            raise ValueError(f"rotary_dim {self.position.rotary_dim} exceeds head_dim {self.head_dim}")
        self.q_width = self.num_heads * self.head_dim
        self.kv_width = self.num_kv_heads * self.head_dim
        self.w_qkv: Optional[torch.Tensor] = None
        self.w_o: Optional[torch.Tensor] = None
        self.q_norm: Optional[torch.Tensor] = None
        self.k_norm: Optional[torch.Tensor] = None
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None

    # -- tensors -----------------------------------------------------------------------------------
    def _needs(self) -> dict[str, TensorNeed]:
        needs = {
            "q_proj": TensorNeed(self.name_of("q_proj"), (self.q_width, self.hidden_size), MATRIX, "normal"),
            "k_proj": TensorNeed(self.name_of("k_proj"), (self.kv_width, self.hidden_size), MATRIX, "normal"),
            "v_proj": TensorNeed(self.name_of("v_proj"), (self.kv_width, self.hidden_size), MATRIX, "normal"),
            "o_proj": TensorNeed(self.name_of("o_proj"), (self.hidden_size, self.q_width), MATRIX, "normal"),
        }
        if self.qk_norm == "full_width":
            needs["q_norm"] = TensorNeed(self.name_of("q_norm"), (self.q_width,), VECTOR, "around_one")
            needs["k_norm"] = TensorNeed(self.name_of("k_norm"), (self.kv_width,), VECTOR, "around_one")
        elif self.qk_norm == "per_head":
            needs["q_norm"] = TensorNeed(self.name_of("q_norm"), (self.head_dim,), VECTOR, "around_one")
            needs["k_norm"] = TensorNeed(self.name_of("k_norm"), (self.head_dim,), VECTOR, "around_one")
        return needs

    def tensor_needs(self):
        return list(self._needs().values())

    def load(self, source: TensorSource) -> None:
        needs = self._needs()
        self.w_qkv = torch.cat([source.fetch(needs[n]) for n in ("q_proj", "k_proj", "v_proj")], dim=0).contiguous()
        self.w_o = source.fetch(needs["o_proj"])
        if self.qk_norm != "none":
            self.q_norm = source.fetch(needs["q_norm"])
            self.k_norm = source.fetch(needs["k_norm"])

    # -- cache and tables ----------------------------------------------------------------------------
    def cache_need(self) -> CacheNeed:
        return CacheNeed(kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                         window=int(self.window) if self.window is not None else None)

    def prepare(self, num_positions: int, device) -> None:
        if self.position is not None and self.position.rotary_dim > 0:
            self.cos, self.sin = self.position.shared_tables(num_positions, device)

    # -- one step --------------------------------------------------------------------------------------
    def forward(self, ctx, act: torch.Tensor, line: LineView, writes_cache: bool) -> torch.Tensor:
        tokens = act.shape[0]
        qkv = linear(act, self.w_qkv)                                        # float32 [T, q + 2 kv]
        q = ctx.buffer("attention.q", (tokens, self.q_width), self.dtype)
        rotary_dim = self.position.rotary_dim if self.position is not None else 0
        ops.qkv_prepare(qkv, self.q_norm, self.k_norm, self.qk_norm_eps, self.cos, self.sin, ctx.tok_pos, ctx.tok_slot,
                        line.page_table, q, line.keys, line.values, num_heads=self.num_heads,
                        num_kv_heads=self.num_kv_heads, head_dim=self.head_dim, rotary_dim=rotary_dim,
                        interleaved=bool(self.position.interleaved) if self.position is not None else False,
                        write_cache=writes_cache, per_head=self.qk_norm == "per_head",
                        tables_final=True)      # the step's tables were there before the projection above began
        out = ctx.buffer("attention.out", (tokens, self.q_width), self.dtype)
        self.attend(ctx, q, line, out)
        return linear(out, self.w_o)

    def attend(self, ctx, q: torch.Tensor, line: LineView, out: torch.Tensor) -> None:
        """Tensor-core kernels for bfloat16 and head sizes of 32, 64, 96 or 128 (tcgen05 for prompts with head
        sizes 64 and 128, mma.sync otherwise); the general kernel for everything else."""
        common = dict(num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                      scale=self.softmax_scale, window=self.window)
        if self.dtype == torch.bfloat16 and self.head_dim in ops.MMA_HEAD_DIMS:
            if ctx.is_decode and self.num_heads // self.num_kv_heads <= 16:
                chunks = (ctx.max_kv_len + ops.ATTENTION_CHUNK - 1) // ops.ATTENTION_CHUNK
                part_o = ctx.buffer("attention.part_o", (ctx.num_seqs, self.num_heads, chunks, self.head_dim), torch.float32)
                part_ml = ctx.buffer("attention.part_ml", (ctx.num_seqs, self.num_heads, chunks, 2), torch.float32)
                # head sizes 64 and 128: the pages come into shared memory by TMA; others: loads into registers
                decode = ops.attention_decode_tma if self.head_dim in ops.TC_ATTENTION_HEAD_DIMS else ops.attention_decode_mma
                decode(q, line.keys, line.values, line.page_table, ctx.seq_start, ctx.seq_slot, part_o, part_ml, out,
                       max_chunks=chunks, **common)
            elif self.head_dim in ops.TC_ATTENTION_HEAD_DIMS and ctx.max_q_len >= TC_ATTENTION_MIN_QUERIES:
                # prompts: 128 queries of one head per block, both products on tcgen05
                tile_seq, tile_q0 = ctx.query_tiles(ops.TC_ATTENTION_QUERIES)
                ops.attention_prefill_tc(q, line.keys, line.values, line.page_table, tile_seq, tile_q0, ctx.seq_slot,
                                         ctx.seq_start, ctx.seq_q_len, ctx.cu_q_len, out, **common)
            else:
                tile_seq, tile_q0 = ctx.query_tiles(16)
                ops.attention_prefill_mma(q, line.keys, line.values, line.page_table, tile_seq, tile_q0, ctx.seq_slot,
                                          ctx.seq_start, ctx.seq_q_len, ctx.cu_q_len, out, **common)
            return
        ops.attention_generic(q, line.keys, line.values, line.page_table, ctx.tok_pos, ctx.tok_slot, out,
                              num_heads=self.num_heads, num_kv_heads=self.num_kv_heads, head_dim=self.head_dim,
                              scale=self.softmax_scale, window=self.window)


register_part("mixer", "gqa_attention", GQAAttention, replace=True)
