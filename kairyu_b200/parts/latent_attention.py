"""Latent attention: attention whose keys and values are all products of one compressed row a token.

A token's row ``c = rmsnorm(W_dkv x)`` (``kv_rank`` wide) is all that is cached.  Head h has
``k = W_uk[h] c`` and ``v = W_uv[h] c``; since ``q.k = (W_uk[h]^T q).c`` and
``sum_j p_j v_j = W_uv[h] (sum_j p_j c_j)``, the up-projections move to the query and to the
output, and what runs over the cache is multi-query attention with ONE key/value head of width
``kv_rank`` whose keys and values are the same rows.  So the paged attention kernels of this
package serve it unchanged (the cached rows are passed as keys and as values), and a token costs
``kv_rank`` cached numbers whatever the number of heads.  There is no position encoding; ``window``
(a token sees itself and the ``window - 1`` before it) and ``scale`` are parameters.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.attention import run_paged_attention
from kairyu_b200.parts.base import MIXERS, CacheView, Mixer, PagedKVSpec, StepContext, TensorSpec


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        head_dim: int,
        value_dim: int,
        kv_rank: int,
        scale: float,
        norm_eps: float,
        window: Optional[int] = None,
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.value_dim = value_dim
        self.kv_rank = kv_rank
        self.scale = float(scale)
        self.norm_eps = float(norm_eps)
        self.window = window
        self.dtype = dtype
        self.q_size = num_heads * head_dim
        self.w_in: Optional[torch.Tensor] = None      # [q_size + kv_rank, hidden]: q rows, then the down-projection's
        self.latent_norm: Optional[torch.Tensor] = None
        self.w_absorb: Optional[torch.Tensor] = None  # [heads, kv_rank, head_dim]: W_uk[h]^T
        self.w_up_v: Optional[torch.Tensor] = None    # [heads, value_dim, kv_rank]
        self.w_o: Optional[torch.Tensor] = None

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        return [
            TensorSpec(f"{p}.q", (self.q_size, self.hidden_size)),
            TensorSpec(f"{p}.dkv", (self.kv_rank, self.hidden_size)),
            TensorSpec(f"{p}.dkv.norm", (self.kv_rank,), role="vector", init="norm"),
            TensorSpec(f"{p}.uk", (self.q_size, self.kv_rank)),
            TensorSpec(f"{p}.uv", (self.num_heads * self.value_dim, self.kv_rank)),
            TensorSpec(f"{p}.o", (self.hidden_size, self.num_heads * self.value_dim)),
        ]

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        self.w_in = torch.cat([tensors[f"{p}.q"], tensors[f"{p}.dkv"]], dim=0).contiguous()
        self.latent_norm = tensors[f"{p}.dkv.norm"].contiguous()
        self.w_absorb = tensors[f"{p}.uk"].view(self.num_heads, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_up_v = tensors[f"{p}.uv"].view(self.num_heads, self.value_dim, self.kv_rank).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.latent_norm, self.w_absorb, self.w_up_v, self.w_o))

    def cache_specs(self) -> tuple[Any, ...]:
        # one "head" of kv_rank columns a position and no value rows of their own
        return (PagedKVSpec(1, self.kv_rank, self.window, v_head_dim=0),)

    HEADS_PER_CALL = 16  # the tensor-core attention kernels take up to 16 query heads a key/value head

    def _tensor_cores(self) -> bool:
        return self.dtype == torch.bfloat16 and kernels.attention_mma_supported(self.kv_rank, min(self.num_heads, self.HEADS_PER_CALL), 1)

    def query_tile_sizes(self) -> tuple[int, ...]:
        if not self._tensor_cores():
            return ()
        wide = kernels.attention_prefill_wide_tile_rows(self.kv_rank)
        return (kernels.attention_prefill_tile_rows(self.kv_rank),) + ((wide,) if wide else ())

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        tokens = x.shape[0]
        ws = ctx.workspace
        heads, rank = self.num_heads, self.kv_rank
        packed = ws.buffer("latent.packed", tokens, self.q_size + rank, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        if cache.writes:
            kernels.latent_norm_write(
                packed, self.q_size, rank, self.latent_norm, self.norm_eps, cache.k,
                positions=ctx.positions, row_ids=ctx.row_ids, block_table=ctx.block_tables[cache.group],
                write_from=ctx.write_from, flag=ctx.error_flag,
            )
        q_latent = ws.buffer("latent.q", tokens, heads * rank, self.dtype)
        kernels.heads_linear(packed[:, : self.q_size].unflatten(1, (heads, self.head_dim)), self.w_absorb, q_latent.view(tokens, heads, rank))
        mixed = ws.buffer("latent.mixed", tokens, heads * rank, self.dtype)
        rows = CacheView(k=cache.k, v=cache.k, page_size=cache.page_size, group=cache.group, writes=False)
        # all heads read the same rows; more heads than a kernel takes go in several calls over column ranges
        per_call = self.HEADS_PER_CALL if self._tensor_cores() else heads
        for first in range(0, heads, per_call):
            count = min(per_call, heads - first)
            columns = slice(first * rank, (first + count) * rank)
            run_paged_attention(q_latent[:, columns], mixed[:, columns], rows, ctx, num_q_heads=count, num_kv_heads=1, head_dim=rank,
                                scale=self.scale, window=self.window or 0)
        values = ws.buffer("latent.values", tokens, heads * self.value_dim, self.dtype)
        kernels.heads_linear(mixed.view(tokens, heads, rank), self.w_up_v, values.view(tokens, heads, self.value_dim))
        out = ws.buffer("latent.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(values, self.w_o, None, out)
        return out
