"""Differential attention over the paged cache: every query head takes two softmax maps over the
same values and subtracts one from the other.

A head has two queries and its key/value head two keys a token (``head_dim`` wide each, stored side
by side: map 1, then map 2) and one value (``value_dim`` wide).  Per map m::

    s_m(i, j) = softcap * tanh(q_m(i) . k_m(j) * scale / softcap)         (no cap when softcap is None)
    a_m(i)    = sum_j softmax_j s_m(i, j) v(j)      over the keys i sees (itself and the window - 1 before it)

and the head's output is ``o = a_1 - lam * a_2`` with one ``lam`` a layer,
``lam = exp(lq1 . lk1) - exp(lq2 . lk2) + lam_init`` from four stored vectors; then ``o`` is divided by
its root mean square over the head (eps inside the root, no weight) and multiplied by ``1 - lam_init``.
The heads go side by side through the output product.  Positions do not enter the scores.

Query head h uses key/value head ``h // (num_heads / num_kv_heads)``.  What is cached per token and
key/value head is one key row of ``2 * head_dim`` and one value row of ``value_dim``
(``PagedKVSpec(kv_heads, 2 * head_dim, keep, v_head_dim=value_dim)``).

A layer with ``own_kv=False`` has no key and value projections and writes nothing: its call reads the
cache slot another layer of the same geometry wrote earlier in the step (``LayerCall.writes_cache=False``),
with its own queries, window and constants.  ``keep`` is how many positions the cache slot keeps: at
least the widest window among the layers that read it (None: all).

Steps: one product for q|k|v, the page write, attention, the output product.  For a few bfloat16 rows the
two products take the norms around the mixer into their epilogues (``fusable_norm``), as the package's other
attention does.  Scores, softmax, the combination and the head norm are 32-bit in both modes; ``lam`` is
computed once, at loading, in 32-bit.
"""

from __future__ import annotations

from typing import Any, Mapping, Optional

import torch

from kairyu_b200 import kernels
from kairyu_b200.parts.base import MIXERS, CacheView, Mixer, PagedKVSpec, StepContext, TensorSpec

MAPS = 2


@MIXERS.register("differential_attention")
class DifferentialAttention(Mixer):
    graph_safe = True

    def __init__(
        self,
        *,
        prefix: str,
        hidden_size: int,
        num_heads: int,
        num_kv_heads: int,
        head_dim: int,
        value_dim: int,
        scale: float,
        lam_init: float,
        norm_eps: float,
        softcap: Optional[float] = None,
        window: Optional[int] = None,
        keep: Optional[int] = None,
        own_kv: bool = True,
        dtype: torch.dtype,
        device: str,
        **_: object,
    ) -> None:
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} query heads are not a multiple of {num_kv_heads} KV heads")
        self.prefix = prefix
        self.hidden_size = hidden_size
        self.num_heads = num_heads
        self.num_kv_heads = num_kv_heads
        self.head_dim = head_dim
        self.value_dim = value_dim
        self.scale = float(scale)
        self.lam_init = float(lam_init)
        self.norm_eps = float(norm_eps)
        self.softcap = float(softcap) if softcap else 0.0
        self.window = window
        self.keep = keep if own_kv else None
        self.own_kv = own_kv
        self.dtype = dtype
        self.q_size = num_heads * MAPS * head_dim
        self.k_size = num_kv_heads * MAPS * head_dim
        self.v_size = num_kv_heads * value_dim
        self.out_size = num_heads * value_dim
        self.packed_width = self.q_size + (self.k_size + self.v_size if own_kv else 0)
        self.w_in: Optional[torch.Tensor] = None  # [q | k | v rows, hidden]; q rows only without own_kv
        self.w_o: Optional[torch.Tensor] = None
        self.lam: float = self.lam_init  # until the four vectors are loaded

    # -- weights
    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        specs = [TensorSpec(f"{p}.q", (self.q_size, self.hidden_size))]
        if self.own_kv:
            specs += [
                TensorSpec(f"{p}.k", (self.k_size, self.hidden_size)),
                TensorSpec(f"{p}.v", (self.v_size, self.hidden_size)),
            ]
        specs += [TensorSpec(f"{p}.{name}", (self.head_dim,), role="vector", init="normal") for name in ("lq1", "lk1", "lq2", "lk2")]
        specs.append(TensorSpec(f"{p}.o", (self.hidden_size, self.out_size)))
        return specs

    def load(self, tensors: Mapping[str, torch.Tensor]) -> None:
        p = self.prefix
        rows = [tensors[f"{p}.q"]] + ([tensors[f"{p}.k"], tensors[f"{p}.v"]] if self.own_kv else [])
        self.w_in = torch.cat(rows, dim=0).contiguous()
        self.w_o = tensors[f"{p}.o"].contiguous()
        lq1, lk1, lq2, lk2 = (tensors[f"{p}.{name}"].float() for name in ("lq1", "lk1", "lq2", "lk2"))
        if not lq1.is_meta:
            # one number a layer, from weights alone: formed once, in 32-bit
            first = torch.exp((lq1 * lk1).sum())
            second = torch.exp((lq2 * lk2).sum())
            self.lam = float(first - second + torch.tensor(self.lam_init, dtype=torch.float32, device=first.device))

    def bytes_streamed(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.w_in, self.w_o))

    # -- cache
    def cache_specs(self) -> tuple[Any, ...]:
        if not self.own_kv:
            return ()
        return (PagedKVSpec(self.num_kv_heads, MAPS * self.head_dim, self.keep, v_head_dim=self.value_dim),)

    def _tensor_cores(self) -> bool:
        return self.dtype == torch.bfloat16 and kernels.diff_attention_mma_supported(self.head_dim, self.value_dim, self.num_heads, self.num_kv_heads)

    def query_tile_sizes(self) -> tuple[int, ...]:
        return (kernels.DIFF_ATTENTION_TILE,) if self._tensor_cores() else ()

    # -- compute
    def fusable_norm(self, tokens: int) -> bool:
        """Whether the q|k|v and the output product can take the norms around them into their epilogues."""
        return kernels.fused_norm_shapes_ok(tokens, self.hidden_size, self.out_size)

    def forward(self, x, ctx: StepContext, cache: CacheView, fold=None):
        """``x``: rows, or a ``kernels.PreNormed``; ``fold`` (a ``kernels.ResidualNorm``): the output product
        adds its result to the residual and returns the ``PreNormed`` for the next norm."""
        tokens = x.shape[0]
        ws = ctx.workspace
        packed = ws.buffer("diff.packed", tokens, self.packed_width, self.dtype)
        kernels.linear(x, self.w_in, None, packed)
        block_table = ctx.block_tables[cache.group]
        if self.own_kv and cache.writes:
            kernels.paged_kv_write(
                packed, self.q_size, self.q_size + self.k_size, cache.k, cache.v,
                positions=ctx.positions, row_ids=ctx.row_ids, block_table=block_table, write_from=ctx.write_from, flag=ctx.error_flag,
            )
        mixed = ws.buffer("diff.mixed", tokens, self.out_size, self.dtype)
        constants = dict(
            num_q_heads=self.num_heads, maps=MAPS, scale=self.scale, softcap=self.softcap, window=self.window or 0,
            lam=self.lam, head_norm_eps=self.norm_eps, out_scale=1.0 - self.lam_init, flag=ctx.error_flag,
        )
        if self._tensor_cores() and not ctx.extras.get("force_generic_attention", False):
            kernels.diff_attention_mma(packed, mixed, cache.k, cache.v, ctx=ctx, block_table=block_table, **constants)
        else:
            kernels.diff_attention_generic(
                packed, mixed, cache.k, cache.v, positions=ctx.positions, row_ids=ctx.row_ids, block_table=block_table, **constants
            )
        if fold is not None:
            kernels.linear(mixed, self.w_o, None, None, fold=fold)
            return fold.result()
        out = ws.buffer("diff.out", tokens, self.hidden_size, self.dtype)
        kernels.linear(mixed, self.w_o, None, out)
        return out
