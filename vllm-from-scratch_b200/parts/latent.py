"""Attention over cached latent rows.

Every position leaves one row ``c`` of ``latent_dim`` numbers in the cache: a down projection of the
layer's input, RMS-normed with a plain weight.  A head's keys and values are up projections of these
rows, ``k = U_k c`` and ``v = U_v c``, so neither needs a place of its own: with ``q' = U_k^T q`` the score
is ``q' . c``, the weighted sum of the values is ``U_v (sum_j p_j c_j)``, and the attention itself runs
over the cached rows alone, as one key/value head of size ``latent_dim`` that all query heads share and
whose rows serve as keys and as values.  No positions enter; an optional window; an optional sink per
head (one more term ``exp(sink_h)`` in the softmax denominator, unscaled, without key or value).

A layer may own no down projection and read the rows another layer cached (``own_latent=False``; the
schedule entry then names the owner in ``cache_from``), with up projections, queries, window and sinks of
its own.
"""

from __future__ import annotations

from typing import Any, Mapping

import torch

from .. import kernels
from ..kernels import grouped
from .base import MIXERS, CacheView, KVPagesNeed, Mixer, PartEnv, PositionEncoding, StepContext, WeightInfo


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """params: ``num_heads``, ``head_dim`` (queries and keys), ``value_dim``, ``latent_dim``, ``scale``,
    ``window`` (None = all keys), ``norm_eps`` (of the norm on the latent rows), ``sinks`` (default False),
    ``own_latent`` (default True), ``cache_window`` (positions the cache keeps where a reader's window is
    longer than the owner's; default: the window), ``weight_names`` (query, down, down norm, key up, value
    up, sink, output; default ``q``, ``dkv``, ``dkv.norm``, ``uk``, ``uv``, ``sink``, ``o``)."""

    graph_safe = True

    def __init__(self, params: Mapping[str, Any], env: PartEnv, position: PositionEncoding) -> None:
        super().__init__(params, env, position)
        if position.rotary_dim:
            raise ValueError("latent attention takes no rotation: give it position encoding 'none'")
        self.num_heads = int(params["num_heads"])
        self.head_dim = int(params["head_dim"])
        self.value_dim = int(params["value_dim"])
        self.latent_dim = int(params["latent_dim"])
        self.scale = float(params.get("scale", self.head_dim ** -0.5))
        window = params.get("window")
        self.window = None if window is None else int(window)
        self.cache_window = params.get("cache_window", self.window)
        self.norm_eps = float(params["norm_eps"])
        self.has_sinks = bool(params.get("sinks", False))
        self.own_latent = bool(params.get("own_latent", True))
        if self.latent_dim > 512:
            raise ValueError(f"latent_dim={self.latent_dim}: the attention kernels take rows of up to 512")
        if self.window is not None and self.window <= 0:
            raise ValueError(f"window must be positive, got {self.window}")
        self.names = tuple(params.get("weight_names", ("q", "dkv", "dkv.norm", "uk", "uv", "sink", "o")))
        self.q_down = self.down_norm = self.key_up_t = self.value_up = self.sink = self.out_proj = None

    def expected_weights(self) -> dict[str, WeightInfo]:
        hidden, heads, d, dv, rank = self.env.hidden_size, self.num_heads, self.head_dim, self.value_dim, self.latent_dim
        q, down, down_norm, key_up, value_up, sink, out = self.names
        names = {q: WeightInfo((heads * d, hidden)), key_up: WeightInfo((heads * d, rank)),
                 value_up: WeightInfo((heads * dv, rank)), out: WeightInfo((hidden, heads * dv))}
        if self.own_latent:
            names[down] = WeightInfo((rank, hidden))
            names[down_norm] = WeightInfo((rank,), "vector")
        if self.has_sinks:
            names[sink] = WeightInfo((heads,), "vector")
        return names

    def load_weights(self, tensors: Mapping[str, torch.Tensor]) -> None:
        q, down, down_norm, key_up, value_up, sink, out = self.names
        heads, d, dv, rank = self.num_heads, self.head_dim, self.value_dim, self.latent_dim
        # one product for the queries and the down projection
        self.q_down = (torch.cat([tensors[q], tensors[down]], dim=0) if self.own_latent else tensors[q]).contiguous()
        self.down_norm = tensors[down_norm] if self.own_latent else None
        # q' = U_k^T q per head: a matrix [rank, d] per head; the values' up projection is [dv, rank] as stored
        self.key_up_t = tensors[key_up].view(heads, d, rank).transpose(1, 2).contiguous()
        self.value_up = tensors[value_up].view(heads, dv, rank).contiguous()
        self.sink = tensors[sink].contiguous() if self.has_sinks else None
        self.out_proj = tensors[out].contiguous()

    def cache_need(self) -> KVPagesNeed | None:
        # A layer that reads another's rows still says what it reads; the model gives it the owner's.
        return KVPagesNeed(1, self.latent_dim, self.cache_window, value_dim=0)

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: CacheView) -> torch.Tensor:
        if cache.kind != "pages":
            raise ValueError("latent attention needs a cache of pages")
        if cache.writable != self.own_latent:
            raise ValueError("a latent layer writes the cache it owns and only reads another layer's: "
                             f"own_latent={self.own_latent}, the cache is {'its own' if cache.writable else 'lent'}")
        group = ctx.groups[cache.group]
        tokens = x.shape[0]
        heads, d, dv, rank = self.num_heads, self.head_dim, self.value_dim, self.latent_dim
        projected = torch.empty((tokens, self.q_down.shape[0]), dtype=x.dtype, device=x.device)
        kernels.gemm(x, self.q_down, projected)
        if self.own_latent:
            kernels.head_norm_scale_cache(projected, ctx.positions, group.slot_mapping, None, self.down_norm,
                                          self.norm_eps, None, None, cache.keys, None, 0, 1, rank, 0,
                                          group.page_size, column=heads * d)
        q_latent = torch.empty((tokens, heads * rank), dtype=x.dtype, device=x.device)
        grouped.head_gemm(projected, self.key_up_t, q_latent)
        attended = torch.empty((tokens, heads * rank), dtype=x.dtype, device=x.device)
        kernels.biased_paged_attention(
            q_latent, cache.keys, cache.keys, attended, ctx.query_start, ctx.seq_lens, group.block_table, None,
            heads, 1, rank, rank, group.page_size, self.scale, self.window, ctx.max_query_len, ctx.max_seq_len,
            ctx.num_decode, sinks=self.sink)
        values = torch.empty((tokens, heads * dv), dtype=x.dtype, device=x.device)
        grouped.head_gemm(attended, self.value_up, values)
        out = torch.empty((tokens, self.env.hidden_size), dtype=x.dtype, device=x.device)
        kernels.gemm(values, self.out_proj, out)
        return out
