"""Arrangement of a layer's parts around the residual stream.

``pre_norm``: ``h += mixer(norm1(h)); h += feed_forward(norm2(h))``, written with
the not-yet-added output carried beside the residual so that every addition is
fused into the next norm (minivllm/models/qwen3.py:216-233).

For steps of a few tokens, where the mixer and the feed-forward say that they split norms
(:meth:`~.base.Mixer.splits_norms`), neither norm runs as a kernel of its own: the product
ahead of a norm adds into the residual and hands on :class:`~.base.HalfNormedRows`, the
product behind it applies the root; the second product of the feed-forward does so under
the next block's first norm."""

from __future__ import annotations

import torch

from .. import kernels
from .base import BLOCKS, Block, CacheView, HalfNormedRows, Norm, NormedAddend, StepContext  # noqa: F401


@BLOCKS.register("pre_norm")
class PreNormBlock(Block):
    norm_roles = ("mixer", "feed_forward")
    graph_safe = True

    def _splits_norms(self, tokens: int) -> bool:
        return (self.norms["feed_forward"].split() is not None and self.mixer.splits_norms(tokens)
                and self.feed_forward.splits_norms(tokens))

    def first_norm(self) -> Norm:
        return self.norms["mixer"]

    def takes_half_normed(self, tokens: int) -> bool:
        return self.norms["mixer"].split() is not None and self._splits_norms(tokens)

    def folds_into(self, norm: Norm, tokens: int) -> bool:
        return norm.split() is not None and self._splits_norms(tokens)

    def forward(self, x: torch.Tensor | HalfNormedRows | None, residual: torch.Tensor, ctx: StepContext,
                cache: CacheView, next_norm: Norm | None = None) -> torch.Tensor | HalfNormedRows:
        normed = x if isinstance(x, HalfNormedRows) else self.norms["mixer"].forward(x, residual)
        if not self._splits_norms(residual.shape[0]):
            mixed = self.mixer.forward(normed, ctx, cache)
            normed = self.norms["feed_forward"].forward(mixed, residual)
            return self.feed_forward.forward(normed, ctx)
        half = self.mixer.forward(normed, ctx, cache, fold=(residual, self.norms["feed_forward"]))
        return self.feed_forward.forward(half, ctx, fold=None if next_norm is None else (residual, next_norm))


@BLOCKS.register("sandwich_norm")
class SandwichNormBlock(Block):
    """A norm in front of and behind each sublayer: ``h += post_mixer(mixer(mixer_norm(h)))``, then,
    where the layer has a feed-forward, ``h += post_feed_forward(feed_forward(feed_forward_norm(h)))``.

    What a sublayer returns travels on as a :class:`~.base.NormedAddend` under the norm behind it, so
    that norm, the sum into the residual and the norm in front of the next sublayer (the next layer's,
    or the model's last one) are one kernel."""

    graph_safe = True
    needs_feed_forward = False

    def __init__(self, params, env, *, mixer, feed_forward, norms) -> None:
        self.norm_roles = (("mixer", "post_mixer", "feed_forward", "post_feed_forward") if feed_forward is not None
                           else ("mixer", "post_mixer"))
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms)
        for role, norm in self.norms.items():
            if role.startswith("post_") and not hasattr(norm, "addend"):
                raise ValueError(f"block at {env.prefix!r}: the norm behind a sublayer ({role}) must be able to "
                                 f"travel with its rows (an `addend` method)")

    def forward(self, x, residual: torch.Tensor, ctx: StepContext, cache: CacheView):
        normed = self.norms["mixer"].forward(x, residual)
        mixed = self.norms["post_mixer"].addend(self.mixer.forward(normed, ctx, cache))
        if self.feed_forward is None:
            return mixed
        normed = self.norms["feed_forward"].forward(mixed, residual)
        return self.norms["post_feed_forward"].addend(self.feed_forward.forward(normed, ctx))


@BLOCKS.register("post_norm")
class PostNormBlock(Block):
    """A norm behind each sublayer and none in front: ``h += post_mixer(mixer(h))``, then, where the layer
    has one, ``h += post_feed_forward(feed_forward(h))``, then, where the layer has one, ``h +=
    post_side(side(h, tokens))``.  Every sublayer reads the residual stream itself (in the run dtype).

    What a sublayer returns travels on as a :class:`~.base.NormedAddend`; the kernel that normalises it and
    adds it into the float32 residual also writes the sum in the run dtype, which the next sublayer (the next
    layer's mixer) reads.  In the float32 run mode the sublayers read the residual in place."""

    graph_safe = True
    needs_feed_forward = False
    takes_side = True

    def __init__(self, params, env, *, mixer, feed_forward, norms, side=None) -> None:
        roles = ["post_mixer"]
        if feed_forward is not None:
            roles.append("post_feed_forward")
        if side is not None:
            roles.append("post_side")
        self.norm_roles = tuple(roles)
        super().__init__(params, env, mixer=mixer, feed_forward=feed_forward, norms=norms, side=side)
        for role, norm in self.norms.items():
            if not hasattr(norm, "addend"):
                raise ValueError(f"block at {env.prefix!r}: the norm behind a sublayer ({role}) must be able to "
                                 f"travel with its rows (an `addend` method)")

    def _rows(self, pending: NormedAddend | None, residual: torch.Tensor) -> torch.Tensor:
        """Add what is pending into the residual and return the stream as the next sublayer reads it."""
        if pending is not None and not isinstance(pending, NormedAddend):
            raise ValueError("a post-norm block takes what is handed to it as rows under the norm behind them")
        addend = (None, None, 0.0) if pending is None else (pending.rows, pending.weight, pending.eps)
        if self.env.dtype == torch.float32:
            if pending is not None:
                kernels.add_normed_rmsnorm(*addend, residual, None, 0.0, None)
            return residual
        rows = torch.empty(residual.shape, dtype=self.env.dtype, device=residual.device)
        kernels.add_normed_rmsnorm(*addend, residual, None, 0.0, rows)
        return rows

    def forward(self, x, residual: torch.Tensor, ctx: StepContext, cache: CacheView) -> NormedAddend:
        pending = self.norms["post_mixer"].addend(self.mixer.forward(self._rows(x, residual), ctx, cache))
        if self.feed_forward is not None:
            rows = self._rows(pending, residual)
            pending = self.norms["post_feed_forward"].addend(self.feed_forward.forward(rows, ctx))
        if self.side is not None:
            rows = self._rows(pending, residual)
            pending = self.norms["post_side"].addend(self.side.forward(rows, ctx))
        return pending
