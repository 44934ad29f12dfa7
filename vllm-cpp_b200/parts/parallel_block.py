"""The arrangement in which a layer's sublayers run side by side on one normed input:

    h = n(x);   x <- x + mixer(h) + feed_forward(h)

with one norm in front of both (a layer without a feed-forward adds the mixer's result alone), and what a model adds to
the stream where a repeated stretch of layers starts over.

Nothing is added here.  The block hands both results on as a :class:`PendingSum`; whichever norm reads the stream next
(the next layer's, or the model's last on the wanted rows) adds them all and norms in one kernel
(ops.sum_add_rmsnorm), so a layer costs one row kernel.  The stream and every sum into it are 32-bit.

:class:`LoopReentry` (family ``reentry``) is what ``LayerRun.opens`` asks for: before pass t over the repeated stretch
the stream receives the embedding's rows once more (every pass but the first) and a learned vector of the pass.  It adds
nothing itself either: it joins both to the pending sum, so the pass's first norm does it in the same kernel.
"""
from __future__ import annotations

import torch

from .. import ops
from ..weights.loader import TensorSpec
from .base import Block, Part


class PendingSum:
    """Results (32-bit [T, H], or [S, T, H] k-slice partial sums) that are still to be added to the stream, with an
    optional second stream's rows and an optional vector."""

    MAX_TERMS = 4

    def __init__(self, terms, row_extra=None, vec_extra=None):
        self.terms = [t for t in terms if t is not None]
        self.row_extra, self.vec_extra = row_extra, vec_extra

    def _settle(self, resid):
        """More results than one kernel adds: the first ones go into the stream ahead."""
        while len(self.terms) > self.MAX_TERMS:
            ops.sum_add_rmsnorm(resid, self.terms[:self.MAX_TERMS], None, 0.0, None)
            self.terms = self.terms[self.MAX_TERMS:]

    def add_then_norm(self, resid, next_gain, next_eps, out, rows=None):
        if rows is None:
            self._settle(resid)
        elif len(self.terms) > self.MAX_TERMS:
            raise ValueError(f"{len(self.terms)} pending results on a list of rows (up to {self.MAX_TERMS})")
        ops.sum_add_rmsnorm(resid, self.terms, next_gain, next_eps, out, rows, self.row_extra, self.vec_extra)

    def add(self, resid):
        self._settle(resid)
        ops.sum_add_rmsnorm(resid, self.terms, None, 0.0, None, None, self.row_extra, self.vec_extra)


def as_pending_sum(resid, pending) -> PendingSum:
    """What an arrangement before left pending, as a sum that can take more terms."""
    if pending is None:
        return PendingSum([])
    if isinstance(pending, PendingSum):
        return pending
    if torch.is_tensor(pending):
        return PendingSum([pending.float() if pending.dtype != torch.float32 else pending])
    pending.add(resid)      # a result that knows its own way into the stream (a post-norm, several streams)
    return PendingSum([])


class ParallelBlock(Block):
    """parts: ``norm1``, ``mixer`` and, unless the layer has none, ``feed_forward``."""

    def forward(self, resid, pending, ctx, cache, writes=True):
        mark = getattr(ctx, "mark", lambda label: None)
        if pending is not None and torch.is_tensor(pending) and pending.dtype != torch.float32:
            pending = as_pending_sum(resid, pending)
        h = self.parts["norm1"].forward(resid, pending)
        d = self.parts["mixer"].forward(h, ctx, cache, writes)
        mark("mixer")
        ff = self.parts.get("feed_forward")
        if ff is None:
            return PendingSum([d])
        d2 = ff.forward(h, ctx)
        mark("feed_forward")
        return PendingSum([d, d2])


class LoopReentry(Part):
    """params: ``hidden_size``, ``passes``; ``step_tensor`` (None: no vector per pass): a tensor [passes, hidden] whose
    row t is added before pass t; ``add_embedding`` (default True): before every pass but the first the embedding's rows
    are added once more."""
    family = "reentry"

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden, self.passes = int(params["hidden_size"]), int(params["passes"])
        self.step_name = params.get("step_tensor")
        self.add_embedding = bool(params.get("add_embedding", True))
        self.needs_embedding = self.add_embedding and self.passes > 1
        self.steps = None

    def tensor_specs(self):
        if self.step_name is None:
            return []
        return [TensorSpec(str(self.step_name), (self.passes, self.hidden), "bias")]

    def bind(self, store):
        if self.step_name is not None:
            self.steps = store.vector(str(self.step_name)).float().contiguous()

    def forward(self, resid, pending, first_rows, t: int):
        """-> the pending sum with what pass ``t`` starts with joined to it."""
        if not 0 <= t < self.passes:
            raise ValueError(f"pass {t} of {self.passes}")
        out = as_pending_sum(resid, pending)
        if out.row_extra is not None or out.vec_extra is not None:
            out.add(resid)      # (a pass that opens right behind another opening: settle the first)
            out = PendingSum([])
        row = first_rows if self.add_embedding and t > 0 else None
        vec = self.steps[t] if self.steps is not None else None
        return PendingSum(out.terms, row, vec)
