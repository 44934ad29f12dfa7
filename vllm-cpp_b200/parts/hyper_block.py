"""The pre-norm arrangement over several residual streams ("hyper-connections"), with an optional token shift on what
the mixer reads:

    streams x_1 .. x_S, all equal to the embedding's row at the start of the model; for sublayer q (mixer, feed-forward):
        u = sum_s in_q[s] x_s                      the read-out
        y = sublayer(n(u))                         n(v) = w * v / sqrt(mean(v^2) + eps)
        x_r <- sum_s mix_q[s, r] x_s + out_q[r] y  all streams at once, from the old ones
    after the last layer the streams are added up.

With one stream and no mixing tensors (``streams`` 0 or 1 and ``mixing`` False) this is the plain x <- x + sublayer(n(x)).

Token shift: the mixer reads h_t + (h_(t-1) - h_t) * mu per channel instead of h_t = n(u)_t, with h_(t-1) as it was before
this replacement and zeros before a request's first token; the last h of a request is part of its state, kept here
(a fixed-size state beside whatever the mixer keeps).

The write-back of one sublayer, the read-out of the next and its norm are one kernel (ops.hyper_mix_norm), so the block
hands its last result on as a :class:`PendingStreams`: the next layer's first read-out, or the model's last norm on the
wanted rows, does the write-back.  Streams, sums, norms and the shift are 32-bit.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Block, CacheSpec


class PendingStreams:
    """A sublayer's result (32-bit sums or k-slice partial sums) that is still to be written back into the streams."""

    def __init__(self, streams, delta, mix, outw):
        self.streams, self.delta, self.mix, self.outw = streams, delta, mix, outw

    def add_then_norm(self, resid, next_gain, next_eps, out, rows=None):
        """The write-back, the plain sum of the streams and a norm of it, in one pass (the model's last norm)."""
        ops.hyper_mix_norm(self.streams, y=self.delta, mix=self.mix, outw=self.outw, gain=next_gain, eps=next_eps, out=out,
                           rows=rows)
        if rows is None and self.streams.shape[0] > 1:
            resid.copy_(self.streams.sum(0))

    def add(self, resid):
        """The write-back alone; ``resid`` then holds the sum of the streams."""
        ops.hyper_mix_norm(self.streams, y=self.delta, mix=self.mix, outw=self.outw)
        if self.streams.shape[0] > 1 or self.streams.data_ptr() != resid.data_ptr():
            resid.copy_(self.streams.sum(0))


class HyperStreamsBlock(Block):
    """parts: ``norm1``, ``mixer`` and, unless the layer has none, ``norm2`` and ``feed_forward``.
    params: ``hidden_size``; ``streams`` (default 1); ``mixing`` (default: streams > 1): tensors ``hc1.in``, ``hc1.out``
    [S], ``hc1.mix`` [S, S] ([from, to]) and ``hc2.*`` with a feed-forward; ``token_shift`` (default False): tensor
    ``shift`` [hidden]."""

    def __init__(self, params, prefix, build, parts):
        super().__init__(params, prefix, build, parts)
        self.hidden = int(params["hidden_size"])
        self.S = max(1, int(params.get("streams") or 1))
        self.mixing = bool(params.get("mixing", self.S > 1))
        self.shift = bool(params.get("token_shift", False))
        self.has_ff = "feed_forward" in parts
        if self.has_ff != ("norm2" in parts):
            raise ValueError("a feed-forward and its norm come together")
        if self.S > 1 and not self.mixing:
            raise ValueError("several streams need their mixing tensors")
        self.mu = None
        self.hc = [(None, None, None), (None, None, None)]      # per sublayer: (in, out, mix)

    # ---- weights ----
    def _sublayers(self):
        return ("hc1", "hc2")[:2 if self.has_ff else 1]

    def tensor_specs(self):
        p, S = self.prefix, self.S
        specs = super().tensor_specs()
        if self.mixing:
            for n in self._sublayers():
                specs += [TensorSpec(f"{p}{n}.in", (S,), "vector"), TensorSpec(f"{p}{n}.out", (S,), "vector"),
                          TensorSpec(f"{p}{n}.mix", (S, S), "mixing")]
        if self.shift:
            specs.append(TensorSpec(p + "shift", (self.hidden,), "unit"))
        return specs

    def bind(self, store):
        super().bind(store)
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        if self.mixing:
            for i, n in enumerate(self._sublayers()):
                self.hc[i] = (f32(n + ".in"), f32(n + ".out"), f32(n + ".mix"))
        if self.shift:
            self.mu = f32("shift")

    # ---- per-request state ----
    def cache_spec(self):
        theirs = self.mixer.cache_spec()
        theirs = () if theirs is None else (theirs if isinstance(theirs, tuple) else (theirs,))
        mine = (CacheSpec("state", shape=(self.hidden,), dtype="float32"),) if self.shift else ()
        return (mine + theirs) or None

    def _split(self, cache):
        """(this block's state view or None, what the mixer is handed)."""
        if cache is None:
            return None, None
        views = cache if isinstance(cache, tuple) else (cache,)
        mine = None
        if self.shift:
            mine, views = views[0], views[1:]
        theirs = self.mixer.cache_spec()
        return mine, (views if isinstance(theirs, tuple) else (views[0] if views else None))

    # ---- one step ----
    def forward(self, resid, pending, ctx, cache, writes=True):
        mark = getattr(ctx, "mark", lambda label: None)
        T, W = resid.shape
        dt, dev = self.build.compute_dtype, resid.device
        init = y = mix = outw = None
        if isinstance(pending, PendingStreams) and pending.streams.shape[0] == self.S:
            streams, y, mix, outw = pending.streams, pending.delta, pending.mix, pending.outw
        else:
            # the first layer of the step (or a layer of another arrangement came before): every stream starts as the
            # stream so far
            if hasattr(pending, "add"):
                pending.add(resid)
            elif pending is not None:
                resid.add_((pending.sum(0) if pending.dim() == 3 else pending).float())
            if self.S == 1:
                streams = resid.view(1, T, W)
            else:
                streams = ctx.plan(("residual streams", self.S, W), lambda: workspace.empty((self.S, T, W), torch.float32, dev))
                init = resid
        own, mixer_cache = self._split(cache)
        norm1 = self.parts["norm1"]
        h = workspace.empty((T, W), dt, dev)
        if self.shift:
            h32 = workspace.empty((T, W), torch.float32, dev)
            ops.hyper_mix_norm(streams, init=init, y=y, mix=mix, outw=outw, inw=self.hc[0][0], gain=norm1.gain32(),
                               eps=norm1.eps, out=h32)
            ops.token_shift(h32, self.mu, own.state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, h)
        else:
            ops.hyper_mix_norm(streams, init=init, y=y, mix=mix, outw=outw, inw=self.hc[0][0], gain=norm1.gain32(),
                               eps=norm1.eps, out=h)
        d = self.mixer.forward(h, ctx, mixer_cache, writes)
        mark("mixer")
        if not self.has_ff:
            return PendingStreams(streams, d, self.hc[0][2], self.hc[0][1])
        norm2 = self.parts["norm2"]
        h2 = workspace.empty((T, W), dt, dev)
        ops.hyper_mix_norm(streams, y=d, mix=self.hc[0][2], outw=self.hc[0][1], inw=self.hc[1][0], gain=norm2.gain32(),
                           eps=norm2.eps, out=h2)
        d2 = self.parts["feed_forward"].forward(h2, ctx)
        mark("feed_forward")
        return PendingStreams(streams, d2, self.hc[1][2], self.hc[1][1])
