"""Two recurrent mixers whose state is a matrix per head, S [d, dv] in 32-bit, carried in the request's slot:

the gated delta rule (``DeltaRuleMixer``)

    q, k, v = silu(conv(W_q x)), silu(conv(W_k x)), silu(conv(W_v x))      a short causal convolution per channel
    q <- q / sqrt(sum q^2 + 1e-6) * d^(-1/2),   k <- k / sqrt(sum k^2 + 1e-6)          per head
    beta = sigmoid(W_b x),   g = exp(-exp(A_log_h) softplus(W_a x + dt_bias_h))       one of each per head
    S <- g S;   w = beta (v - S^T k);   S <- S + k w^T;   o = S^T q                   (the read-out sees this token's write)
    out = W_o [ gain * o_h / sqrt(mean(o_h^2) + eps) * silu(W_g x)_h ]

with ``kv_heads`` heads of q and k, head h reading q/k head h // (heads / kv_heads); and the gated linear form
(``GatedLinearMixer``), in which the forget gate also decides what is written:

    q = silu(W_q x),   f = low + (1 - low) sigmoid(W_f x + b_f),   v = W_v x
    S <- diag(f) S + (1 - f) v^T;   o = S^T q;   out = W_o [ gain * o_h / sqrt(mean(o_h^2) + eps) ]

All projections of a mixer are one stacked product.  Everything behind the projections and the convolution -- unit
norms, gates, decays, the state, the heads' norms -- is 32-bit.  Beside the state the delta rule keeps the convolution's
last taps - 1 inputs per request.  The recurrences run token after token (ops.matrix_rnn), however a prompt is cut.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import CacheSpec, Mixer
from .linear import matmul_tn


class _MatrixStateMixer(Mixer):
    def _sizes(self, p):
        self.hidden, self.heads = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.dv = int(p["head_dim"]), int(p["v_head_dim"])
        self.eps = float(p.get("eps", 1e-5))
        if not 1 <= self.d <= 512:
            raise ValueError(f"{self.d} state rows a head: the recurrence keeps 1 to 512")

    def _read_out(self, o, u, gate_col, ctx, dt):
        """The heads' norm (and gate) on the recurrence's 32-bit result, then the output projection."""
        g = workspace.empty(o.shape, dt, o.device)
        ops.head_norm_gate(o, self.norm_w, self.eps, ctx.q_start, ctx.q_len, ctx.E, self.heads, self.dv, g,
                           gate=u if gate_col is not None else None, gate_col=gate_col or 0)
        return matmul_tn(g, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)


class DeltaRuleMixer(_MatrixStateMixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads`` (default num_heads), ``head_dim`` (d), ``v_head_dim``
    (dv), ``conv_taps``, ``eps``.  Tensors under the prefix: ``q``, ``k`` [kv_heads d, H], ``v``, ``g`` [heads dv, H], each
    of q, k, v with ``.conv`` [channels, taps]; ``b``, ``a`` [heads, H]; ``A_log``, ``dt_bias`` [heads]; ``norm`` [dv];
    ``o`` [H, heads dv]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self._sizes(params)
        self.kv_heads = int(params.get("num_kv_heads") or self.heads)
        self.taps = int(params["conv_taps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"{self.heads} heads are not a multiple of {self.kv_heads} heads of queries and keys")
        if self.taps < 1:
            raise ValueError("a convolution has at least the current token's tap")
        self.qk, self.inner = self.kv_heads * self.d, self.heads * self.dv
        self.conv_channels = 2 * self.qk + self.inner
        self.w_in = self.w_o = self.conv_w = self.dt_bias = self.rate = self.norm_w = None

    def cache_spec(self):
        state = CacheSpec("state", shape=(self.heads, self.dv, self.d), dtype="float32")
        if self.taps > 1:
            return (state, CacheSpec("state", shape=(self.taps - 1, self.conv_channels), dtype="float32"))
        return state

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        rows = (("q", self.qk), ("k", self.qk), ("v", self.inner))
        return ([TensorSpec(p + n, (r, H)) for n, r in rows]
                + [TensorSpec(p + n + ".conv", (r, self.taps), "bias") for n, r in rows]
                + [TensorSpec(p + "g", (self.inner, H)), TensorSpec(p + "b", (self.heads, H)), TensorSpec(p + "a", (self.heads, H)),
                   TensorSpec(p + "A_log", (self.heads,), "bias"), TensorSpec(p + "dt_bias", (self.heads,), "bias"),
                   TensorSpec(p + "norm", (self.dv,), "vector"), TensorSpec(p + "o", (H, self.inner))])

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        # columns of the stacked product: q | k | v (what the convolution reads) | g | b | a
        self.w_in = store.matrices([p + n for n in ("q", "k", "v", "g", "b", "a")])
        self.w_o = store.matrix(p + "o")
        self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        self.dt_bias, self.norm_w = f32("dt_bias"), f32("norm")
        self.rate = torch.exp(f32("A_log")).contiguous()

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("a recurrent mixer keeps a state of its own: it cannot read one another run left")
        state, conv_state = (cache[0].state, cache[1].state) if isinstance(cache, tuple) else (cache.state, None)
        T, dev, cc = x.shape[0], x.device, self.conv_channels
        u = matmul_tn(x, self.w_in, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        conv_in = u[..., :cc]
        xc = workspace.empty((T, cc), torch.float32, dev)
        ops.causal_conv(conv_in, self.conv_w, conv_state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, out_conv=xc, act="silu")
        if self.taps > 1 and any(n > 1 for n in ctx.host_q_len):
            # (entries of one token were brought up to date by the convolution itself)
            ops.conv_state_update(conv_in, conv_state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E)
        o = workspace.empty((T, self.inner), torch.float32, dev)
        ops.matrix_rnn("delta", u, state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, o, heads=self.heads, kv_heads=self.kv_heads,
                       d=self.d, dv=self.dv, x=xc, q_col=0, k_col=self.qk, v_col=2 * self.qk, b_col=cc + self.inner,
                       a_col=cc + self.inner + self.heads, dt_bias=self.dt_bias, rate=self.rate)
        return self._read_out(o, u, cc, ctx, x.dtype)


class GatedLinearMixer(_MatrixStateMixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (d), ``v_head_dim`` (dv), ``eps``.  Tensors under the prefix:
    ``q``, ``f`` [heads d, H], ``f.b``, ``lower`` [heads d], ``v`` [heads dv, H], ``norm`` [dv], ``o`` [H, heads dv]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self._sizes(params)
        self.qk, self.inner = self.heads * self.d, self.heads * self.dv
        self.w_in = self.w_o = self.f_bias = self.lower = self.norm_w = None

    def cache_spec(self):
        return CacheSpec("state", shape=(self.heads, self.dv, self.d), dtype="float32")

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        return [TensorSpec(p + "q", (self.qk, H)), TensorSpec(p + "f", (self.qk, H)), TensorSpec(p + "f.b", (self.qk,), "bias"),
                TensorSpec(p + "lower", (self.qk,), "unit"), TensorSpec(p + "v", (self.inner, H)),
                TensorSpec(p + "norm", (self.dv,), "vector"), TensorSpec(p + "o", (H, self.inner))]

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        self.w_in = store.matrices([p + n for n in ("q", "f", "v")])
        self.w_o = store.matrix(p + "o")
        self.f_bias, self.lower, self.norm_w = f32("f.b"), f32("lower"), f32("norm")

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("a recurrent mixer keeps a state of its own: it cannot read one another run left")
        T, dev = x.shape[0], x.device
        u = matmul_tn(x, self.w_in, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        o = workspace.empty((T, self.inner), torch.float32, dev)
        ops.matrix_rnn("gated", u, cache.state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, o, heads=self.heads, d=self.d,
                       dv=self.dv, q_col=0, k_col=self.qk, v_col=2 * self.qk, f_bias=self.f_bias, lower=self.lower)
        return self._read_out(o, u, None, ctx, x.dtype)


class DecayedLinearMixer(_MatrixStateMixer):
    """Gated linear attention: a learned decay per state row (key channel), from a low-rank projection of the input:

        q = W_q x * d^(-1/2),   k = W_k x,   v = W_v x
        f = sigmoid(W_a2 (W_a1 x) + b)^(1 / tau)                       one decay per head and key channel
        S <- diag(f) S + k v^T;   o = S^T q;   out = W_o [ gain * o_h / sqrt(mean(o_h^2) + eps) * silu(W_g x)_h ]

    params: ``hidden_size``, ``num_heads``, ``head_dim`` (d), ``v_head_dim`` (dv), ``tau``, ``eps``; ``rank`` (0 or left
    out: the inner size of the low-rank pair is whatever the checkpoint's tensors have).  Tensors under the prefix:
    ``q``, ``k`` [heads d, H], ``v``, ``g`` [heads dv, H], ``a1`` [rank, H], ``a2`` [heads d, rank], ``a2.b`` [heads d],
    ``norm`` [dv], ``o`` [H, heads dv].  q, k, v, g and a1 are one stacked product; the decay (its logarithm, the power)
    and the state are 32-bit."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self._sizes(params)
        self.tau = float(params["tau"])
        self.rank = int(params.get("rank") or 0)
        if not self.tau > 0:
            raise ValueError("the decay's temperature must be positive")
        self.qk, self.inner = self.heads * self.d, self.heads * self.dv
        self.w_in = self.w_a2 = self.w_o = self.a_bias = self.norm_w = None

    def cache_spec(self):
        return CacheSpec("state", shape=(self.heads, self.dv, self.d), dtype="float32")

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        r = self.rank or -1     # -1: any size, as long as both tensors agree (checked when they are bound)
        return [TensorSpec(p + "q", (self.qk, H)), TensorSpec(p + "k", (self.qk, H)), TensorSpec(p + "v", (self.inner, H)),
                TensorSpec(p + "g", (self.inner, H)), TensorSpec(p + "a1", (r, H)), TensorSpec(p + "a2", (self.qk, r)),
                TensorSpec(p + "a2.b", (self.qk,), "bias"), TensorSpec(p + "norm", (self.dv,), "vector"),
                TensorSpec(p + "o", (H, self.inner))]

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        # columns of the stacked product: q | k | v | g | a1
        self.w_in = store.matrices([p + n for n in ("q", "k", "v", "g", "a1")])
        self.w_a2 = store.matrix(p + "a2")
        self.rank = int(self.w_a2.shape[1])
        if self.w_in.shape[0] != 2 * self.qk + 2 * self.inner + self.rank:
            raise ValueError(f"{p}a1 and {p}a2 disagree about the rank of the decay's projection")
        self.w_o = store.matrix(p + "o")
        self.a_bias, self.norm_w = f32("a2.b"), f32("norm")

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("a recurrent mixer keeps a state of its own: it cannot read one another run left")
        T, dev = x.shape[0], x.device
        u = matmul_tn(x, self.w_in, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        a_col = 2 * self.qk + 2 * self.inner
        low = workspace.empty((T, self.rank), x.dtype, dev)
        ops.bias_act(u[..., a_col:a_col + self.rank], low, "identity")
        z = matmul_tn(low, self.w_a2, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        o = workspace.empty((T, self.inner), torch.float32, dev)
        ops.matrix_rnn("decayed", u, cache.state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, o, heads=self.heads, d=self.d,
                       dv=self.dv, q_col=0, k_col=self.qk, v_col=2 * self.qk, z=z, f_bias=self.a_bias, tau=self.tau)
        return self._read_out(o, u, 2 * self.qk + self.inner, ctx, x.dtype)


class RetentionMixer(_MatrixStateMixer):
    """Retention: linear attention with one fixed decay per head and neither softmax nor denominator:

        q, k = rot(W_q x), rot(W_k x) * d^(-1/2),   v = W_v x        rot: the first ``rotary_dim`` lanes of a head turn
        S <- decay_h S + k v^T;   o = S^T q                           by position * base^(-2i / rotary_dim)
        out = W_o [ o_h / sqrt(mean(o_h^2) + eps) * silu(W_g x)_h ]   (no gain on the heads' norm)

    params: ``hidden_size``, ``num_heads``, ``head_dim`` (d), ``v_head_dim`` (dv), ``decay`` (a number per head),
    ``rope_base``, ``rotary_dim``, ``pairing`` ("half", the default, or "interleaved"), ``eps``.  Tensors under the prefix:
    ``q``, ``k`` [heads d, H], ``v``, ``g`` [heads dv, H], ``o`` [H, heads dv].  Angles, the rotation and the state are
    32-bit."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        from .window_attention import rotary_frequencies
        self._sizes(params)
        decay = [float(g) for g in params["decay"]]
        if len(decay) != self.heads:
            raise ValueError(f"{len(decay)} decays for {self.heads} heads")
        self.decay = torch.tensor(decay, dtype=torch.float32, device=build.device)
        self.rot = int(params.get("rotary_dim") if params.get("rotary_dim") is not None else self.d)
        if self.rot % 2 or not 0 <= self.rot <= self.d:
            raise ValueError(f"{self.rot} turning lanes in heads of {self.d}: an even number up to the head size")
        pairing = str(params.get("pairing") or "half")
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing '{pairing}' is not one of 'half', 'interleaved'")
        self.interleaved = pairing == "interleaved"
        self.freq = rotary_frequencies(build, float(params.get("rope_base", 10000.0)), self.rot) if self.rot else None
        self.qk, self.inner = self.heads * self.d, self.heads * self.dv
        self.w_in = self.w_o = None
        self.norm_w = None      # the heads' norm has no gain

    def cache_spec(self):
        return CacheSpec("state", shape=(self.heads, self.dv, self.d), dtype="float32")

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        return [TensorSpec(p + "q", (self.qk, H)), TensorSpec(p + "k", (self.qk, H)), TensorSpec(p + "v", (self.inner, H)),
                TensorSpec(p + "g", (self.inner, H)), TensorSpec(p + "o", (H, self.inner))]

    def bind(self, store):
        p = self.prefix
        self.w_in = store.matrices([p + n for n in ("q", "k", "v", "g")])
        self.w_o = store.matrix(p + "o")

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("a recurrent mixer keeps a state of its own: it cannot read one another run left")
        T, dev = x.shape[0], x.device
        u = matmul_tn(x, self.w_in, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        o = workspace.empty((T, self.inner), torch.float32, dev)
        ops.matrix_rnn("retention", u, cache.state, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, o, heads=self.heads, d=self.d,
                       dv=self.dv, q_col=0, k_col=self.qk, v_col=2 * self.qk, decay=self.decay, ctx_len=ctx.ctx_len,
                       freq=self.freq, rot=self.rot, interleaved=self.interleaved)
        return self._read_out(o, u, 2 * self.qk + self.inner, ctx, x.dtype)
