"""Attention whose keys and values are expanded from one small latent vector per token:

    c_q = g_q n(W_dq x)                 q = W_uq c_q               per head [d plain lanes | r rotated lanes]
    [c' | k_r] = W_dkv x                c = g_kv n(c')             c: kv_rank lanes; k_r: r lanes, one key part for all heads
    k_h = [W_uk[h] c | rot(k_r)]        v_h = W_uv[h] c
    s_ij = scale * (q_i,plain . k_j,plain + rot(q_i,r) . rot(k_j,r)),   causal softmax,   out = W_o [heads' sums]

n(v) = v / sqrt(mean(v^2) + eps).  Only c and the rotated key part are kept per token.  Since
q_plain . (W_uk[h] c) = (W_uk[h]^T q_plain) . c and sum_j w_j W_uv[h] c_j = W_uv[h] sum_j w_j c_j, the queries are carried
into the latent space and attention runs over the cached rows themselves: one shared KV head whose keys are
[c | rot(k_r)] (kv_rank + r lanes) and whose values are c; the heads' values are expanded from the weighted latent sums
afterwards.  The step's cost per key no longer depends on the heads' own sizes, and nothing is expanded per cached token.

Rotation pairs lane i with lane i + r/2; the angle is position * f_i in 32-bit.  The frequencies f_i may be stretched
(``rope_frequencies``): f_i / factor for pairs that turn slowly, f_i for those that turn fast, a linear ramp between,
and cos and sin times 0.1 ln(factor) + 1.  ``scale`` is used as given.  Norms, angles, scores and softmax are 32-bit;
the latent rows, the queries and the expanded values are stored in the compute dtype.

Where the attention kernels on the tensor cores take the key rows' width (bfloat16, kv_rank + r of 64 or 128 lanes),
the value rows are stored as wide as the key rows, [c | zeros]: those kernels read keys and values of one width.  The
weighted sums then carry r lanes of zeros that the expansion skips; the cache grows by r lanes a token.
"""
from __future__ import annotations

import math

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import CacheSpec, Mixer
from .linear import matmul_tn
from .window_attention import MMA_ATTENTION, paged_attention


def rope_frequencies(dims: int, base: float, scaling: dict | None = None):
    """-> (the dims/2 frequencies as 64-bit floats, the factor on cos and sin).  ``scaling`` (or None): ``factor``,
    ``original`` (the length the plain frequencies were meant for), ``fast`` and ``slow`` (turns over that length above
    which a pair is left alone, and below which it is slowed by ``factor``)."""
    half = dims // 2
    f = [float(base) ** (-2.0 * i / dims) for i in range(half)]
    if not scaling or not scaling.get("factor"):
        return f, 1.0
    factor, orig = float(scaling["factor"]), float(scaling["original"])

    def pair_of(turns: float) -> float:      # the (fractional) pair that makes this many turns over the original length
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(float(base)))

    lo = max(math.floor(pair_of(float(scaling["fast"]))), 0)
    hi = min(math.ceil(pair_of(float(scaling["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


class LatentAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``head_dim`` (plain lanes d), ``rot_dim`` (r, even), ``v_head_dim``,
    ``q_rank``, ``kv_rank``, ``scale``, ``eps``, ``rope_base``, ``rope_scaling`` (None or factor/original/fast/slow).
    Tensors under the prefix: ``dq`` [q_rank, H], ``dq.norm`` [q_rank], ``uq`` [heads (d + r), q_rank], ``dkv``
    [kv_rank + r, H], ``dkv.norm`` [kv_rank], ``uk`` [heads d, kv_rank], ``uv`` [heads vd, kv_rank], ``o`` [H, heads vd]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden, self.nh = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.r, self.vd = int(p["head_dim"]), int(p["rot_dim"]), int(p["v_head_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale, self.eps = float(p["scale"]), float(p.get("eps", 1e-6))
        if self.r % 2:
            raise ValueError(f"{self.r} rotated lanes: lanes turn in pairs")
        self.khd = self.kv_rank + self.r          # lanes of a cached key row
        if not 1 <= self.khd <= 256:
            raise ValueError(f"a latent of {self.kv_rank} lanes with {self.r} rotated ones: the attention kernels take "
                             f"key rows of up to 256 lanes")
        freqs, self.rope_gain = rope_frequencies(self.r, float(p.get("rope_base", 10000.0)), p.get("rope_scaling")) \
            if self.r else ([], 1.0)
        self.freq = torch.tensor(freqs or [0.0], dtype=torch.float64).to(torch.float32).to(build.device)
        # lanes of a cached value row: as many as a key row's where the tensor-core kernels then take both
        wide = (MMA_ATTENTION and self.r and build.compute_dtype == torch.bfloat16
                and ops.attn_mma_supported(build.compute_dtype, self.khd))
        self.vw = self.khd if wide else self.kv_rank
        self.w_down = self.w_uq = self.w_o = self.m_uk = self.m_uv = self.q_gain = self.kv_gain = None

    def cache_spec(self):
        return CacheSpec("kv", num_kv_heads=1, head_dim=self.khd, v_head_dim=0 if self.vw == self.khd else self.vw)

    def tensor_specs(self):
        p, H, nh = self.prefix, self.hidden, self.nh
        return [TensorSpec(p + "dq", (self.q_rank, H)), TensorSpec(p + "dq.norm", (self.q_rank,), "vector"),
                TensorSpec(p + "uq", (nh * (self.d + self.r), self.q_rank)),
                TensorSpec(p + "dkv", (self.khd, H)), TensorSpec(p + "dkv.norm", (self.kv_rank,), "vector"),
                TensorSpec(p + "uk", (nh * self.d, self.kv_rank)), TensorSpec(p + "uv", (nh * self.vd, self.kv_rank)),
                TensorSpec(p + "o", (H, nh * self.vd))]

    def bind(self, store):
        p = self.prefix
        self.w_down = store.matrices([p + "dq", p + "dkv"])       # both down projections read the same rows: one product
        self.w_uq, self.w_o = store.matrix(p + "uq"), store.matrix(p + "o")
        # head h's small matrices, [h][out][in]: W_uk[h]^T carries a query into the latent space, W_uv[h] a latent sum out
        self.m_uk = store.matrix(p + "uk").view(self.nh, self.d, self.kv_rank).transpose(1, 2).contiguous()
        self.m_uv = store.matrix(p + "uv").view(self.nh, self.vd, self.kv_rank).contiguous()
        self.q_gain = store.vector(p + "dq.norm").float().contiguous()
        self.kv_gain = store.vector(p + "dkv.norm").float().contiguous()

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("this attention part keeps its own latent rows: it cannot read a cache another run filled")
        kv = cache
        T, dev, dt = x.shape[0], x.device, x.dtype
        nh, d, r, vd, kr, khd = self.nh, self.d, self.r, self.vd, self.kv_rank, self.khd
        group = ctx.groups[kv.group]
        u = matmul_tn(x, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        cq = workspace.empty((T, self.q_rank), dt, dev)
        ops.latent_norm_rope_store(u, self.q_gain, self.kv_gain, self.eps, ctx.positions, self.freq, self.rope_gain,
                                   group.slot_map, cq, kv.pages, group.page_size, self.q_rank, kr, r, ctx.status, v_width=self.vw)
        q = matmul_tn(cq, self.w_uq, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        ql = workspace.empty((T, nh * khd), dt, dev)
        ops.head_linear(q, self.m_uk, ql, heads=nh, n_in=d, n_out=kr, in_head_stride=d + r, out_head_stride=khd)
        if r:
            ops.rope_rows(q, ctx.positions, self.freq, self.rope_gain, ql, heads=nh, dims=r, width=r, in_head_stride=d + r,
                          in_off=d, out_head_stride=khd, out_off=kr)
        lat = workspace.empty((T, nh * self.vw), dt, dev)
        paged_attention(ctx, kv, ql, lat, nh=nh, nkv=1, hd=khd, vd=self.vw, scale=self.scale)
        heads = workspace.empty((T, nh * vd), dt, dev)
        ops.head_linear(lat, self.m_uv, heads, heads=nh, n_in=kr, n_out=vd, in_head_stride=self.vw, out_head_stride=vd)
        return matmul_tn(heads, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
