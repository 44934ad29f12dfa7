"""Grouped-query attention without rotation, for designs that tell positions apart by distance:

    u = W [q; k; v] x + b                         (one stacked product)
    u'_t = sum_j c[:, j] u_(t - taps + 1 + j)     a short causal convolution per channel, zero before the first token
    q, k  <-  each head divided by its root mean square over the head (no gain; eps inside the root)
    s_ij = scale * (q_i . k_j) - a_h ln(1 + b_h (i - j))
    i sees j  iff  j <= i and (i - j < window or j < keep_first)
    softmax over the visible keys, weighted sum of the values, output projection.

Query head h reads key/value head h // (heads / kv_heads); keys have ``head_dim`` lanes, values ``v_head_dim``.  The
first ``keep_first`` keys of a request stay visible at their true distances.  Every option can be switched off (no
bias, no convolution, no norm, no penalty, no window), so the part serves other designs of this family.  Further
options, all off unless asked for:

    ``whole_norm``      q <- g_q * q / rms(q) over all of a token's query lanes at once (before they are split into
                        heads), with a gain per lane; the same for its key lanes (instead of the per-head unit norm)
    ``softcap`` c       s <- c tanh(s / c) on the scaled score, before any distance term
    ``slope_exponent`` a   slope_h (i - j) is taken off the score, slope_h = 2^(-a (h + 1) / heads)
    ``sink``            a silent key of score 0 and no value in every softmax: w_j = exp(s_j) / (1 + sum_j exp(s_j))

Per request the part keeps the keys and values in pages (given back as the window passes, except the pages of the
kept first keys) and, for the convolution, the last taps - 1 rows of the stacked projection as a fixed-size state.
Scores, softmax, the penalty, the norms and the convolution are 32-bit; keys, values and queries are stored in the
compute dtype.  In bfloat16 with keys and values of 64 or 128 lanes the scores and the weighted sums run on the
tensor cores (the kernels of the rotary attention part, with these options: tcgen05 for prompt portions where the
page size allows, mma.sync for decoded tokens); otherwise on the plain kernel.
"""
from __future__ import annotations

import os

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .attention import (CLUSTER_MERGE, DECODE_ROWS, MMA_DECODE_ROWS, MMA_SPAN_ROWS, SPAN_ROWS, TCGEN05_SPANS,
                        AttentionPlan)
from .base import CacheSpec, Mixer
from .linear import matmul_tn


# 0 keeps every step on the plain attention kernel (comparison runs, tests)
MMA_ATTENTION = os.environ.get("VLLM_CPP_B200_WINDOW_ATTN_MMA", "1") != "0"
# whether the tensor-core kernels take the cap, the slope and the sink (else steps with them run on the plain kernel)
EXTRAS_ON_TENSOR_CORES = True
# whether they take a sink with a learned score per head (else such steps run on the plain kernel)
SINK_SCORES_ON_TENSOR_CORES = True


def paged_attention(ctx, kv, q, out, *, nh, nkv, hd, vd, scale, window=0, keep_first=0, dist_a=None, dist_b=None,
                    softcap=0.0, slope=None, sink=False):
    """(``sink``: False, True -- a silent key of score 0 --, or a float32 tensor [nh] of the silent key's score per head.)
    Scores, softmax and weighted sums of one step over the paged keys and values ``kv``: ``q`` [T, nh * hd] against
    keys of ``hd`` lanes, values of ``vd`` lanes into ``out`` [T, nh * vd].  Single tokens are cut into key slices and
    merged, prompt portions into row tiles; bfloat16 with keys and values of 64 or 128 lanes runs on the tensor cores
    (tcgen05 for prompt portions where the page size allows, mma.sync for decoded tokens), everything else on the
    plain kernel.  Whoever keeps its keys in pages of this layout calls this (the window attention below; attention
    over latent rows, whose one KV head's values are the first lanes of its keys)."""
    x = q
    # no query reads more keys than the window and the kept first ones: no more key slices than those fill
    reach = window + keep_first if window else 0
    # bfloat16 with keys and values of 64 or 128 lanes: the tensor-core kernel; else the plain one
    extras = dict(softcap=softcap, slope=slope, sink=sink)
    learned_sink = torch.is_tensor(sink)
    has_extras = bool(softcap or slope is not None or learned_sink or sink)
    mma = (MMA_ATTENTION and vd == hd and kv.pages.dim() == 5 and ops.attn_mma_supported(x.dtype, hd)
           and (EXTRAS_ON_TENSOR_CORES or not has_extras) and (SINK_SCORES_ON_TENSOR_CORES or not learned_sink))
    dec_rows, span_rows = (MMA_DECODE_ROWS, MMA_SPAN_ROWS) if mma else (DECODE_ROWS, SPAN_ROWS)
    clustered = hd if mma and CLUSTER_MERGE and torch.cuda.is_available() else None
    group = ctx.groups[kv.group]
    plan = ctx.plan(("attention", nh, nkv, mma, clustered, reach),
                    lambda: AttentionPlan(ctx, nh, nkv, dec_rows, span_rows, clustered, max_keys=reach))
    common = dict(nh=nh, nkv=nkv, hd=hd, window=window, status=ctx.status, table_row=ctx.slots, scale=scale,
                  keep_first=keep_first, dist_a=dist_a, dist_b=dist_b, **extras)
    args = (q, out, kv.pages, group.block_table, ctx.q_start, ctx.q_len, ctx.ctx_len)
    if plan.n_dec:
        S = plan.nslices
        cluster = plan.cluster if mma else 0
        part_o = part_ml = None
        if S > 1 and not cluster:
            part_o = workspace.empty((plan.n_dec * nh * S, vd), torch.float32, x.device)
            part_ml = workspace.empty((plan.n_dec * nh * S, 2), torch.float32, x.device)
        if mma:
            ops.attn_mma(*args, plan.dec_items, plan.n_dec * S, dec_rows, part_o, part_ml,
                         slice_counters=plan.slice_counters if S > 1 else None, dec_rows=plan.dec_rows, cluster=cluster,
                         **common)
        else:
            ops.attn_window_bias(*args, plan.dec_items, plan.n_dec * S, dec_rows, part_o, part_ml, hd_v=vd, **common)
            if S > 1:
                ops.attn_merge(part_o, part_ml, plan.dec_rows, out, plan.n_dec, nh, vd, S)
    if plan.n_span_items:
        if mma and TCGEN05_SPANS and ops.attn_tc_supported(x.dtype, hd, kv.pages.shape[3]):
            ops.attn_tc(*args, plan.span_items, plan.n_span_items, work=plan.span_work, **common)
        elif mma:
            ops.attn_mma(*args, plan.span_items, plan.n_span_items, span_rows, None, None, **common)
        else:
            ops.attn_window_bias(*args, plan.span_items, plan.n_span_items, span_rows, None, None,
                                 hd_v=vd, **common)


class ConvWindowAttention(Mixer):
    """params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_head_dim`` (default head_dim),
    ``scale`` (default 1/sqrt(head_dim)), ``window`` (0: all keys), ``keep_first``, ``conv_taps`` (0: none), ``eps``,
    ``unit_norm`` (default True), ``distance_penalty`` (default True), ``bias`` (default True); ``whole_norm``,
    ``softcap``, ``slope_exponent``, ``sink`` (see above; default off).
    Tensors under ``<prefix>``: q [nh*hd, H], k [nkv*hd, H], v [nkv*vd, H], each with ``.b`` and ``.conv``
    [channels, taps]; r1, r2 [nh] (a_h, b_h); q.norm [nh*hd], k.norm [nkv*hd] (whole_norm); o [H, nh*vd]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.hd ** -0.5
        self.window = int(p.get("window") or 0)
        self.keep_first = int(p.get("keep_first") or 0) if self.window else 0
        self.taps = int(p.get("conv_taps") or 0)
        self.eps = float(p.get("eps", 1e-6))
        self.unit_norm = bool(p.get("unit_norm", True))
        self.penalty = bool(p.get("distance_penalty", True))
        self.has_bias = bool(p.get("bias", True))
        self.whole_norm = bool(p.get("whole_norm", False))
        self.softcap = float(p.get("softcap") or 0.0)
        self.slope_exponent = p.get("slope_exponent")
        self.sink = bool(p.get("sink", False))
        if self.whole_norm and (self.taps or self.has_bias):
            raise ValueError("the norm over the whole projection comes without a bias and without a convolution")
        if self.whole_norm:
            self.unit_norm = False
        if self.penalty and self.slope_exponent is not None:
            raise ValueError("a logarithmic distance penalty and a slope at once")
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} KV heads")
        for n in (self.hd, self.vd):
            if not 1 <= n <= 256:
                raise ValueError(f"head size {n} is not supported: the kernels take 1 to 256")
        self.channels = self.nh * self.hd + self.nkv * (self.hd + self.vd)
        self.w_qkv = self.w_o = self.bias = self.conv_w = self.dist_a = self.dist_b = None
        self.q_gain = self.k_gain = self.slope = None

    def cache_spec(self):
        kv = CacheSpec("kv", num_kv_heads=self.nkv, head_dim=self.hd, window=self.window, keep_first=self.keep_first,
                       v_head_dim=0 if self.vd == self.hd else self.vd)
        if self.taps > 1:
            return (kv, CacheSpec("state", shape=(self.taps - 1, self.channels), dtype="float32"))
        return kv

    def tensor_specs(self):
        p, H, nh, nkv, hd, vd = self.prefix, self.hidden, self.nh, self.nkv, self.hd, self.vd
        rows = (("q", nh * hd), ("k", nkv * hd), ("v", nkv * vd))
        specs = [TensorSpec(p + n, (r, H)) for n, r in rows] + [TensorSpec(p + "o", (H, nh * vd))]
        if self.has_bias:
            specs += [TensorSpec(p + n + ".b", (r,), "bias") for n, r in rows]
        if self.taps:
            specs += [TensorSpec(p + n + ".conv", (r, self.taps), "bias") for n, r in rows]
        if self.penalty:
            specs += [TensorSpec(p + "r1", (nh,), "positive"), TensorSpec(p + "r2", (nh,), "positive")]
        if self.whole_norm:
            specs += [TensorSpec(p + "q.norm", (nh * hd,), "vector"), TensorSpec(p + "k.norm", (nkv * hd,), "vector")]
        return specs

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        self.w_qkv = store.matrices([p + "q", p + "k", p + "v"])
        self.w_o = store.matrix(p + "o")
        if self.has_bias:
            self.bias = torch.cat([f32("q.b"), f32("k.b"), f32("v.b")]).contiguous()
        if self.taps:
            self.conv_w = torch.cat([f32("q.conv"), f32("k.conv"), f32("v.conv")], dim=0).contiguous()
        if self.penalty:
            self.dist_a, self.dist_b = f32("r1"), f32("r2")
        if self.whole_norm:
            self.q_gain, self.k_gain = f32("q.norm"), f32("k.norm")
        if self.slope_exponent is not None:
            # 2^(-a (h + 1) / heads): 64-bit on the host, rounded once
            h = torch.arange(1, self.nh + 1, dtype=torch.float64)
            self.slope = torch.pow(2.0, -float(self.slope_exponent) * h / self.nh).to(torch.float32).to(self.build.device)

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("this attention part keeps its own keys: it cannot read a cache another run filled")
        kv, st = (cache[0], cache[1].state) if isinstance(cache, tuple) else (cache, None)
        T = x.shape[0]
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        group = ctx.groups[kv.group]
        qkv = matmul_tn(x, self.w_qkv, ctx.status, out_dtype=torch.float32, allow_partials=True)
        q = workspace.empty((T, nh * hd), x.dtype, x.device)
        if self.whole_norm:
            ops.qkv_wholenorm_store(qkv, self.q_gain, self.k_gain, self.eps, ctx.q_start, ctx.q_len, group.slot_map, ctx.E,
                                    q, kv.pages, nh, nkv, hd, vd, ctx.status)
        else:
            ops.qkv_conv_norm_store(qkv, self.bias, self.conv_w, st, ctx.q_start, ctx.q_len, ctx.slots, group.slot_map, ctx.E,
                                    q, kv.pages, nh, nkv, hd, vd, self.eps, ctx.status, use_norm=self.unit_norm)
        if self.taps > 1 and any(n > 1 for n in ctx.host_q_len):
            # (entries of one token were brought up to date by the kernel above)
            ops.conv_state_update(qkv, st, ctx.q_start, ctx.q_len, ctx.slots, ctx.E, bias=self.bias)
        out = workspace.empty((T, nh * vd), x.dtype, x.device)
        paged_attention(ctx, kv, q, out, nh=nh, nkv=nkv, hd=hd, vd=vd, scale=self.scale, window=self.window,
                        keep_first=self.keep_first, dist_a=self.dist_a, dist_b=self.dist_b, softcap=self.softcap,
                        slope=self.slope, sink=self.sink)
        return matmul_tn(out, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True)


def rotary_frequencies(build, base: float, dims: int) -> torch.Tensor:
    """base^(-2i / dims), i < dims / 2: 64-bit on the host, rounded once to 32-bit, shared by parts with equal numbers."""
    key = ("rotary_freq", float(base), int(dims))
    if key not in build.shared:
        i = torch.arange(dims // 2, dtype=torch.float64)
        build.shared[key] = (float(base) ** (-2.0 * i / dims)).to(torch.float32).to(build.device)
    return build.shared[key]


class RotaryWindowAttention(Mixer):
    """Grouped-query softmax attention with rotary positions, every variation a parameter:

        q, k, v = W_q x, W_k x, W_v x                 (one stacked product; no biases)
        ``values_from_keys``: there is no W_v; v = k as projected, before any norm or rotation (v_head_dim = head_dim)
        ``whole_norm``:       q <- g_q * q / rms(q) over all of a token's query lanes at once, k likewise with g_k
        the first ``rotary_dim`` lanes of every q and k head turn by position * base^(-2i / rotary_dim), lanes paired
        in halves (i, i + rotary_dim/2; ``pairing`` "half") or as neighbours (2i, 2i+1; "interleaved")
        ``rotate_values``:    the value of position j turns by j over all its lanes (same pairing, frequencies
                              base^(-2m / v_head_dim)) and is cached so; a head's weighted sum at position i is turned
                              back by i, which leaves every value turned by j - i
        s_ij = scale * (q_i . k_j);  i sees j iff 0 <= i - j < window (window 0: every j <= i)
        ``sink``:             exp(sink_h), a learned score per head that is not scaled, joins the softmax's denominator
        softmax, weighted sum of the values, output projection.

    params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``v_head_dim`` (default head_dim), ``scale``,
    ``window``, ``rope_base``, ``rotary_dim``, ``pairing``, ``eps`` and the flags above (all default False).
    Tensors under ``<prefix>``: q [nh hd, H], k [nkv hd, H], v [nkv vd, H] (unless values_from_keys), o [H, nh vd];
    q.norm [nh hd], k.norm [nkv hd] (whole_norm); sink [nh] (sink).

    Norms, angles, scores and softmax are 32-bit; queries, keys and values are stored in the compute dtype.  Keys and
    values lie in pages that are given back as the window passes."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden = int(p["hidden_size"])
        self.nh, self.nkv, self.hd = int(p["num_heads"]), int(p["num_kv_heads"]), int(p["head_dim"])
        self.vd = int(p.get("v_head_dim") or self.hd)
        self.scale = float(p["scale"]) if p.get("scale") is not None else self.hd ** -0.5
        self.window = int(p.get("window") or 0)
        self.eps = float(p.get("eps", 1e-6))
        self.rot = int(p.get("rotary_dim") if p.get("rotary_dim") is not None else self.hd)
        self.interleaved = str(p.get("pairing") or "half") == "interleaved"
        if str(p.get("pairing") or "half") not in ("half", "interleaved"):
            raise ValueError(f"rotary pairing '{p.get('pairing')}' is not one of 'half', 'interleaved'")
        self.values_from_keys = bool(p.get("values_from_keys", False))
        self.whole_norm = bool(p.get("whole_norm", False))
        self.rotate_values = bool(p.get("rotate_values", False))
        self.has_sink = bool(p.get("sink", False))
        if self.nh % self.nkv:
            raise ValueError(f"{self.nh} query heads are not a multiple of {self.nkv} KV heads")
        if self.values_from_keys and self.vd != self.hd:
            raise ValueError("keys that double as values have the keys' size")
        if self.rot % 2 or not 0 <= self.rot <= self.hd:
            raise ValueError(f"{self.rot} turning lanes in heads of {self.hd}: an even number up to the head size")
        if self.rotate_values and self.vd % 2:
            raise ValueError(f"values of {self.vd} lanes cannot turn in pairs")
        for n in (self.hd, self.vd):
            if not 1 <= n <= 256:
                raise ValueError(f"head size {n} is not supported: the kernels take 1 to 256")
        base = float(p.get("rope_base", 10000.0))
        self.freq = rotary_frequencies(build, base, self.rot) if self.rot else None
        self.vfreq = rotary_frequencies(build, base, self.vd) if self.rotate_values else None
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = self.sink = None

    def cache_spec(self):
        return CacheSpec("kv", num_kv_heads=self.nkv, head_dim=self.hd, window=self.window,
                         v_head_dim=0 if self.vd == self.hd else self.vd)

    def _rows(self):
        rows = [("q", self.nh * self.hd), ("k", self.nkv * self.hd)]
        return rows if self.values_from_keys else rows + [("v", self.nkv * self.vd)]

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        specs = [TensorSpec(p + n, (r, H)) for n, r in self._rows()] + [TensorSpec(p + "o", (H, self.nh * self.vd))]
        if self.whole_norm:
            specs += [TensorSpec(p + "q.norm", (self.nh * self.hd,), "vector"), TensorSpec(p + "k.norm", (self.nkv * self.hd,), "vector")]
        if self.has_sink:
            specs.append(TensorSpec(p + "sink", (self.nh,), "bias"))
        return specs

    def bind(self, store):
        p = self.prefix
        f32 = lambda name: store.vector(p + name).float().contiguous()
        self.w_qkv = store.matrices([p + n for n, _ in self._rows()])
        self.w_o = store.matrix(p + "o")
        if self.whole_norm:
            self.q_gain, self.k_gain = f32("q.norm"), f32("k.norm")
        if self.has_sink:
            self.sink = f32("sink")

    def forward(self, x, ctx, cache, writes=True):
        if not writes:
            raise ValueError("this attention part keeps its own keys: it cannot read a cache another run filled")
        kv = cache
        T = x.shape[0]
        nh, nkv, hd, vd = self.nh, self.nkv, self.hd, self.vd
        group = ctx.groups[kv.group]
        qkv = matmul_tn(x, self.w_qkv, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        q = workspace.empty((T, nh * hd), x.dtype, x.device)
        ops.qkv_rope_store(qkv, self.q_gain, self.k_gain, self.eps, ctx.positions, self.freq, self.vfreq, group.slot_map, q,
                           kv.pages, nh, nkv, hd, vd, ctx.status, rot=self.rot, interleaved=self.interleaved,
                           values_from_keys=self.values_from_keys)
        out = workspace.empty((T, nh * vd), x.dtype, x.device)
        paged_attention(ctx, kv, q, out, nh=nh, nkv=nkv, hd=hd, vd=vd, scale=self.scale, window=self.window,
                        sink=self.sink if self.has_sink else False)
        if self.rotate_values:
            ops.rotate_heads(out, ctx.positions, self.vfreq, heads=nh, width=vd, dims=vd, interleaved=self.interleaved, sign=-1.0)
        return matmul_tn(out, self.w_o, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
