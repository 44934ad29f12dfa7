"""A feed-forward of many small experts, of which a router picks a few per token, plus an optional shared expert
that every token runs:

    z = W_r y  (32-bit sums)          the `top` experts with the largest logits are chosen
    w_e = sigmoid(z_e)                as it is ("sigmoid"), or the softmax over the chosen logits ("softmax")
    out = sum_e expert_e(w_e y) + shared(y)        expert(v) = W_down act(W_up v), no biases

Options: ``gated`` experts, expert(v) = W_down (act(W_gate v) * (W_up v)), gate and up as one stacked product whose rows
alternate; and the router "grouped_sigmoid": s = sigmoid(z), the choice score is s + ``correction`` (a learned vector),
the experts form ``router_groups`` equal groups of neighbours of which only the ``router_keep`` best can be chosen from
(a group's score is the sum of its two largest choice scores), the ``top`` largest choice scores win, and a chosen
expert's weight is s * ``router_scale`` (without the correction, not renormalised).

The weight multiplies what the expert reads (``weight_on`` "input": the product w_e y is rounded to the compute dtype as
any stored activation) or what it returns ("output").  Nothing asks the host which expert got how many tokens: the
step's (token, choice) pairs are sorted by expert on the device into tiles of rows, each tile meeting one expert's
weights, and the grids are laid out for the most tiles the step can need -- so a captured step replays the part.
The router's rows ride on the shared expert's up projection (one product for both).
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import FeedForward
from .linear import matmul_tn


def grouped_tile_rows(n_pairs: int, n_experts: int) -> int:
    """Rows of a token tile of the grouped product: small tiles while an expert gets few of the step's pairs (a tile is
    padded to its size), the products' widest once the experts' runs are long."""
    avg = n_pairs / max(n_experts, 1)
    return 16 if avg <= 8 else (32 if avg <= 24 else (64 if avg <= 48 else 128))


class RoutedExperts(FeedForward):
    """params: ``hidden_size``, ``num_experts``, ``top``, ``expert_size`` (an expert's hidden size), ``shared_size`` (0:
    no shared expert), ``activation`` (default "relu2"), ``router_weights`` ("sigmoid" or "softmax"), ``weight_on``
    ("input" or "output"); ``gated`` (default False); ``router`` ("top_logits", the default, or "grouped_sigmoid" with
    ``router_groups`` (0: one group), ``router_keep``, ``router_scale`` (default 1), ``correction`` (default True)).
    Tensors under the prefix: ``router`` [E, H]; ``e<i>.up`` [F, H], ``e<i>.down`` [H, F]; ``e<i>.gate`` [F, H] (gated);
    ``correction`` [E]; ``shared.up`` [Fs, H], ``shared.down`` [H, Fs]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        p = params
        self.hidden, self.E, self.top = int(p["hidden_size"]), int(p["num_experts"]), int(p["top"])
        self.ff, self.sff = int(p["expert_size"]), int(p.get("shared_size") or 0)
        self.activation = str(p.get("activation", "relu2"))
        self.router_weights = str(p.get("router_weights", "sigmoid"))
        self.weight_on = str(p.get("weight_on", "input"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{self.activation}' is not one of {sorted(ops.ACTIVATIONS)}")
        if self.router_weights not in ("sigmoid", "softmax") or self.weight_on not in ("input", "output"):
            raise ValueError("router_weights is 'sigmoid' or 'softmax', weight_on 'input' or 'output'")
        if not 1 <= self.top <= self.E:
            raise ValueError(f"{self.top} of {self.E} experts")
        self.gated = bool(p.get("gated", False))
        self.router = str(p.get("router", "top_logits"))
        if self.router not in ("top_logits", "grouped_sigmoid"):
            raise ValueError("router is 'top_logits' or 'grouped_sigmoid'")
        self.groups, self.keep = int(p.get("router_groups") or 0), int(p.get("router_keep") or 0)
        self.router_scale = float(p.get("router_scale", 1.0))
        self.has_correction = self.router == "grouped_sigmoid" and bool(p.get("correction", True))
        if self.groups > 1 and (self.E % self.groups or not 1 <= self.keep <= self.groups
                                or self.keep * (self.E // self.groups) < self.top):
            raise ValueError(f"{self.groups} groups of which {self.keep} are kept cannot serve {self.top} of {self.E} experts")
        if self.gated and self.activation not in ("silu",):
            raise ValueError("gated experts use the SiLU gate")
        self.correction = None
        self.w_side = self.w_up = self.w_down = self.w_shared_down = None

    def tensor_specs(self):
        p, H = self.prefix, self.hidden
        specs = [TensorSpec(p + "router", (self.E, H))]
        for e in range(self.E):
            specs += [TensorSpec(f"{p}e{e}.up", (self.ff, H)), TensorSpec(f"{p}e{e}.down", (H, self.ff))]
            if self.gated:
                specs.append(TensorSpec(f"{p}e{e}.gate", (self.ff, H)))
        if self.has_correction:
            specs.append(TensorSpec(p + "correction", (self.E,), "bias"))
        if self.sff:
            specs += [TensorSpec(p + "shared.up", (self.sff, H)), TensorSpec(p + "shared.down", (H, self.sff))]
        return specs

    def bind(self, store):
        p = self.prefix
        if self.gated:
            # per expert gate_i in row 2i, up_i in row 2i + 1: the SiLU-gate reads neighbours
            self.w_up = torch.stack([store.matrices([f"{p}e{e}.gate", f"{p}e{e}.up"], interleave=True)
                                     for e in range(self.E)]).contiguous()
        else:
            self.w_up = store.matrices([f"{p}e{e}.up" for e in range(self.E)]).view(self.E, self.ff, self.hidden)
        if self.has_correction:
            self.correction = store.vector(p + "correction").float().contiguous()
        self.w_down = store.matrices([f"{p}e{e}.down" for e in range(self.E)]).view(self.E, self.hidden, self.ff)
        # the shared expert's up projection with the router's rows under it
        self.w_side = store.matrices(([p + "shared.up"] if self.sff else []) + [p + "router"])
        if self.sff:
            self.w_shared_down = store.matrix(p + "shared.down")

    def forward(self, x, ctx):
        T, H = x.shape
        dev, E, top, sff = x.device, self.E, self.top, self.sff
        side = matmul_tn(x, self.w_side, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        sel_e = workspace.empty((T, top), torch.int32, dev)
        sel_w = workspace.empty((T, top), torch.float32, dev)
        if self.router == "grouped_sigmoid":
            ops.moe_route_grouped(side[..., sff:], self.correction, self.groups, self.keep, self.router_scale, ctx.q_start,
                                  ctx.q_len, ctx.E, top, sel_e, sel_w)
        else:
            ops.moe_route(side[..., sff:], ctx.q_start, ctx.q_len, ctx.E, top, sel_e, sel_w,
                          softmax_weights=self.router_weights == "softmax")
        on_input = self.weight_on == "input"
        # bfloat16 with rows the TMA unit can address: the experts' products on the tensor cores, the tokens' rows
        # gathered (and weighted) in sorted order first; else the plain products, which read through the order
        tensor_cores = (self.activation in ("relu2", "silu") and self.ff % 8 == 0 and ops.gemm_grouped_ok(x, self.w_up)
                        and ops.gemm_grouped_ok(x, self.w_down))
        tile_rows = grouped_tile_rows(T * top, E) if tensor_cores else ops.moe_tile_rows()
        tiles = ops.moe_tiles_cap(T * top, E, tile_rows)
        rows = tiles * tile_rows
        pos_of = workspace.empty((T * top,), torch.int32, dev)
        src_of = workspace.empty((rows,), torch.int32, dev)
        tile_expert = workspace.empty((tiles,), torch.int32, dev)
        ops.moe_group(sel_e, E, tiles, pos_of, src_of, tile_expert, tile_rows)
        h1 = workspace.empty((rows, self.ff), x.dtype, dev)
        y = workspace.empty((rows, H), torch.float32, dev)
        # gated experts: the stacked product's 32-bit sums first, then the SiLU-gate over neighbouring columns
        gu = workspace.empty((rows, 2 * self.ff), torch.float32, dev) if self.gated else None
        if tensor_cores:
            xs = workspace.empty((rows, H), x.dtype, dev)
            ops.moe_gather(x, src_of, sel_w if on_input else None, top, xs)
            if self.gated:
                ops.gemm_bf16_grouped(self.w_up, xs, tile_expert, tile_rows, gu, ctx.status)
                ops.swiglu(gu, h1)
            else:
                ops.gemm_bf16_grouped(self.w_up, xs, tile_expert, tile_rows, h1, ctx.status, act=self.activation)
            ops.gemm_bf16_grouped(self.w_down, h1, tile_expert, tile_rows, y, ctx.status)
        else:
            if self.gated:
                ops.moe_gemm(x, self.w_up, tile_expert, gu, src_of=src_of, sel_w=sel_w if on_input else None, top=top)
                ops.swiglu(gu, h1)
            else:
                ops.moe_gemm(x, self.w_up, tile_expert, h1, src_of=src_of, sel_w=sel_w if on_input else None, top=top,
                             act=self.activation)
            ops.moe_gemm(h1, self.w_down, tile_expert, y)
        shared = None
        if sff:
            sa = workspace.empty((T, sff), x.dtype, dev)
            ops.bias_act(side[..., :sff], sa, self.activation)
            shared = matmul_tn(sa, self.w_shared_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        out = workspace.empty((T, H), torch.float32, dev)
        ops.moe_combine(y, pos_of, top, ctx.q_start, ctx.q_len, ctx.E, out, shared=shared, sel_w=None if on_input else sel_w)
        return out
