"""SwiGLU feed-forward: down(silu(gate(y)) * up(y)), silu(z) = z / (1 + exp(-z))
(src/model.cpp:964-966, 1237-1244), with separate input and output buffers for the
down projection.  gate and up become one [2I, H] matrix at load, gate_i in row 2i
and up_i in row 2i+1, so that one product yields both side by side: in the
tensor-core kernel the two land in adjacent accumulator lanes and the SiLU-gate
is a shuffle away in its epilogue."""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import FeedForward
import os

from .linear import choose_splits, matmul_tn

# The SiLU-gate runs in the gate-and-up product's epilogue when that product is not cut into k-slices (whose sums must
# exist before the SiLU): always where its units fill the SMs anyway (the 14B sizes, 272 feature tiles: 8 tokens
# 58.6 -> 56.5 us, 64 tokens 67.6 -> 60.1 against product and SiLU-gate kernel), and above this many tokens, from where
# the one kernel without slices is as fast as the two with them (8B sizes, 64 tokens: 45.8 against 45.7 us; 128: 51.1
# against 52.8; 32: 44.0 against 40.8) and the step has a kernel boundary less.
FUSE_ABOVE_TOKENS = int(os.environ.get("VLLM_CPP_B200_SWIGLU_FUSE_ABOVE", "63"))


class SwiGLUMLP(FeedForward):
    """params: ``hidden_size``, ``intermediate_size``.
    Tensors: ``<prefix>gate_proj.weight`` [I,H], ``up_proj.weight`` [I,H], ``down_proj.weight`` [H,I]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.w_gate_up = None
        self.w_down = None

    def tensor_specs(self):
        p, H, I = self.prefix, self.hidden, self.inter
        return [TensorSpec(p + "gate_proj.weight", (I, H)), TensorSpec(p + "up_proj.weight", (I, H)),
                TensorSpec(p + "down_proj.weight", (H, I))]

    def bind(self, store):
        p = self.prefix
        self.w_gate_up = store.matrices([p + "gate_proj.weight", p + "up_proj.weight"], interleave=True)
        self.w_down = store.matrix(p + "down_proj.weight")

    def forward(self, x, ctx):
        act = workspace.empty((x.shape[0], self.inter), x.dtype, x.device)
        T, K = x.shape
        if x.dtype == torch.bfloat16 and ops.gemm_tma_ok(x, self.w_gate_up) and (
                T > FUSE_ABOVE_TOKENS or ops.gemm_effective_splits(K, choose_splits(self.w_gate_up.shape[0], T, K)) == 1):
            # no k-slices are needed, or they no longer pay: the SiLU-gate runs in the product's epilogue
            ops.gemm_bf16_swiglu(self.w_gate_up, x, act, ctx.status, after_small_kernel=True)   # (after a norm)
        else:
            gate_up = matmul_tn(x, self.w_gate_up, ctx.status, allow_partials=True, after_small_kernel=True)   # (after a norm)
            ops.swiglu(gate_up, act)
            return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True)


class DenseMLP(FeedForward):
    """down(act(up(y))): one hidden layer, act the exact (erf) GELU unless ``activation`` names another
    ("gelu_erf", "gelu_tanh": 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))), "silu", or "polynorm": a n(z) + b n(z^2)
    + c n(z^3) + e with powers lane by lane, n(v) = v / sqrt(mean(v^2) + eps) over a token's hidden lanes and the four
    learned numbers a, b, c, e).  The hidden layer's sums and the activation are 32-bit; what the down projection reads
    is in the compute dtype.

    params: ``hidden_size``, ``intermediate_size``; optional ``activation``, ``up_tensor`` and ``down_tensor``
    (names under the prefix, default "up_proj.weight" and "down_proj.weight"); with "polynorm" also ``act_tensor``
    (default "act", a tensor [4]) and ``eps``."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "gelu_erf"))
        if self.activation not in ops.ACTIVATIONS and self.activation != "polynorm":
            raise ValueError(f"activation '{self.activation}' is not one of {sorted(ops.ACTIVATIONS) + ['polynorm']}")
        self.act_name = prefix + str(params.get("act_tensor", "act"))
        self.eps = float(params.get("eps", 1e-6))
        self.coef = None
        self.up_name = prefix + str(params.get("up_tensor", "up_proj.weight"))
        self.down_name = prefix + str(params.get("down_tensor", "down_proj.weight"))
        self.w_up = self.w_down = None
        self.side_rows = 0
        self.side = None

    def tensor_specs(self):
        specs = [TensorSpec(self.up_name, (self.inter, self.hidden)), TensorSpec(self.down_name, (self.hidden, self.inter))]
        if self.activation == "polynorm":
            specs.append(TensorSpec(self.act_name, (4,), "vector"))
        return specs

    def bind(self, store):
        self.w_up = store.matrix(self.up_name)
        self.w_down = store.matrix(self.down_name)
        if self.activation == "polynorm":
            self.coef = store.vector(self.act_name).float().contiguous()

    def attach_side_rows(self, weight) -> None:
        """Stacks ``weight`` [rows, hidden] under the up projection (after ``bind``): whoever else multiplies the part's
        input by a matrix gets its sums from the same product.  After ``forward`` they are in ``self.side``
        ([T, rows] or [S, T, rows] partial sums, 32-bit, a view)."""
        self.w_up = torch.cat([self.w_up, weight.to(self.w_up.dtype)], dim=0).contiguous()
        self.side_rows = int(weight.shape[0])

    def forward(self, x, ctx):
        u = matmul_tn(x, self.w_up, ctx.status, out_dtype=torch.float32, allow_partials=True)
        if self.side_rows:
            self.side = u[..., self.inter:]
            u = u[..., :self.inter]
        act = workspace.empty((x.shape[0], self.inter), x.dtype, x.device)
        if self.activation == "polynorm":
            ops.polynorm(u, self.coef, self.eps, act)
        else:
            ops.bias_act(u, act, self.activation)
        return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)


class GatedMLP(FeedForward):
    """down(act(gate(y) + b_g) * (up(y) + b_u)) + b_d: a feed-forward with a gate beside its up projection, any of the
    activations of ``ops.ACTIVATIONS``, and optional biases on all three projections.  gate and up are one stacked
    product (the gate's rows first); its sums, the biases and the activation are 32-bit.  The down projection's bias is
    not added here: the part offers it as ``output_bias`` to whoever adds the result to the stream.

    params: ``hidden_size``, ``intermediate_size``, ``activation`` (default "silu"), ``bias`` (default False), and the
    tensor names under the prefix ``gate_tensor``, ``up_tensor``, ``down_tensor`` (default "gate", "up", "down"; a bias is
    the matrix's name plus ".b")."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden = int(params["hidden_size"])
        self.inter = int(params["intermediate_size"])
        self.activation = str(params.get("activation", "silu"))
        if self.activation not in ops.ACTIVATIONS:
            raise ValueError(f"activation '{self.activation}' is not one of {sorted(ops.ACTIVATIONS)}")
        self.has_bias = bool(params.get("bias", False))
        self.names = tuple(prefix + str(params.get(k, d)) for k, d in (("gate_tensor", "gate"), ("up_tensor", "up"), ("down_tensor", "down")))
        self.w_gate_up = self.w_down = self.bias = self.output_bias = None

    def tensor_specs(self):
        g, u, d = self.names
        H, I = self.hidden, self.inter
        specs = [TensorSpec(g, (I, H)), TensorSpec(u, (I, H)), TensorSpec(d, (H, I))]
        if self.has_bias:
            specs += [TensorSpec(g + ".b", (I,), "bias"), TensorSpec(u + ".b", (I,), "bias"), TensorSpec(d + ".b", (H,), "bias")]
        return specs

    def bind(self, store):
        g, u, d = self.names
        self.w_gate_up = store.matrices([g, u])
        self.w_down = store.matrix(d)
        if self.has_bias:
            self.bias = torch.cat([store.vector(g + ".b").float(), store.vector(u + ".b").float()]).contiguous()
            self.output_bias = store.vector(d + ".b").float().contiguous()

    def forward(self, x, ctx):
        gu = matmul_tn(x, self.w_gate_up, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
        act = workspace.empty((x.shape[0], self.inter), x.dtype, x.device)
        ops.gated_act(gu, act, self.activation, self.bias)
        return matmul_tn(act, self.w_down, ctx.status, out_dtype=torch.float32, allow_partials=True, after_small_kernel=True)
