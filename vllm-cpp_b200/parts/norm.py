"""RMSNorm: y = w * x / sqrt(mean(x^2) + eps), the gain multiplying directly
(src/model.cpp:924-930), fused with the addition of the pending delta into the
32-bit residual stream (the reference adds separately, src/model.cpp:1226-1227, 1248-1250)."""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Norm


class RMSNorm(Norm):
    """params: ``size``, ``eps``; optional ``name`` (default "weight"); ``one_plus`` (default False): the tensor holds the
    gain less one (values around zero), y = (1 + w) * x / sqrt(mean(x^2) + eps), the sum made in 32-bit.
    Tensor: ``<prefix><name>`` [size]."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.size = int(params["size"])
        self.eps = float(params["eps"])
        self.name = self.prefix + str(params.get("name", "weight"))
        self.one_plus = bool(params.get("one_plus", False))
        self.weight = None
        self._gain32 = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.size,), "bias" if self.one_plus else "vector")]

    def bind(self, store):
        self.weight = store.vector(self.name)
        if self.one_plus:
            self.weight = (1.0 + self.weight.float()).contiguous()

    def gain32(self):
        """The gain as a 32-bit vector (made once): what the kernels that fuse this norm with other steps read."""
        if self._gain32 is None:
            self._gain32 = self.weight.float().contiguous()
        return self._gain32

    def forward(self, resid, delta, rows=None):
        n = resid.shape[0] if rows is None else rows.numel()
        out = workspace.empty((n, self.size), self.build.compute_dtype, resid.device)
        if delta is not None and not torch.is_tensor(delta):
            # what the arrangement before left is more than a sum to add (a result still to be normed and scaled, say):
            # it knows the kernel that does its addition and this norm in one pass
            delta.add_then_norm(resid, self.gain32(), self.eps, out, rows)
            return out
        ops.add_rmsnorm(resid, delta, self.weight, self.eps, out, rows)
        return out
