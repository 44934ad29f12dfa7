"""Several mixers side by side on the same input, their results normed and averaged:

    out = 1/N sum_b gain_b * y_b / sqrt(mean(y_b^2) + eps),   y_b = mixer_b(x)

each result normed over the model width with a plain gain of its own (ops.branch_norm_mean, 32-bit, straight from the
output projections' sums or k-slice partial sums).  The branches are mixers of any kind, named in the parameters like a
layer names its parts; what they keep per request (pages, fixed-size states) is kept side by side, each branch handed
its own views.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..registry import part_class
from ..weights.loader import TensorSpec
from .base import Mixer


class NormedBranchesMixer(Mixer):
    """params: ``hidden_size``, ``eps``, ``branches``: a list of (PartSpec of family mixer, sub-prefix, name of the
    branch's gain tensor under this part's prefix), up to four.  Tensors: the branches' own under ``<prefix><sub-prefix>``
    and a gain [hidden] each."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.hidden = int(params["hidden_size"])
        self.eps = float(params.get("eps", 1e-6))
        self.branches, self.gain_names = [], []
        for spec, sub, gain in params["branches"]:
            self.branches.append(part_class("mixer", spec.kind)(spec.params, prefix + sub, build))
            self.gain_names.append(prefix + gain)
        if not 1 <= len(self.branches) <= 4:
            raise ValueError(f"{len(self.branches)} branches (1 to 4)")
        self.gains = None

    @property
    def capturable(self):
        return all(getattr(b, "capturable", True) for b in self.branches)

    def tensor_specs(self):
        return ([s for b in self.branches for s in b.tensor_specs()]
                + [TensorSpec(n, (self.hidden,), "vector") for n in self.gain_names])

    def bind(self, store):
        for b in self.branches:
            b.bind(store)
        self.gains = [store.vector(n).float().contiguous() for n in self.gain_names]

    def _specs(self):
        """Per branch, what it keeps, as a tuple (maybe empty)."""
        out = []
        for b in self.branches:
            s = b.cache_spec()
            out.append(() if s is None else (s if isinstance(s, tuple) else (s,)))
        return out

    def cache_spec(self):
        flat = tuple(s for per in self._specs() for s in per)
        return flat or None

    def forward(self, x, ctx, cache, writes=True):
        views = () if cache is None else (cache if isinstance(cache, tuple) else (cache,))
        results, at = [], 0
        for b, per in zip(self.branches, self._specs()):
            mine = views[at:at + len(per)]
            at += len(per)
            own = b.cache_spec()
            handed = mine if isinstance(own, tuple) else (mine[0] if mine else None)
            results.append(b.forward(x, ctx, handed, writes))
        out = workspace.empty((x.shape[0], self.hidden), torch.float32, x.device)
        ops.branch_norm_mean([r if r.dtype == torch.float32 else r.float() for r in results], self.gains, self.eps, out)
        return out
