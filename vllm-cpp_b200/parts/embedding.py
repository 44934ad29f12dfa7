"""Token embedding (x[t,:] = E[id_t,:], src/model.cpp:1157-1163) and the LM head
(logits = y . W^T in 32-bit, W the head matrix or the embedding table when they
are tied, src/model.cpp:560-566, 1260-1263).

Both are parts like any other, found through the registry (families ``embedding``
and ``head``), so that an architecture whose embedding is scaled, whose head has
a bias or caps its logits, registers its own without a change here.

``embedding``  ``forward(ids, n_tokens, status) -> [n_tokens, hidden]`` 32-bit, the
               start of the residual stream; ``table`` is what a tied head shares.
``head``       ``attach(embedding)`` once after both are built, then
               ``forward(y, status) -> [rows, vocab]`` 32-bit logits.
"""
from __future__ import annotations

import torch

from .. import ops, workspace
from ..weights.loader import TensorSpec
from .base import Part
from .linear import matmul_tn


class Embedding(Part):
    family = "embedding"
    table = None

    def forward(self, ids, n_tokens, status):
        raise NotImplementedError


class Head(Part):
    family = "head"

    def attach(self, embedding) -> None:
        """Called once, after the model's embedding part exists (a tied head takes its table from there)."""

    def forward(self, y, status=None):
        raise NotImplementedError


class TokenEmbedding(Embedding):
    """params: ``tensor`` (checkpoint name of the table), ``vocab_size``, ``hidden_size``; optional ``row_scale`` (default 1):
    a constant on the gathered row (a tied head reads the table itself, without it)."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.name, self.vocab, self.hidden = str(params["tensor"]), int(params["vocab_size"]), int(params["hidden_size"])
        self.scale = float(params.get("row_scale", 1.0))
        self.table = None

    def tensor_specs(self):
        return [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        self.table = store.matrix(self.name)

    def forward(self, ids, n_tokens, status):
        out = workspace.empty((n_tokens, self.hidden), torch.float32, ids.device)
        if self.scale != 1.0:
            ops.embed_scaled_pos(self.table, ids, None, None, self.scale, out, status)
        else:
            ops.embed_gather(self.table, ids, out, status)
        return out


class SinusoidalTokenEmbedding(TokenEmbedding):
    """x[t] = E[id_t] + s(p_t): a sinusoid of the token's position is added to its embedding, entry 2i of s(p) being
    sin(p * base^(-2i/hidden)) and entry 2i+1 the cosine of the same angle.  The frequencies are computed in 64-bit
    on the host and rounded once; angles, sines and cosines are 32-bit on the device, so no table bounds the positions.

    params: ``tensor``, ``vocab_size``, ``hidden_size``, ``base`` (default 10000)."""
    uses_positions = True      # the model hands forward the tokens' positions too

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.base = float(params.get("base", 10000.0))
        key = ("sinusoid_freq", self.hidden, self.base)
        if key not in build.shared:
            i = torch.arange((self.hidden + 1) // 2, dtype=torch.float64)
            build.shared[key] = (self.base ** (-2.0 * i / self.hidden)).to(torch.float32).to(build.device)
        self.inv_freq = build.shared[key]

    def forward(self, ids, n_tokens, status, positions=None):
        if positions is None:
            raise ValueError("this embedding adds a position term: it needs the tokens' positions")
        out = workspace.empty((n_tokens, self.hidden), torch.float32, ids.device)
        ops.embed_sinusoid(self.table, ids, positions, self.inv_freq, out, status)
        return out


class PositionalTokenEmbedding(TokenEmbedding):
    """x[t] = scale * E[id_t] + P[p_t]: the token's embedding times a constant, plus a learned vector for its position
    (not scaled).  The table of positions bounds a request's length.

    params: ``tensor``, ``position_tensor``, ``vocab_size``, ``hidden_size``, ``max_positions``, ``scale`` (default 1)."""
    uses_positions = True

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.pos_name = str(params["position_tensor"])
        self.max_positions = int(params["max_positions"])
        self.scale = float(params.get("scale", 1.0))
        self.pos_table = None

    def tensor_specs(self):
        return super().tensor_specs() + [TensorSpec(self.pos_name, (self.max_positions, self.hidden))]

    def bind(self, store):
        super().bind(store)
        self.pos_table = store.matrix(self.pos_name)

    def forward(self, ids, n_tokens, status, positions=None):
        if positions is None:
            raise ValueError("this embedding adds a position vector: it needs the tokens' positions")
        out = workspace.empty((n_tokens, self.hidden), torch.float32, ids.device)
        ops.embed_scaled_pos(self.table, ids, positions, self.pos_table, self.scale, out, status)
        return out


class LMHead(Head):
    """params: ``tensor`` (checkpoint name of the head matrix, or None: the embedding table is the head),
    ``vocab_size``, ``hidden_size``; optional ``softcap`` c > 0: logits <- c tanh(logits / c)."""

    def __init__(self, params, prefix, build):
        super().__init__(params, prefix, build)
        self.name = params.get("tensor")
        self.vocab, self.hidden = int(params["vocab_size"]), int(params["hidden_size"])
        self.softcap = float(params.get("softcap") or 0.0)
        self.embedding = None
        self.weight = None

    def attach(self, embedding):
        self.embedding = embedding

    def tensor_specs(self):
        return [] if self.name is None else [TensorSpec(self.name, (self.vocab, self.hidden))]

    def bind(self, store):
        if self.name is None:
            if self.embedding is None or self.embedding.table is None:
                raise ValueError("a tied LM head needs an embedding part that has a table")
            self.weight = self.embedding.table
        else:
            self.weight = store.matrix(self.name)

    def forward(self, y, status=None):
        logits = matmul_tn(y, self.weight, status, out_dtype=torch.float32, after_small_kernel=True)   # (after the last norm)
        if self.softcap > 0:
            ops.softcap(logits, self.softcap)
        return logits
