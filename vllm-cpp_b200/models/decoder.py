"""The generic decoder: embedding, a list of layers, the order they run in, final
norm, LM head -- built from a :class:`ModelSpec` through the part registries.

The forward pass follows the reference's layer loop (src/model.cpp:1176-1263)
with two generalisations that are data in the spec: the execution order is a
list of (layer, cache) runs, so a layer may run twice or read a cache another run
filled; and each layer names its own parts, so mixers and feed-forwards may
differ along the depth.  Final norm and LM head run only on the rows whose logits
were asked for (the reference: last position only, src/model.cpp:1255-1263).
"""
from __future__ import annotations

from .. import workspace
from ..parts.base import BuildContext, CacheSpec
from ..registry import ModelSpec, part_class
from ..weights.loader import TensorSpec, WeightStore


def _build_layer(lspec, build: BuildContext):
    parts = {}
    for role, entry in lspec.parts.items():
        pspec, sub = entry[0], entry[1]
        parts[role] = part_class(lspec.family_of(role), pspec.kind)(pspec.params, lspec.prefix + sub, build)
    return part_class("block", lspec.block.kind)(lspec.block.params, lspec.prefix, build, parts)


class DecoderModel:
    def __init__(self, spec: ModelSpec, build: BuildContext):
        self.spec = spec
        self.build = build
        emb, head = spec.embedding_spec(), spec.head_spec()
        self.embedding = part_class("embedding", emb.kind)(emb.params, "", build)
        self.layers = [_build_layer(l, build) for l in spec.layers]
        self.final_norm = None
        if spec.final_norm is not None:
            self.final_norm = part_class("norm", spec.final_norm.kind)(spec.final_norm.params, spec.final_norm_prefix, build)
        self.lm_head = part_class("head", head.kind)(head.params, "", build)
        self.lm_head.attach(self.embedding)
        self.reentry = None
        if spec.reentry is not None:
            self.reentry = part_class("reentry", spec.reentry.kind)(spec.reentry.params, "", build)
        self.order = list(spec.order)
        self._handed = None     # (the per-id views last given to forward, the same by run)
        for run in self.order:
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"the execution order names layer {run.layer}, the model has {len(self.layers)}")

    @property
    def capturable(self) -> bool:
        """Whether a decoding step of this model can be captured as a CUDA graph."""
        parts = [p for layer in self.layers for p in layer.parts.values()] + [self.embedding, self.lm_head]
        parts += [self.reentry] if self.reentry is not None else []
        return all(getattr(p, "capturable", True) for p in parts)

    # ---- weights ----
    def tensor_specs(self) -> list[TensorSpec]:
        specs = list(self.embedding.tensor_specs())
        for layer in self.layers:
            specs += layer.tensor_specs()
        if self.final_norm is not None:
            specs += self.final_norm.tensor_specs()
        if self.reentry is not None:
            specs += self.reentry.tensor_specs()
        return specs + self.lm_head.tensor_specs()

    def load(self, store: WeightStore) -> None:
        store.check(self.tensor_specs())
        self.embedding.bind(store)
        for layer in self.layers:
            layer.bind(store)
        if self.final_norm is not None:
            self.final_norm.bind(store)
        if self.reentry is not None:
            self.reentry.bind(store)
        self.lm_head.bind(store)

    # ---- caches ----
    def _run_specs(self) -> dict[int, object]:
        """cache id of the execution order -> what the writing run's layer keeps there (one spec or a tuple)."""
        specs: dict[int, object] = {}
        for run in self.order:
            if run.cache is None or not run.writes:
                continue
            spec = self.layers[run.layer].cache_spec()
            if spec is None:
                raise ValueError(f"layer {run.layer} was given cache {run.cache} but its mixer keeps nothing")
            if run.cache in specs:
                raise ValueError(f"cache {run.cache} is written by more than one run")
            specs[run.cache] = spec
        for run in self.order:
            if run.cache is not None and not run.writes:
                if run.cache not in specs:
                    raise ValueError(f"layer {run.layer} reads cache {run.cache}, which no run writes")
                if self.layers[run.layer].cache_spec() != specs[run.cache]:
                    raise ValueError(f"layer {run.layer} reads cache {run.cache} of another shape than it expects")
        return specs

    def cache_specs(self) -> dict:
        """cache id -> :class:`CacheSpec`.  A run whose layer keeps several things (a tuple of specs: pages of keys
        and values beside a fixed-size state, say) has one id per thing, ``(run's cache id, index)``."""
        specs: dict = {}
        for cid, spec in self._run_specs().items():
            if isinstance(spec, tuple):
                for k, s in enumerate(spec):
                    specs[(cid, k)] = s
            else:
                specs[cid] = spec
        return specs

    def run_caches(self, views: dict) -> dict:
        """cache id of the execution order -> the view (or tuple of views) its runs are handed, from the per-id views."""
        return {cid: (tuple(views[(cid, k)] for k in range(len(spec))) if isinstance(spec, tuple) else views[cid])
                for cid, spec in self._run_specs().items()}

    # ---- one step ----
    def forward(self, ctx, caches):
        """ctx: the step's tensors; caches: cache id -> view.  Returns 32-bit logits [rows, vocab]."""
        mark = getattr(ctx, "mark", lambda label: None)     # kernel groups for the profile, where the step keeps one

        def embed():
            if getattr(self.embedding, "uses_positions", False):
                return self.embedding.forward(ctx.token_ids, ctx.T, ctx.status, positions=ctx.positions)
            return self.embedding.forward(ctx.token_ids, ctx.T, ctx.status)

        resid = embed()
        # a part that re-enters the embedding's rows later in the step gets them in a buffer of their own (the stream
        # itself is updated in place): the same gather once more, into the region that lives as long as the step
        first_rows = None
        if self.reentry is not None and getattr(self.reentry, "needs_embedding", False):
            with workspace.whole_step():
                first_rows = embed()
        mark("embedding")
        pending = None
        if self._handed is None or self._handed[0] is not caches:
            self._handed = (caches, self.run_caches(caches))
        caches = self._handed[1]
        for i, run in enumerate(self.order):
            cache = caches[run.cache] if run.cache is not None else None
            workspace.begin_run(i)      # the run's buffers come from the scratch region that run i - 2 used
            if run.opens is not None and self.reentry is not None:
                pending = self.reentry.forward(resid, pending, first_rows, run.opens)
            pending = self.layers[run.layer].forward(resid, pending, ctx, cache, run.writes)
        workspace.end_runs()
        if ctx.n_rows == 0:
            return None
        if self.final_norm is None and hasattr(pending, "add"):
            pending.add(resid)      # (a result that its arrangement left to be normed, scaled and added)
            pending = None
        if self.final_norm is None:
            # an architecture without a final norm: the head reads the wanted rows of the stream as they are
            x = resid if pending is None else resid + (pending.sum(0) if pending.dim() == 3 else pending).float()
            y = x[ctx.logit_rows.long()].to(self.build.compute_dtype)
        else:
            y = self.final_norm.forward(resid, pending, rows=ctx.logit_rows)
        logits = self.lm_head.forward(y, ctx.status)
        mark("head")
        return logits
