"""Mefupel: from its typed configuration to a model description.

A decoder whose layers are listed one by one in config.json; a run of them may repeat with the same weights, each pass
with a cache and state of its own, and before every pass the stream receives a learned vector of the pass and (every
pass but the first) the embedding's rows once more.  Every layer norms the stream once (the gain stored less one) and
its mixer and its feed-forward both read that, their results added to the stream together.  Three mixer types:
"attention" -- grouped-query softmax attention under a sliding window, q and k turned in neighbouring pairs, the
values turned by their own position and the heads' sums turned back by the query's; "gla" -- gated linear attention
with a decay per key channel from a low-rank projection, a per-head norm and an output gate; "parallel" -- two
mixers on the same input whose results are normed over the width and averaged: a window attention whose keys double as
values, with q and k normed over the whole projection, turned in halves, and a learned sink per head in the softmax,
beside a retention with one fixed decay per head.  The feed-forward is one hidden layer with a normed polynomial of
degree three as its activation.  Final norm, untied head.

Tensor names: ``embed``, ``head``, ``final.norm``, ``loop.step``; layer i under ``l<i>.``: ``norm1``; attention
``mix.{q,k,v,o}``; gla ``mix.{q,k,v,g,o,norm,a1,a2,a2.b}``; parallel ``mix.left.{q,k,q.norm,k.norm,sink,o}``,
``mix.right.{q,k,v,g,o}``, ``mix.left.out``, ``mix.right.out``; feed-forward ``mlp.{up,down,act}``.
This file only writes data.
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.mefupel import MefupelConfig
from ..registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture


def _window_attention(cfg: MefupelConfig, m, **flags) -> PartSpec:
    return PartSpec("rotary_window_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "v_head_dim": m.vdim,
        "scale": m.scale, "window": m.window, "rope_base": m.rot.base, "rotary_dim": m.rot.dims, "eps": cfg.norm_eps, **flags})


def _attention(cfg: MefupelConfig, m) -> PartSpec:
    return _window_attention(cfg, m, pairing="interleaved", rotate_values=True)


def _gla(cfg: MefupelConfig, m) -> PartSpec:
    return PartSpec("decayed_linear", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                       "tau": m.tau, "rank": m.rank, "eps": cfg.norm_eps})


def _parallel(cfg: MefupelConfig, m) -> PartSpec:
    left = _window_attention(cfg, m.left, pairing="half", values_from_keys=True, whole_norm=True, sink=True)
    r = m.right
    right = PartSpec("retention", {"hidden_size": cfg.width, "num_heads": r.heads, "head_dim": r.dim, "v_head_dim": r.vdim,
                                   "decay": tuple(r.decay), "rope_base": r.rot.base, "rotary_dim": r.rot.dims, "pairing": "half",
                                   "eps": cfg.norm_eps})
    return PartSpec("normed_branches", {"hidden_size": cfg.width, "eps": cfg.norm_eps,
                                        "branches": ((left, "left.", "left.out"), (right, "right.", "right.out"))})


MIXERS = {"attention": _attention, "gla": _gla, "parallel": _parallel}      # layer type -> its mixer's description


def describe_mefupel(cfg: MefupelConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": "", "one_plus": True})
    block = PartSpec("parallel", {})
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type not in MIXERS:
            raise ConfigError(f"layer {i}: no mixer of type '{layer.type}' (known: {sorted(MIXERS)})")
        parts = {"norm1": (norm, "norm1"), "mixer": (MIXERS[layer.type](cfg, layer.mixer), "mix.")}
        if layer.mlp is not None:
            parts["feed_forward"] = (PartSpec("dense", {
                "hidden_size": cfg.width, "intermediate_size": layer.mlp.ff, "activation": "polynorm", "eps": cfg.norm_eps,
                "up_tensor": "up", "down_tensor": "down", "act_tensor": "act"}), "mlp.")
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, parts=parts))
    # every run of a layer, a repeated one too, has a cache and state of its own
    order = tuple(LayerRun(layer=l, cache=n, writes=True, opens=t) for n, (l, t) in enumerate(cfg.runs()))
    reentry = None
    if cfg.has_loop:
        reentry = PartSpec("loop_reentry", {"hidden_size": cfg.width, "passes": cfg.loop_times, "step_tensor": "loop.step",
                                            "add_embedding": True})
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions, embed_tensor="embed",
        layers=tuple(layers), order=order, final_norm=norm, final_norm_prefix="final.norm", lm_head_tensor="head",
        reentry=reentry)


register_architecture("Mefupel", MefupelConfig, describe_mefupel)
