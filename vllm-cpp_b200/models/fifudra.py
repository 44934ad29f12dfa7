"""Fifudra: from its typed configuration to a model description.

A decoder whose layers are listed one by one in config.json; a run of them may repeat with the same weights, each pass
with a cache and state of its own.  Token embedding times a constant; pre-norm layers over ``streams`` residual streams
that every sublayer reads through learned read-out weights and writes back through a learned mixing matrix
("hyper-connections"; one plain stream where the configuration names none); the mixer reads its normed input shifted
towards the previous token's per channel.  Three mixer types: "latent_attention" -- queries through a normed latent,
keys and values expanded from one small normed latent per token plus one rotated key part shared by the heads, rotary
frequencies optionally stretched, causal softmax; "delta" -- the gated delta rule on a matrix state per head behind
short convolutions; "hgrn2" -- linear attention whose forget gate, bounded below, also decides what is written.  Two
feed-forwards: a dense SiLU-gated one, and routed gated experts whose router chooses by corrected sigmoid scores within
the best groups of experts.  Final norm on the sum of the streams; the head is the embedding table itself.

Tensor names: ``embed``, ``final.norm``; layer i under ``l<i>.``: ``norm1``, ``norm2``, ``shift``, ``hc1.{in,out,mix}``,
``hc2.{in,out,mix}``; latent attention ``mix.{dq,dq.norm,uq,dkv,dkv.norm,uk,uv,o}``; delta ``mix.{q,k,v}`` (+ ``.conv``),
``mix.{b,a,A_log,dt_bias,g,norm,o}``; hgrn2 ``mix.{q,f,f.b,lower,v,norm,o}``; dense ``mlp.{gate,up,down}``; experts
``mlp.router``, ``mlp.correction``, ``mlp.e<j>.{gate,up,down}``.  This file only writes data.
"""
from __future__ import annotations

from ..config.base import ConfigError
from ..config.fifudra import FifudraConfig
from ..registry import LayerRun, LayerSpec, ModelSpec, PartSpec, register_architecture


def _latent_attention(cfg: FifudraConfig, m) -> PartSpec:
    rot = m.rot
    scaling = None
    if rot.factor:
        scaling = {"factor": rot.factor, "original": rot.original, "fast": rot.fast, "slow": rot.slow}
    return PartSpec("latent_attention", {
        "hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "rot_dim": m.rot_dim, "v_head_dim": m.vdim,
        "q_rank": m.q_rank, "kv_rank": m.kv_rank, "scale": m.scale, "eps": cfg.norm_eps, "rope_base": rot.base,
        "rope_scaling": scaling})


def _delta(cfg: FifudraConfig, m) -> PartSpec:
    return PartSpec("delta_rule", {"hidden_size": cfg.width, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim,
                                   "v_head_dim": m.vdim, "conv_taps": m.conv, "eps": cfg.norm_eps})


def _hgrn2(cfg: FifudraConfig, m) -> PartSpec:
    return PartSpec("gated_linear", {"hidden_size": cfg.width, "num_heads": m.heads, "head_dim": m.dim, "v_head_dim": m.vdim,
                                     "eps": cfg.norm_eps})


MIXERS = {"latent_attention": _latent_attention, "delta": _delta, "hgrn2": _hgrn2}      # layer type -> its mixer's description


def _feed_forward(cfg: FifudraConfig, mlp) -> PartSpec:
    if mlp.kind == "dense":
        return PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": mlp.ff, "activation": "silu", "bias": False})
    return PartSpec("routed_experts", {"hidden_size": cfg.width, "num_experts": mlp.experts, "top": mlp.top, "expert_size": mlp.ff,
                                       "shared_size": 0, "activation": "silu", "gated": True, "weight_on": "output",
                                       "router": "grouped_sigmoid", "router_groups": mlp.groups, "router_keep": mlp.keep,
                                       "router_scale": mlp.scale, "correction": True})


def describe_fifudra(cfg: FifudraConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": ""})
    block = PartSpec("hyper_streams", {"hidden_size": cfg.width, "streams": cfg.streams or 1, "mixing": cfg.streams > 0,
                                       "token_shift": True})
    layers = []
    for i, layer in enumerate(cfg.layers):
        if layer.type not in MIXERS:
            raise ConfigError(f"layer {i}: no mixer of type '{layer.type}' (known: {sorted(MIXERS)})")
        parts = {"norm1": (norm, "norm1"), "mixer": (MIXERS[layer.type](cfg, layer.mixer), "mix.")}
        if layer.mlp is not None:
            parts.update({"norm2": (norm, "norm2"), "feed_forward": (_feed_forward(cfg, layer.mlp), "mlp.")})
        layers.append(LayerSpec(prefix=f"l{i}.", block=block, parts=parts))
    # every run of a layer, a repeated one too, has a cache and state of its own
    order = tuple(LayerRun(layer=l, cache=n, writes=True) for n, l in enumerate(cfg.run_order()))
    return ModelSpec(
        hidden_size=cfg.width, vocab_size=cfg.vocab, max_positions=cfg.max_positions, embed_tensor="embed",
        layers=tuple(layers), order=order, final_norm=norm, final_norm_prefix="final.norm", lm_head_tensor=None,
        embedding=PartSpec("token_embedding", {"tensor": "embed", "vocab_size": cfg.vocab, "hidden_size": cfg.width,
                                               "row_scale": cfg.embedding_scale}))


register_architecture("Fifudra", FifudraConfig, describe_fifudra)
