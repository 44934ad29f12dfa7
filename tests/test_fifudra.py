"""Fifudra in the engine against the plain implementation (tests/plain_fifudra.py): each mechanism's kernel alone, then
whole models through bin/trace_run (whole prompts, decoding, portions down to two tokens, mixed batches with pages and
slots used again) and greedy generation through the engine's entry point, on small configurations of its own."""
import json
import math

import numpy as np
import pytest
import torch

import plain_fifudra as P
import replay_util as R
from conftest import random_tokens

gpu = pytest.mark.gpu
F64 = torch.float64


def configs():
    from vllm_cpp_b200.config.fifudra import (DeltaSpec as D, FifudraConfig, FifudraLayer as L, FifudraMlp as F, Hgrn2Spec as G,
                                              LatentAttentionSpec as A, RotarySpec as Rot)
    return {
        # no experts anywhere (bfloat16 can be judged row by row): two streams; the middle two layers run twice; fewer
        # rotated lanes than plain ones with stretched frequencies; a delta layer without a feed-forward whose values are
        # wider than its keys; pages of 4
        "A": (FifudraConfig(vocab=150, width=48, norm_eps=1e-5, embedding_scale=3.0, streams=2, loop_start=1, loop_stop=3, loop_times=2,
                            layers=(
            L("latent_attention", A(heads=3, dim=8, rot_dim=4, vdim=6, q_rank=10, kv_rank=12, scale=0.3,
                                    rot=Rot(base=100.0, dims=4, factor=4.0, original=32.0, fast=4.0, slow=1.0)), F("dense", ff=40)),
            L("delta", D(heads=4, kv_heads=2, dim=8, vdim=12, conv=3)),
            L("hgrn2", G(heads=2, dim=6, vdim=10), F("dense", ff=24)),
            L("latent_attention", A(heads=2, dim=4, rot_dim=8, vdim=20, q_rank=7, kv_rank=5, scale=25.0,
                                    rot=Rot(base=10000.0, dims=8)), F("dense", ff=16)))), 4),
        # experts everywhere: four streams, nothing repeated; groups of two of which half are kept, a router without
        # groups and a scale left out, groups of which one is kept; state rows of 64 lanes; a sharp softmax; pages of 16
        "B": (FifudraConfig(vocab=260, width=64, norm_eps=1e-6, streams=4, layers=(
            L("delta", D(heads=2, kv_heads=2, dim=64, vdim=64, conv=4), F("moe", ff=24, experts=8, top=2, scale=2.5, groups=4, keep=2)),
            L("latent_attention", A(heads=4, dim=16, rot_dim=16, vdim=16, q_rank=24, kv_rank=48, scale=12.0,
                                    rot=Rot(base=500.0, dims=16, factor=8.0, original=64.0, fast=8.0, slow=2.0)),
              F("moe", ff=16, experts=6, top=3)),
            L("hgrn2", G(heads=3, dim=16, vdim=8), F("moe", ff=20, experts=4, top=2, scale=0.5, groups=2, keep=1)))), 16),
        # one stream that still has its mixing tensors, a width that is no multiple of 4, the last two layers three times;
        # one head with 33 state rows, groups of one expert, a convolution of one tap (no state of its own), five heads on
        # one head of queries and keys, two rotated lanes; pages of 8
        "C": (FifudraConfig(vocab=97, width=50, norm_eps=1e-4, embedding_scale=0.5, streams=1, loop_start=1, loop_stop=3, loop_times=3,
                            layers=(
            L("hgrn2", G(heads=1, dim=33, vdim=5), F("moe", ff=9, experts=6, top=1, scale=0.5, groups=6, keep=2)),
            L("latent_attention", A(heads=5, dim=6, rot_dim=2, vdim=7, q_rank=5, kv_rank=9, scale=1.0,
                                    rot=Rot(base=50.0, dims=2, factor=1.5, original=16.0, fast=2.0, slow=0.5))),
            L("delta", D(heads=5, kv_heads=1, dim=20, vdim=10, conv=1), F("dense", ff=11)))), 8),
        # no streams at all (the plain residual sum), no repetition, a convolution of two taps, three heads on cached rows of
        # 64 lanes
        "D": (FifudraConfig(vocab=120, width=32, norm_eps=1e-5, embedding_scale=2.0, layers=(
            L("delta", D(heads=2, kv_heads=1, dim=16, vdim=16, conv=2), F("dense", ff=24)),
            L("latent_attention", A(heads=3, dim=8, rot_dim=8, vdim=8, q_rank=12, kv_rank=56, scale=0.35,
                                    rot=Rot(base=10000.0, dims=8)), F("dense", ff=24)),
            L("hgrn2", G(heads=4, dim=8, vdim=8)))), 16),
    }


LENGTHS = {"A": [40, 75, 150, 33, 90, 64, 17, 2], "B": [1, 7, 33, 64, 170, 97, 130, 3], "C": [50, 3, 77, 140, 9, 31],
           "D": [65, 2, 130, 20, 48]}
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}
MIN_MARGIN = 0.02       # no routing decision of the test models is closer than this


HOT = (30.0, 9.0)        # the two large entries of a token's embedding row (times the embedding's scale)


def lane_pair(token, lanes):
    first = token % lanes
    return first, (first + 1 + (token // lanes) % (lanes - 1)) % lanes


def decisive_correction(mlp, lanes, width, g, tries=1500):
    """Corrections, some negative, under which every token's choice of groups and of experts is settled by a wide margin:
    the best of ``tries`` random draws, judged on the router's scores for every pair of hot lanes."""
    E = mlp.experts
    router = {"experts": E, "top": mlp.top, "groups": {"count": mlp.groups, "keep": mlp.keep} if mlp.groups else None}
    unit = math.sqrt(width / (HOT[0] ** 2 + HOT[1] ** 2))          # the norm leaves the hot lanes at these sizes
    rows = []
    for a in range(lanes):
        for b in range(lanes):
            if a != b:
                z = torch.zeros(E, dtype=F64)
                z[a % E] += HOT[0] * unit
                z[b % E] += HOT[1] * unit
                rows.append(z)
    z, eye = torch.stack(rows), torch.eye(E, dtype=F64)
    found = []
    for _ in range(tries):
        c = ((torch.rand(E, generator=g, dtype=F64) - 0.5) * 0.7).to(torch.bfloat16).double()
        gaps = []
        chosen, _ = P.route(z, eye, c, router, gaps)
        found.append((gaps[0], len({tuple(sorted(row)) for row in chosen.tolist()}), c))
    # among the draws under which tokens still differ in whom they choose
    varied = 0.6 * max(n for _, n, _ in found)
    return max((f for f in found if f[1] >= varied), key=lambda f: f[0])[2]


def hand_made(cfg, tensors, seed):
    """Random weights changed by hand where chance would hide a fault.  The decays of the delta rule are spread from
    fast to very slow and the forget gates' lower bounds reach close to one, so a lost state or a token far back
    shows.  The routers are made decisive: random ones have close calls every hundred tokens or so, which 16-bit
    activations decide differently from the 64-bit plain implementation.  Each token's embedding gets a large entry in
    one of the first lanes and a smaller one in another (by its id), the routers read those lanes, and the corrections
    are spread widely, some negative, so that groups and corrections both change who is chosen."""
    g = torch.Generator().manual_seed(seed)
    lanes = max([l.mlp.experts for l in cfg.layers if l.mlp is not None and l.mlp.kind == "moe"] + [0])
    if lanes:
        emb = tensors["embed"].float()
        emb[:, :lanes] = 0
        for t in range(cfg.vocab):
            first, second = lane_pair(t, lanes)
            emb[t, first] = HOT[0] / cfg.embedding_scale
            emb[t, second] = HOT[1] / cfg.embedding_scale
        tensors["embed"] = emb.to(torch.bfloat16)
        # (the head is the embedding table: the last norm passes nothing of those lanes, or they would drown the logits)
        tensors["final.norm"] = torch.cat([torch.zeros(lanes), tensors["final.norm"].float()[lanes:]]).to(torch.bfloat16)
    for k in list(tensors):
        if k.endswith("mix.A_log"):
            tensors[k] = torch.linspace(-6.0, 0.5, tensors[k].numel()).to(torch.bfloat16)
        elif k.endswith("mix.lower"):
            tensors[k] = torch.linspace(0.0, 0.995, tensors[k].numel()).to(torch.bfloat16)
        elif k.endswith("mlp.router"):
            E, W = tensors[k].shape
            r = torch.zeros(E, W)
            for lane in range(lanes):
                r[lane % E, lane] = 1.0
            tensors[k] = r.to(torch.bfloat16)
        elif k.endswith("mlp.correction"):
            layer = cfg.layers[int(k.split(".")[0][1:])]
            tensors[k] = decisive_correction(layer.mlp, lanes, cfg.width, g).to(torch.bfloat16)
    return tensors


@pytest.fixture(scope="module")
def fifudra_dirs(tmp_path_factory):
    from vllm_cpp_b200 import write_random_model
    from vllm_cpp_b200.weights.safetensors_io import read_safetensors, write_safetensors
    out = {}
    for i, (name, (cfg, _)) in enumerate(configs().items()):
        d = tmp_path_factory.mktemp(f"fifudra_{name}")
        write_random_model(cfg, 31 + i, d, dtype="bfloat16")
        tensors = {k: v.clone() for k, v in read_safetensors(d / "model.safetensors").items()}
        write_safetensors(d / "model.safetensors", hand_made(cfg, tensors, 7 + i), {"format": "pt"})
        out[name] = d
    return out


class Oracle:
    def __init__(self, dirs):
        self.models = {n: P.read_model(d) for n, d in dirs.items()}
        self.cache = {}
        self.margins = []

    def __call__(self, name, tokens):
        key = (name, tuple(tokens))
        if key not in self.cache:
            self.cache[key] = P.forward(*self.models[name], list(tokens), margins=self.margins).numpy()
        return self.cache[key]


@pytest.fixture(scope="module")
def oracle(fifudra_dirs):
    return Oracle(fifudra_dirs)


def requests_of(name):
    vocab = configs()[name][0].vocab
    return {f"r{i}": random_tokens(vocab, n, 7 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


# -------------------------------------------------------------------------- without a GPU


def test_config_reads_every_size_and_constant():
    from vllm_cpp_b200 import ConfigError
    from vllm_cpp_b200.config.fifudra import FifudraConfig
    rot = {"base": 777.0, "dims": 6, "scaling": {"factor": 3.0, "original": 100, "fast": 16.0, "slow": 2.0}}
    d = {"architecture": "Fifudra", "vocab": 50, "width": 24, "norm": {"eps": 3e-4}, "embedding": {"scale": 2.5}, "streams": 5,
         "loop": {"start": 1, "stop": 3, "times": 4},
         "layers": [{"type": "latent_attention", "mlp": None,
                     "mixer": {"heads": 6, "dim": 10, "rot_dim": 6, "vdim": 14, "q_rank": 9, "kv_rank": 11, "scale": 0.5, "rot": rot}},
                    {"type": "delta", "mlp": {"kind": "dense", "ff": 31},
                     "mixer": {"heads": 4, "kv_heads": 2, "dim": 6, "vdim": 9, "conv": 3}},
                    {"type": "hgrn2", "mixer": {"heads": 3, "dim": 8, "vdim": 5},
                     "mlp": {"kind": "moe", "router": {"experts": 9, "top": 2, "scale": 1.75, "groups": {"count": 3, "keep": 2}},
                             "expert": {"ff": 5}}},
                    {"type": "hgrn2", "mixer": {"heads": 1, "dim": 8, "vdim": 8},
                     "mlp": {"kind": "moe", "router": {"experts": 2, "top": 1, "groups": None}, "expert": {"ff": 3}}}]}
    cfg = FifudraConfig.from_dict(d)
    assert (cfg.vocab, cfg.width, cfg.norm_eps, cfg.embedding_scale, cfg.streams) == (50, 24, 3e-4, 2.5, 5)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (1, 3, 4)
    assert cfg.run_order() == (0, 1, 2, 1, 2, 1, 2, 1, 2, 3)
    a, b, c, e = cfg.layers
    m = a.mixer
    assert (m.heads, m.dim, m.rot_dim, m.vdim, m.q_rank, m.kv_rank, m.scale, a.mlp) == (6, 10, 6, 14, 9, 11, 0.5, None)
    assert (m.rot.base, m.rot.dims, m.rot.factor, m.rot.original, m.rot.fast, m.rot.slow) == (777.0, 6, 3.0, 100.0, 16.0, 2.0)
    assert (b.mixer.heads, b.mixer.kv_heads, b.mixer.dim, b.mixer.vdim, b.mixer.conv, b.mlp.kind, b.mlp.ff) == (4, 2, 6, 9, 3, "dense", 31)
    assert (c.mixer.heads, c.mixer.dim, c.mixer.vdim) == (3, 8, 5)
    assert (c.mlp.kind, c.mlp.experts, c.mlp.top, c.mlp.scale, c.mlp.groups, c.mlp.keep, c.mlp.ff) == ("moe", 9, 2, 1.75, 3, 2, 5)
    assert (e.mlp.scale, e.mlp.groups, e.mlp.keep) == (1.0, 0, 0)
    assert FifudraConfig.from_dict(cfg.to_dict()) == cfg
    # what is left out is off: one stream, no repetition, a scale of one, plain frequencies
    bare = FifudraConfig.from_dict({k: v for k, v in d.items() if k not in ("streams", "loop", "embedding")})
    assert (bare.streams, bare.embedding_scale, bare.run_order()) == (0, 1.0, (0, 1, 2, 3))
    assert FifudraConfig.from_dict(dict(d, streams=None, loop=None)).run_order() == (0, 1, 2, 3)
    plain = dict(d["layers"][0], mixer=dict(d["layers"][0]["mixer"], rot={"base": 10.0, "dims": 6, "scaling": None}))
    assert FifudraConfig.from_dict(dict(d, layers=[plain], loop=None)).layers[0].mixer.rot.factor == 0.0
    layer = d["layers"]
    for bad in ({"layers": []}, {"layers": [dict(layer[0], type="other")]}, {"loop": {"start": 2, "stop": 5, "times": 2}},
                {"layers": [dict(layer[1], mixer=dict(layer[1]["mixer"], kv_heads=3))], "loop": None},
                {"layers": [dict(layer[0], mixer=dict(layer[0]["mixer"], rot=dict(rot, dims=4)))], "loop": None},
                {"layers": [dict(layer[2], mlp=dict(layer[2]["mlp"], router={"experts": 2, "top": 3}))], "loop": None},
                {"layers": [dict(layer[2], mlp=dict(layer[2]["mlp"], router={"experts": 9, "top": 4, "groups": {"count": 3, "keep": 1}}))], "loop": None},
                {"layers": [dict(layer[2], mlp=dict(layer[2]["mlp"], router={"experts": 9, "top": 2, "groups": {"count": 2, "keep": 1}}))], "loop": None},
                {"layers": [dict(layer[1], mlp={"kind": "routed", "ff": 3})], "loop": None}, {"vocab": None}):
        with pytest.raises(ConfigError):
            FifudraConfig.from_dict(dict(d, **bad))


def test_model_folder_is_recognised_and_names_its_tensors(tmp_path):
    from vllm_cpp_b200.models import expected_tensors, load_config
    cfg, _ = configs()["A"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(tmp_path) == cfg
    s = {t.name: tuple(t.shape) for t in expected_tensors(cfg)}
    assert s["embed"] == (150, 48) and s["final.norm"] == (48,) and "head" not in s
    assert s["l0.mix.dq"] == (10, 48) and s["l0.mix.dq.norm"] == (10,) and s["l0.mix.uq"] == (3 * (8 + 4), 10)
    assert s["l0.mix.dkv"] == (12 + 4, 48) and s["l0.mix.dkv.norm"] == (12,) and s["l0.mix.uk"] == (24, 12)
    assert s["l0.mix.uv"] == (18, 12) and s["l0.mix.o"] == (48, 18)
    assert s["l0.shift"] == (48,) and s["l0.hc1.in"] == s["l0.hc2.out"] == (2,) and s["l0.hc1.mix"] == s["l0.hc2.mix"] == (2, 2)
    assert s["l1.mix.q"] == s["l1.mix.k"] == (16, 48) and s["l1.mix.v"] == s["l1.mix.g"] == (48, 48)
    assert s["l1.mix.q.conv"] == (16, 3) and s["l1.mix.v.conv"] == (48, 3) and s["l1.mix.b"] == s["l1.mix.a"] == (4, 48)
    assert s["l1.mix.A_log"] == s["l1.mix.dt_bias"] == (4,) and s["l1.mix.norm"] == (12,) and s["l1.mix.o"] == (48, 48)
    assert not any(k.startswith(("l1.mlp", "l1.norm2", "l1.hc2")) for k in s)      # a layer without a feed-forward
    assert s["l2.mix.q"] == s["l2.mix.f"] == (12, 48) and s["l2.mix.f.b"] == s["l2.mix.lower"] == (12,)
    assert s["l2.mix.v"] == (20, 48) and s["l2.mix.norm"] == (10,) and s["l2.mix.o"] == (48, 20)
    assert s["l2.mlp.gate"] == s["l2.mlp.up"] == (24, 48) and s["l2.mlp.down"] == (48, 24)
    b, _ = configs()["B"]
    s = {t.name: tuple(t.shape) for t in expected_tensors(b)}
    assert s["l0.mlp.router"] == (8, 64) and s["l0.mlp.correction"] == (8,) and s["l0.mlp.e7.gate"] == s["l0.mlp.e7.up"] == (24, 64)
    assert s["l0.mlp.e7.down"] == (64, 24) and "l0.mlp.e8.up" not in s and s["l0.hc1.mix"] == (4, 4)
    d, _ = configs()["D"]
    assert not any(".hc" in t.name for t in expected_tensors(d))                   # one plain stream has no mixing tensors
    c, _ = configs()["C"]
    assert {t.name: tuple(t.shape) for t in expected_tensors(c)}["l0.hc1.mix"] == (1, 1)


def test_what_a_layer_run_keeps_per_request():
    """Every run of a layer, a repeated one too, has a state of its own: the mixer input's last row, then the mixer's."""
    import vllm_cpp_b200.models as models
    cfg, _ = configs()["A"]
    specs = models.build_model(cfg, torch.float32, "cpu").cache_specs()
    assert sorted({k[0] for k in specs}) == [0, 1, 2, 3, 4, 5]           # layers 0, 1, 2, 1, 2, 3
    for run in range(6):
        assert (specs[(run, 0)].kind, specs[(run, 0)].shape, specs[(run, 0)].dtype) == ("state", (48,), "float32")
    kv = specs[(0, 1)]
    assert (kv.kind, kv.num_kv_heads, kv.head_dim, kv.v_head_dim) == ("kv", 1, 12 + 4, 12)       # the latent and the rotated key part
    for run in (1, 3):
        assert (specs[(run, 1)].shape, specs[(run, 1)].dtype) == ((4, 12, 8), "float32")          # heads, value columns, rows
        assert specs[(run, 2)].shape == (2, 2 * 16 + 48)                                       # the convolution's last inputs
    for run in (2, 4):
        assert specs[(run, 1)].shape == (2, 10, 6)
    assert (specs[(5, 1)].head_dim, specs[(5, 1)].v_head_dim) == (5 + 8, 5)
    c, _ = configs()["C"]
    specs = models.build_model(c, torch.float32, "cpu").cache_specs()
    assert specs[(2, 1)].shape == (5, 10, 20) and (2, 2) not in specs       # one tap: the convolution keeps nothing
    # cached rows of 64 lanes in bfloat16: value rows as wide as key rows, for the attention kernels on the tensor cores
    b, _ = configs()["B"]
    kv32 = models.build_model(b, torch.float32, "cpu").cache_specs()[(1, 1)]
    kv16 = models.build_model(b, torch.bfloat16, "cpu").cache_specs()[(1, 1)]
    assert (kv32.head_dim, kv32.v_head_dim) == (64, 48) and (kv16.head_dim, kv16.v_head_dim) == (64, 0)


def test_stretched_frequencies_agree_with_the_plain_ones():
    from vllm_cpp_b200.parts.latent_attention import rope_frequencies
    for dims, base, sc in ((4, 100.0, {"factor": 4.0, "original": 32.0, "fast": 4.0, "slow": 1.0}), (16, 500.0, None),
                           (64, 1e6, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0}),
                           (2, 50.0, {"factor": 1.5, "original": 16.0, "fast": 2.0, "slow": 0.5})):
        f, gain = rope_frequencies(dims, base, sc)
        pf, pgain = P.yarn_frequencies({"dims": dims, "base": base, "scaling": sc})
        assert torch.allclose(torch.tensor(f, dtype=F64), pf, rtol=1e-14, atol=0) and abs(gain - pgain) < 1e-15
    # by hand: 64 lanes, base 1e6: a pair that turns often keeps its frequency, one that turns less than once is slowed
    f, gain = rope_frequencies(64, 1e6, {"factor": 40.0, "original": 4096, "fast": 32.0, "slow": 1.0})
    assert f[0] == 1.0 and abs(f[31] - 1e6 ** (-62 / 64) / 40.0) < 1e-18 and abs(gain - (0.1 * math.log(40.0) + 1)) < 1e-15
    assert all(a > b for a, b in zip(f, f[1:]))


def test_oracle_mechanisms_by_hand():
    t = lambda *x: torch.tensor(x, dtype=F64)
    # token shift: the first row moves towards zero, the others towards the row before, as it was
    h = t([2.0, 4.0], [6.0, 8.0], [1.0, 1.0])
    assert torch.equal(P.token_shift(h, t(0.5, 0.0)), t([1.0, 4.0], [4.0, 8.0], [3.5, 1.0]))
    assert torch.equal(P.token_shift(h[1:], t(0.5, 0.0), before=h[0]), t([4.0, 8.0], [3.5, 1.0]))
    # streams: read-out, and a write-back in which every new stream is made from the old ones ([from, to])
    x = torch.stack([t([1.0], [2.0]), t([10.0], [20.0])])
    assert torch.equal(P.hyper_read(x, t(2.0, 0.5)), t([7.0], [14.0]))
    new = P.hyper_write(x, t([100.0], [200.0]), t([1.0, 3.0], [0.0, 1.0]), t(1.0, -1.0))
    assert torch.equal(new[0], t([101.0], [202.0])) and torch.equal(new[1], t([3.0 + 10 - 100], [6.0 + 20 - 200]))
    # rotation of one pair, lane i with lane i + dims / 2, the rest unchanged
    out = P.rotate(t([1.0, 5.0, 0.0, 7.0, 9.0])[None], torch.tensor([3]), t(0.5, 0.0), 2.0)
    assert torch.allclose(out, t([2 * math.cos(1.5), 10.0, 2 * math.sin(1.5), 14.0, 9.0])[None])
    # the router: a correction changes who is chosen, not the weight; a group outside the kept ones loses even to a
    # negative choice score; a group's score is the sum of its two largest
    router = {"experts": 4, "top": 2, "scale": 3.0, "groups": {"count": 2, "keep": 1}}
    eye = torch.eye(4, dtype=F64)
    z = t([0.0, 0.2, 3.0, 1.0])
    chosen, w = P.route(z, eye, t(0.0, 0.0, 0.0, 0.0), router)
    assert chosen.tolist() == [[2, 3]] and torch.allclose(w, 3 * torch.sigmoid(t([3.0, 1.0])))
    chosen, w = P.route(z, eye, t(0.0, 0.0, -2.0, 0.0), router)
    assert chosen.tolist() == [[1, 0]] and torch.allclose(w, 3 * torch.sigmoid(t([0.2, 0.0])))
    chosen, _ = P.route(z, eye, t(-1.0, -1.0, -2.0, -2.0), router)            # all choice scores negative
    assert chosen.tolist() == [[1, 0]]
    chosen, _ = P.route(t([0.0, 4.0, 3.0, 3.5]), eye, t(0.0, 0.0, 0.0, 0.0), router)   # the largest score sits in the lesser group
    assert chosen.tolist() == [[3, 2]]
    chosen, _ = P.route(z, eye, t(0.0, 0.0, 0.0, 0.0), dict(router, groups=None, top=3))
    assert chosen.tolist() == [[2, 3, 1]]
    # the delta rule, one head of one state row and one value lane: k = 1 after the unit norm, q = d^(-1/2) = 1
    m = {"heads": 1, "kv_heads": 1, "dim": 1, "vdim": 1}
    one, big = t(1.0), 50.0
    w = {"q": t([big, 0.0]), "k": t([big, 0.0]), "v": t([0.0, 1.0]), "q.conv": one[None], "k.conv": one[None], "v.conv": one[None],
         "b": t([0.0, 0.0]), "a": t([0.0, 0.0]), "A_log": t(0.0), "dt_bias": t(0.0), "norm": one, "g": t([big, 0.0]), "o": one[None]}
    for k in ("q", "k", "v", "b", "a", "g"):
        w[k] = w[k].reshape(1, 2)
    w["A_log"], w["dt_bias"] = w["A_log"].reshape(1), w["dt_bias"].reshape(1)
    x = t([1.0, 2.0], [1.0, -3.0])
    g, v0, v1 = math.exp(-math.log(2.0)), P.silu(t(2.0)).item(), P.silu(t(-3.0)).item()
    s0 = 0.5 * v0
    s1 = g * s0 + 0.5 * (v1 - g * s0)
    # (the head's norm divides the one lane by its own size: what is left is the sign, times the gate)
    got = P.delta_rule(x, w, m, 0.0)
    assert torch.allclose(got[:, 0], t(math.copysign(1, s0) * big, math.copysign(1, s1) * big), rtol=1e-6)
    # the gated linear form: f keeps, 1 - f writes
    m = {"heads": 1, "dim": 1, "vdim": 2}
    w = {"q": t([big, 0.0]), "f": t([0.0, 0.0]), "f.b": t(0.0), "lower": t(0.5), "v": t([0.0, 1.0], [0.0, 2.0]), "norm": t(1.0, 1.0),
         "o": torch.eye(2, dtype=F64)}
    for k in ("q", "f"):
        w[k] = w[k].reshape(1, 2)
    got = P.hgrn2(t([1.0, 4.0], [1.0, 8.0]), w, m, 0.0)
    # f = 0.75: S_0 = 0.25 v_0, S_1 = 0.75 S_0 + 0.25 v_1; the norm over the two lanes keeps their ratio 1 : 2
    assert torch.allclose(got, t([1.0, 2.0], [1.0, 2.0]) / math.sqrt(2.5), rtol=1e-9)


def test_the_test_models_route_decisively(fifudra_dirs, oracle):
    """The hand-made routers of the test models: no token's choice of experts or of groups is a close call."""
    for name in ("B", "C"):
        for toks in list(requests_of(name).values())[:4]:
            oracle(name, toks)
    assert oracle.margins and min(oracle.margins) > MIN_MARGIN, min(oracle.margins)


# -------------------------------------------------------------------------- each kernel alone


def dev():
    return torch.device("cuda:0")


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=dev())


def f32(x):
    return None if x is None else x.float().contiguous().to(dev())


def entries_of(lengths):
    """(q_start, q_len) device arrays of a step whose entries have these token counts, rows in entry order."""
    starts = np.concatenate([[0], np.cumsum(lengths)])[:-1]
    return i32(starts.tolist()), i32(list(lengths))


def partial_sums(x, S, g):
    """x [T, C] (64-bit) as S 32-bit partial sums that add up to it (to 32-bit rounding)."""
    if S == 1:
        return x.float().to(dev())
    parts = torch.randn(S - 1, *x.shape, generator=g, dtype=F64)
    return torch.cat([parts, (x - parts.sum(0))[None]]).float().to(dev())


TOL32 = dict(atol=3e-5, rtol=3e-5)
TOL16 = dict(atol=3e-2, rtol=2e-2)


@gpu
@pytest.mark.parametrize("S,W,Sy,out_dtype", [(1, 6, 1, torch.float32), (2, 50, 2, torch.bfloat16), (3, 320, 3, torch.float32),
                                              (4, 64, 1, torch.bfloat16), (8, 2500, 2, torch.float32)])
def test_streams_write_back_read_out_and_norm(S, W, Sy, out_dtype):
    """The first sublayer of a step (every stream starts as the same row), a write-back with the next read-out, a
    write-back alone, the plain residual sum when no mixing is given, and the read-out of a few rows that leaves the
    streams alone."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(S * 1000 + W)
    T, eps = 7, 1e-5
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F64)
    x0, y = rnd(T, W), rnd(T, W) * 2
    mix, outw, inw, gain = torch.eye(S, dtype=F64) + 0.3 * rnd(S, S), 1 + 0.3 * rnd(S), 1 + 0.3 * rnd(S), 1 + 0.1 * rnd(W)
    tol = TOL32 if out_dtype == torch.float32 else TOL16
    # the step's first read-out
    streams = torch.full((S, T, W), float("nan"), device=dev())
    out = torch.empty(T, W, device=dev(), dtype=out_dtype)
    ops.hyper_mix_norm(streams, init=f32(x0), inw=f32(inw), gain=f32(gain), eps=eps, out=out)
    old = x0[None].repeat(S, 1, 1)
    torch.testing.assert_close(streams.double().cpu(), old, atol=1e-6, rtol=1e-6)
    torch.testing.assert_close(out.double().cpu(), P.rms_norm(P.hyper_read(old, inw), gain, eps), **tol)
    # a write-back of partial sums and the read-out for the next sublayer; the streams start unequal
    old = rnd(S, T, W)
    streams = f32(old)
    ops.hyper_mix_norm(streams, y=partial_sums(y, Sy, g), mix=f32(mix), outw=f32(outw), inw=f32(inw), gain=f32(gain), eps=eps, out=out)
    new = P.hyper_write(old, y, mix, outw)
    torch.testing.assert_close(streams.double().cpu(), new, **TOL32)
    torch.testing.assert_close(out.double().cpu(), P.rms_norm(P.hyper_read(new, inw), gain, eps), **tol)
    # the write-back alone
    streams = f32(old)
    ops.hyper_mix_norm(streams, y=partial_sums(y, Sy, g), mix=f32(mix), outw=f32(outw))
    torch.testing.assert_close(streams.double().cpu(), new, **TOL32)
    # some rows only, summed plainly: the streams stay as they were
    streams = f32(old)
    rows = [5, 0, 3]
    few = torch.empty(3, W, device=dev(), dtype=out_dtype)
    ops.hyper_mix_norm(streams, y=partial_sums(y, Sy, g), mix=f32(mix), outw=f32(outw), gain=f32(gain), eps=eps, out=few, rows=i32(rows))
    assert torch.equal(streams.cpu(), old.float())
    torch.testing.assert_close(few.double().cpu(), P.rms_norm(new.sum(0), gain, eps)[rows], **tol)
    if S == 1:
        # no mixing tensors: x <- x + y, then the norm of x
        streams = f32(old)
        ops.hyper_mix_norm(streams, y=partial_sums(y, Sy, g), gain=f32(gain), eps=eps, out=out)
        torch.testing.assert_close(streams.double().cpu(), old + y[None], **TOL32)
        torch.testing.assert_close(out.double().cpu(), P.rms_norm(old[0] + y, gain, eps), **tol)


@gpu
@pytest.mark.parametrize("W,dtype", [(5, torch.float32), (48, torch.bfloat16), (700, torch.float32)])
def test_token_shift_in_portions_equals_the_whole(W, dtype):
    """Two requests in slots 2 and 0 cut into portions of many sizes, a slot given to a new request in between: the row
    before a portion's first comes from the slot, zeros before a request's first token."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(W)
    steps = [(3, 1), (1, 1), (2, 7), (1, 2), (9, 1), (1, 0), (2, 2)]
    total = [sum(s[0] for s in steps), sum(s[1] for s in steps)]
    seqs = [torch.randn(n, W, generator=g, dtype=F64) for n in total]
    mu = torch.rand(W, generator=g, dtype=F64)
    state = torch.zeros(3, W, device=dev())
    state[1] = float("nan")
    tol = TOL32 if dtype == torch.float32 else TOL16
    got, at = [[], []], [0, 0]
    for n0, n1 in steps:
        lens = [n0, n1]
        rows = torch.cat([seqs[r][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, W), float("nan"), dtype=F64)])
        qs, ql = entries_of(lens)
        out = torch.full(rows.shape, 5.0, device=dev(), dtype=dtype)
        ops.token_shift(f32(rows), f32(mu), state, qs, ql, i32([2, 0]), 2, out)
        o = out.double().cpu()
        assert bool((o[n0 + n1:] == 5.0).all())
        got[0].append(o[:n0]); got[1].append(o[n0:n0 + n1])
        at = [at[0] + n0, at[1] + n1]
    for r in range(2):
        torch.testing.assert_close(torch.cat(got[r]), P.token_shift(seqs[r], mu), **tol)
    torch.testing.assert_close(state[2].double().cpu(), seqs[0][-1], atol=1e-6, rtol=1e-6)
    assert bool(torch.isnan(state[1]).all())


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("wide", [False, True])
@pytest.mark.parametrize("q_rank,kv_rank,rot,S,scaling", [(10, 12, 4, 1, True), (5, 9, 2, 2, True), (80, 64, 32, 3, False), (7, 5, 0, 1, False),
                                                          (200, 190, 64, 2, True)])
def test_latent_norms_rotation_and_store(dtype, q_rank, kv_rank, rot, S, scaling, wide):
    """From the stacked down projections: both latents normed with their gains, the shared key part rotated by each
    token's position with the stretched frequencies (far positions too), the cache row [c | k_rot] and the value row c
    in the token's slot (``wide``: value rows as wide as key rows, zeros behind c); rows without a slot store nothing."""
    from vllm_cpp_b200 import ops
    from vllm_cpp_b200.parts.latent_attention import rope_frequencies
    g = torch.Generator().manual_seed(q_rank + rot)
    T, ps, num_pages, eps = 7, 4, 5, 1e-4
    u = torch.randn(T, q_rank + kv_rank + rot, generator=g, dtype=F64) * 3
    gq, gkv = 1 + 0.2 * torch.randn(q_rank, generator=g, dtype=F64), 1 + 0.2 * torch.randn(kv_rank, generator=g, dtype=F64)
    sc = {"factor": 4.0, "original": 64.0, "fast": 8.0, "slow": 1.0} if scaling else None
    positions = [0, 1, 2, 3000, 77, 5, 100000]
    slot_map = [9, 10, 11, 0, 17, -1, 3]
    fr, gain = rope_frequencies(rot, 1000.0, sc) if rot else ([0.0], 1.0)
    freq = torch.tensor(fr, dtype=F64).float().to(dev())
    vw = kv_rank + rot if wide else kv_rank
    pages = torch.full((num_pages, ps * (kv_rank + rot + vw)), float("nan"), device=dev(), dtype=dtype)
    cq = torch.empty(T, q_rank, device=dev(), dtype=dtype)
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.latent_norm_rope_store(partial_sums(u, S, g), f32(gq), f32(gkv), eps, i32(positions), freq, gain, i32(slot_map), cq, pages, ps,
                               q_rank, kv_rank, rot, status, v_width=vw)
    assert status.item() == 0
    tol = TOL32 if dtype == torch.float32 else TOL16
    torch.testing.assert_close(cq.double().cpu(), P.rms_norm(u[:, :q_rank], gq, eps), **tol)
    c = P.rms_norm(u[:, q_rank:q_rank + kv_rank], gkv, eps)
    k_rot = u[:, q_rank + kv_rank:]
    if rot:
        # the kernel's angle is a 32-bit product: the plain rotation gets the same angle
        pfreq, pgain = P.yarn_frequencies({"dims": rot, "base": 1000.0, "scaling": sc})
        ang = (torch.tensor(positions, dtype=torch.float32)[:, None] * pfreq.float()[None]).double()
        half = rot // 2
        a, b = k_rot[:, :half], k_rot[:, half:]
        k_rot = torch.cat([a * torch.cos(ang) - b * torch.sin(ang), b * torch.cos(ang) + a * torch.sin(ang)], 1) * pgain
    host = pages.double().cpu()
    khd = kv_rank + rot
    for t, slot in enumerate(slot_map):
        if slot < 0:
            continue
        page, off = slot // ps, slot % ps
        torch.testing.assert_close(host[page, off * khd:off * khd + kv_rank], c[t], **tol)
        torch.testing.assert_close(host[page, off * khd + kv_rank:(off + 1) * khd], k_rot[t], **tol)
        torch.testing.assert_close(host[page, ps * khd + off * vw:ps * khd + off * vw + kv_rank], c[t], **tol)
        assert bool((host[page, ps * khd + off * vw + kv_rank:ps * khd + (off + 1) * vw] == 0).all())
    assert (~torch.isnan(host)).sum().item() == 6 * (kv_rank + rot + vw)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,H,n_in,n_out,S", [(1, 3, 8, 12, 1), (9, 5, 6, 9, 2), (20, 2, 96, 80, 1), (17, 6, 33, 130, 3),
                                          (70, 3, 96, 80, 1), (130, 2, 12, 150, 2), (64, 2, 128, 96, 1), (97, 2, 30, 20, 1)])       # (long steps: a tile of tokens a block)
def test_a_small_matrix_per_head_and_the_rotation_of_a_slice(dtype, T, H, n_in, n_out, S):
    """Every head's lanes, found at a stride and an offset, meet the head's own matrix; beside them a slice of every head
    is rotated into place."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(T + n_in)
    rot = 6
    stride_in, off_in, stride_out, off_out = n_in + rot, 0, n_out + rot + 3, 2
    x = torch.randn(T, H * stride_in, generator=g, dtype=F64)
    m = (torch.randn(H, n_out, n_in, generator=g, dtype=F64) / n_in ** 0.5).to(dtype).double()
    out = torch.full((T, H * stride_out), 9.0, device=dev(), dtype=dtype)
    ops.head_linear(partial_sums(x, S, g), m.to(dtype).to(dev()), out, heads=H, n_in=n_in, n_out=n_out, in_head_stride=stride_in,
                    in_off=off_in, out_head_stride=stride_out, out_off=off_out)
    freq = torch.tensor([1.0, 0.1, 0.003], dtype=F64)
    positions = torch.arange(T) * 37
    ops.rope_rows(partial_sums(x, S, g), i32(positions.tolist()), f32(freq), 1.25, out, heads=H, dims=rot, width=rot,
                  in_head_stride=stride_in, in_off=n_in, out_head_stride=stride_out, out_off=off_out + n_out)
    got = out.double().cpu().view(T, H, stride_out)
    xs = x.view(T, H, stride_in)
    tol = TOL32 if dtype == torch.float32 else TOL16
    torch.testing.assert_close(got[..., off_out:off_out + n_out], torch.einsum("hjc,thc->thj", m, xs[..., :n_in]), **tol)
    ang = (positions.float()[:, None] * freq.float()[None]).double()[:, None, :]
    a, b = xs[..., n_in:n_in + 3], xs[..., n_in + 3:]
    want = torch.cat([a * torch.cos(ang) - b * torch.sin(ang), b * torch.cos(ang) + a * torch.sin(ang)], -1) * 1.25
    torch.testing.assert_close(got[..., off_out + n_out:off_out + n_out + rot], want, **tol)
    assert bool((got[..., :off_out] == 9.0).all()) and bool((got[..., off_out + n_out + rot:] == 9.0).all())
    if dtype == torch.bfloat16:
        # the input may also be one buffer of the compute dtype
        xb = x.to(dtype)
        ops.head_linear(xb.to(dev()), m.to(dtype).to(dev()), out, heads=H, n_in=n_in, n_out=n_out, in_head_stride=stride_in,
                        out_head_stride=stride_out, out_off=off_out)
        got = out.double().cpu().view(T, H, stride_out)
        torch.testing.assert_close(got[..., off_out:off_out + n_out],
                                   torch.einsum("hjc,thc->thj", m, xb.double().view(T, H, stride_in)[..., :n_in]), **tol)


PORTION_STEPS = [(3, 1), (1, 1), (2, 7), (1, 2), (9, 1), (1, 0), (2, 2), (1, 1), (1, 1), (1, 1), (16, 1), (1, 17)]
DECODE_STEPS = [(4, 2)] + [(1, 1)] * 45
# portions of several staged batches each (the kernels stage 8 or 16 tokens at a time), ending on, before and behind a batch's edge
LONG_STEPS = [(37, 16), (1, 33), (48, 5), (17, 32), (8, 9), (70, 1)]


def run_in_steps(W, steps, S, one_step, seed):
    """Two requests (in slots 2 and 0 of three) cut as ``steps`` says, two rows of padding behind every step;
    ``one_step(u_rows, qs, ql, slots)`` -> that step's result rows.  Returns the requests' inputs and results."""
    g = torch.Generator().manual_seed(seed)
    total = [sum(s[0] for s in steps), sum(s[1] for s in steps)]
    seqs = [torch.randn(n, W, generator=g, dtype=F64) for n in total]
    got, at = [[], []], [0, 0]
    for n0, n1 in steps:
        lens = [n0, n1]
        rows = torch.cat([seqs[r][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, W), float("nan"), dtype=F64)])
        qs, ql = entries_of(lens)
        o = one_step(rows, qs, ql, i32([2, 0]), lens, g).double().cpu()
        got[0].append(o[:n0]); got[1].append(o[n0:n0 + n1])
        at = [at[0] + n0, at[1] + n1]
    return seqs, [torch.cat(x) for x in got]


def check_delta(H, G, d, dv, taps, S, steps, dtype=torch.float32):
    from vllm_cpp_b200 import ops
    W, eps = 24, 1e-5
    g = torch.Generator().manual_seed(H * 100 + d)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F64)
    qk, inner = G * d, H * dv
    cc = 2 * qk + inner
    w = {"q": rnd(qk, W), "k": rnd(qk, W), "v": rnd(inner, W), "g": rnd(inner, W) * 0.5, "b": rnd(H, W) * 0.5, "a": rnd(H, W) * 0.5,
         "q.conv": rnd(qk, taps), "k.conv": rnd(qk, taps), "v.conv": rnd(inner, taps),
         "A_log": torch.linspace(-6.0, 0.5, H, dtype=F64), "dt_bias": rnd(H), "norm": 1 + 0.2 * rnd(dv), "o": torch.eye(inner, dtype=F64)}
    w_in = torch.cat([w[n] for n in ("q", "k", "v", "g", "b", "a")])
    conv_w = f32(torch.cat([w["q.conv"], w["k.conv"], w["v.conv"]]))
    state = torch.zeros(3, H, dv, d, device=dev())
    state[1] = float("nan")
    conv_state = torch.zeros(3, taps - 1, cc, device=dev()) if taps > 1 else None
    rate, dt_bias, gain = f32(torch.exp(w["A_log"])), f32(w["dt_bias"]), f32(w["norm"])

    def one_step(rows, qs, ql, slots, lens, gen):
        T = rows.shape[0]
        u = partial_sums(rows @ w_in.T, S, gen)
        conv_in = u[..., :cc]
        xc = torch.full((T, cc), float("nan"), device=dev())
        ops.causal_conv(conv_in, conv_w, conv_state, qs, ql, slots, 2, out_conv=xc, act="silu")
        if taps > 1 and any(n > 1 for n in lens):
            ops.conv_state_update(conv_in, conv_state, qs, ql, slots, 2)
        o = torch.full((T, inner), float("nan"), device=dev())
        ops.matrix_rnn("delta", u, state, qs, ql, slots, 2, o, heads=H, kv_heads=G, d=d, dv=dv, x=xc, q_col=0, k_col=qk, v_col=2 * qk,
                       b_col=cc + inner, a_col=cc + inner + H, dt_bias=dt_bias, rate=rate)
        out = torch.empty(T, inner, device=dev(), dtype=dtype)
        ops.head_norm_gate(o, gain, eps, qs, ql, 2, H, dv, out, gate=u, gate_col=cc)
        return out

    seqs, got = run_in_steps(W, steps, S, one_step, d * 7 + dv)
    m = {"heads": H, "kv_heads": G, "dim": d, "vdim": dv}
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else TOL16
    for r in range(2):
        torch.testing.assert_close(got[r], P.delta_rule(seqs[r], w, m, eps), **tol)
    assert bool(torch.isnan(state[1]).all())
    return state


@gpu
@pytest.mark.parametrize("H,G,d,dv,taps,S", [(4, 2, 8, 12, 3, 1), (2, 2, 64, 64, 4, 2), (5, 1, 20, 10, 1, 3), (1, 1, 1, 1, 2, 1), (2, 1, 128, 80, 4, 1),
                                             (1, 1, 300, 7, 2, 2), (3, 3, 17, 33, 8, 1)])
def test_delta_rule_in_portions_equals_the_whole(H, G, d, dv, taps, S):
    """Convolution with SiLU, unit norms, gate and decay, the recurrence, the heads' norm and output gate, cut into portions
    of many sizes (the read-out sees the token's own write; q and k heads shared by several value heads)."""
    check_delta(H, G, d, dv, taps, S, PORTION_STEPS)


@gpu
@pytest.mark.parametrize("H,G,d,dv,taps,S", [(2, 1, 128, 40, 4, 1), (1, 1, 300, 9, 2, 1), (3, 3, 24, 70, 3, 2), (2, 2, 5, 300, 2, 1)])
def test_delta_rule_in_long_portions(H, G, d, dv, taps, S):
    check_delta(H, G, d, dv, taps, S, LONG_STEPS)


@gpu
def test_delta_rule_decoding_token_by_token_and_in_bfloat16():
    check_delta(4, 2, 16, 24, 4, 1, DECODE_STEPS)
    check_delta(2, 1, 64, 32, 3, 2, PORTION_STEPS, torch.bfloat16)


def check_gated(H, d, dv, S, steps, dtype=torch.float32):
    from vllm_cpp_b200 import ops
    W, eps = 24, 1e-5
    g = torch.Generator().manual_seed(H * 100 + d)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F64)
    qk, inner = H * d, H * dv
    w = {"q": rnd(qk, W), "f": rnd(qk, W), "f.b": rnd(qk), "lower": torch.linspace(0.0, 0.995, qk, dtype=F64), "v": rnd(inner, W),
         "norm": 1 + 0.2 * rnd(dv), "o": torch.eye(inner, dtype=F64)}
    w_in = torch.cat([w["q"], w["f"], w["v"]])
    state = torch.zeros(3, H, dv, d, device=dev())
    state[1] = float("nan")
    f_bias, lower, gain = f32(w["f.b"]), f32(w["lower"]), f32(w["norm"])

    def one_step(rows, qs, ql, slots, lens, gen):
        T = rows.shape[0]
        u = partial_sums(rows @ w_in.T, S, gen)
        o = torch.full((T, inner), float("nan"), device=dev())
        ops.matrix_rnn("gated", u, state, qs, ql, slots, 2, o, heads=H, d=d, dv=dv, q_col=0, k_col=qk, v_col=2 * qk, f_bias=f_bias,
                       lower=lower)
        out = torch.empty(T, inner, device=dev(), dtype=dtype)
        ops.head_norm_gate(o, gain, eps, qs, ql, 2, H, dv, out)
        return out

    seqs, got = run_in_steps(W, steps, S, one_step, d * 5 + dv)
    m = {"heads": H, "dim": d, "vdim": dv}
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else TOL16
    for r in range(2):
        torch.testing.assert_close(got[r], P.hgrn2(seqs[r], w, m, eps), **tol)
    assert bool(torch.isnan(state[1]).all())


@gpu
@pytest.mark.parametrize("H,d,dv,S", [(2, 6, 10, 1), (1, 33, 5, 2), (3, 16, 8, 3), (4, 48, 32, 1), (1, 128, 128, 1), (2, 1, 3, 2), (1, 270, 40, 1)])
def test_gated_linear_recurrence_in_portions_equals_the_whole(H, d, dv, S):
    """q through a SiLU, the forget gate above its lower bound, what is written is what is not kept; lower bounds up to
    0.995 keep a token for hundreds of steps."""
    check_gated(H, d, dv, S, PORTION_STEPS)


@gpu
@pytest.mark.parametrize("H,d,dv,S", [(2, 128, 48, 1), (1, 270, 11, 1), (3, 20, 66, 2), (2, 3, 280, 1)])
def test_gated_linear_recurrence_in_long_portions(H, d, dv, S):
    check_gated(H, d, dv, S, LONG_STEPS)


@gpu
def test_gated_linear_recurrence_decoding_token_by_token_and_in_bfloat16():
    check_gated(3, 24, 16, 1, DECODE_STEPS)
    check_gated(2, 32, 64, 2, PORTION_STEPS, torch.bfloat16)


@gpu
@pytest.mark.parametrize("E,groups,keep,top", [(16, 4, 2, 4), (8, 4, 2, 2), (6, 6, 2, 1), (6, 0, 0, 3), (4, 2, 1, 2), (64, 8, 3, 6), (5, 1, 1, 2),
                                               (12, 3, 3, 5), (40, 5, 2, 7), (9, 3, 1, 3), (1, 0, 0, 1)])
def test_router_with_corrections_and_groups(E, groups, keep, top):
    """Sigmoid scores; the choice by score + correction (some negative, so that a kept group's negative choice score must
    still beat the experts outside), inside the best groups by the sum of their two largest; weights without the
    correction, times the scale; rows of padding route nowhere."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(E * 10 + top)
    T = 120
    z = torch.randn(T + 2, E, generator=g, dtype=F64) * 2
    corr = torch.randn(E, generator=g, dtype=F64) * 0.7 - 0.8
    router = {"experts": E, "top": top, "scale": 1.5, "groups": {"count": groups, "keep": keep} if groups else None}
    gaps = []
    chosen, weight = P.route(z[:T], torch.eye(E, dtype=F64), corr, router, gaps)
    qs, ql = entries_of([T // 2, 0, T - T // 2])          # the last two rows belong to no entry
    sel_e = torch.full((T + 2, top), -7, dtype=torch.int32, device=dev())
    sel_w = torch.full((T + 2, top), float("nan"), device=dev())
    ops.moe_route_grouped(partial_sums(z, 2, g), f32(corr), groups, keep, 1.5, qs, ql, 3, top, sel_e, sel_w)
    got_e, got_w = sel_e.cpu()[:T].long(), sel_w.double().cpu()[:T]
    # (a pair of scores closer than 32-bit sums can tell apart may fall either way: such rows are left out)
    sure = torch.ones(T, dtype=torch.bool)
    if gaps[0] < 1e-5:
        for t in range(T):
            one = []
            P.route(z[t:t + 1], torch.eye(E, dtype=F64), corr, router, one)
            sure[t] = one[0] >= 1e-5
    assert int(sure.sum()) >= T - 2
    assert torch.equal(got_e[sure], chosen[sure]) and bool((sel_e[T:] == -1).all())
    torch.testing.assert_close(got_w[sure], weight[sure], atol=1e-5, rtol=1e-5)


# -------------------------------------------------------------------------- whole models through the trace replay


def compare(name, dtype, trace, out_dir, requests, oracle):
    vocab = configs()[name][0].vocab
    worst = 0.0
    for step, want in enumerate(trace.wanted):
        got = R.read_step(out_dir, step, vocab)
        if not want:
            assert got is None
            continue
        assert got is not None and got.shape == (len(want), vocab), f"step {step}: {None if got is None else got.shape}"
        ref = np.stack([oracle(name, requests[rid])[pos] for rid, pos in want])
        err = np.abs(got - ref).max(axis=1) / np.abs(ref).max()
        bad = np.nonzero(~(err <= REL_TOL[dtype]))[0]
        assert len(bad) == 0, (f"{name} {dtype}: step {step}, first wrong row {want[bad[0]]} (request, position): "
                               f"relative error {err[bad[0]]:.3e} > {REL_TOL[dtype]}")
        worst = max(worst, err.max())
    return worst


MODES = {"whole": R.whole, "tail": R.tail_one_by_one, "portions": R.portions, "portions_last": R.portions_last, "mixed": R.mixed,
         "mixed_last": R.mixed_last}
REPLAYS = ([(n, "float32", m) for n in "ABCD" for m in MODES] + [(n, "bfloat16", m) for n in "ABCD" for m in ("whole", "portions", "mixed")])


@gpu
@pytest.mark.parametrize("name,dtype,mode", REPLAYS)
def test_replay(name, dtype, mode, fifudra_dirs, oracle, tmp_path):
    """Whole prompts; the last 32 tokens one by one; portions of changing size down to two tokens; up to four live
    requests with pages and slots used again -- the last two also as serving asks (logits of an entry's last token
    only: captured steps), all over a NaN-filled cache."""
    requests = requests_of(name)
    trace = MODES[mode](requests)
    out = R.run_trace(fifudra_dirs[name], dtype, trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    worst = compare(name, dtype, trace, out, requests, oracle)
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}, pool {trace.max_tokens} tokens, {len(trace.steps)} steps")


@gpu
def test_replay_modes_agree_with_each_other(fifudra_dirs, tmp_path):
    """Cutting and batching change the logits by rounding only."""
    for name in ("A", "B"):
        requests = requests_of(name)
        vocab = configs()[name][0].vocab
        rows = {}
        for mode in ("whole", "mixed", "portions"):
            trace = MODES[mode](requests)
            out = R.run_trace(fifudra_dirs[name], "float32", trace, tmp_path / (name + mode), configs()[name][1])
            for step, want in enumerate(trace.wanted):
                got = R.read_step(out, step, vocab)
                for i, key in enumerate(want):
                    rows.setdefault(key, {})[mode] = got[i]
        worst = max(np.abs(v["whole"] - v[m]).max() / np.abs(v["whole"]).max() for v in rows.values() for m in ("mixed", "portions"))
        assert worst < 2e-5, (name, worst)


@gpu
def test_long_decoding(fifudra_dirs, oracle, tmp_path):
    """A short prompt, then 250 tokens one by one: the states carried through 250 steps, the latent rows of 260 positions
    (angles of far positions, pages' borders)."""
    for name in ("A", "B"):
        toks = random_tokens(configs()[name][0].vocab, 260, 99)
        trace = R.tail_one_by_one({"long": toks}, tail=250)
        out = R.run_trace(fifudra_dirs[name], "float32", trace, tmp_path / name, configs()[name][1], extra_args=["--poison"])
        compare(name, "float32", trace, out, {"long": toks}, oracle)


# -------------------------------------------------------------------------- generation through the engine's entry point


@gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name, fifudra_dirs):
    """Several prompts at once through LLM.generate (scheduler, portions under a small token budget, captured decoding
    steps, device-side sampling at temperature 0) against the plain implementation's greedy continuation."""
    from vllm_cpp_b200 import LLM
    cfg, w = P.read_model(fifudra_dirs[name])
    vocab, page = configs()[name][0].vocab, configs()[name][1]
    prompts = [random_tokens(vocab, n, 3 + n) for n in (5, 41, 18, 70, 2)]
    llm = LLM(str(fifudra_dirs[name]), dtype="float32", page_size=page, max_tokens=page * 64, max_num_seqs=3, max_step_tokens=32,
              max_model_len=256)
    got = llm.generate(prompts, max_new_tokens=24, temperature=0.0, top_p=1.0, repeat_penalty=1.0, ignore_eos=True)
    for prompt, g in zip(prompts, got):
        want = P.greedy(cfg, w, prompt, 24)
        # a near tie between two logits may fall the other way in 32-bit: compare up to the first such place
        for i, (a, b) in enumerate(zip(g, want)):
            if a != b:
                logits = P.forward(cfg, w, prompt + want[:i])[-1]
                assert abs(float(logits[a] - logits[b])) < 1e-4, (i, a, b)
                break
        assert len(g) == 24
