"""Mefupel in the engine against the plain implementation (tests/plain_mefupel.py): each mechanism's kernel alone, then
whole models through bin/trace_run (whole prompts, decoding, portions down to two tokens, mixed batches with pages and
slots used again) and greedy generation through the engine's entry point, on small configurations of its own."""
import json
import math

import numpy as np
import pytest
import torch

import plain_mefupel as P
import replay_util as R
from conftest import random_tokens

gpu = pytest.mark.gpu
F64 = torch.float64


def configs():
    from vllm_cpp_b200.config.mefupel import (AttentionSpec as A, GlaSpec as G, MefupelConfig, MefupelLayer as L, MefupelMlp as F,
                                              ParallelSpec as Par, RetentionSpec as Ret, Rotation as Rot)
    return {
        # the last three layers run twice; fewer turning lanes than plain ones everywhere; values narrower than keys; three
        # retention heads with decays from fast to slow; an attention layer without a feed-forward; windows of 9 and 5
        # keys over pages of 4
        "A": (MefupelConfig(vocab=150, width=48, norm_eps=1e-5, has_loop=True, loop_start=1, loop_stop=4, loop_times=2, layers=(
            L("gla", G(heads=2, dim=6, vdim=10, tau=8.0, rank=5), F("dense", ff=40)),
            L("parallel", Par(A(heads=4, kv_heads=2, dim=8, vdim=8, scale=0.35, window=9, rot=Rot(100.0, 4)),
                              Ret(heads=3, dim=6, vdim=4, decay=(0.9, 0.99, 0.5), rot=Rot(50.0, 4))), F("dense", ff=24)),
            L("attention", A(heads=4, kv_heads=2, dim=8, vdim=6, scale=0.4, window=5, rot=Rot(1000.0, 4))),
            L("gla", G(heads=3, dim=4, vdim=4, tau=2.0, rank=8), F("dense", ff=16)))), 4),
        # nothing repeated; heads of 64 lanes, which bfloat16 runs on the tensor cores: an attention over all earlier
        # tokens on one KV head, a left branch under a window of 33 with half of its lanes turning; state rows of 64
        # lanes and values twice as wide; pages of 16
        "B": (MefupelConfig(vocab=260, width=64, norm_eps=1e-6, layers=(
            L("attention", A(heads=2, kv_heads=1, dim=64, vdim=64, scale=0.125, window=0, rot=Rot(10000.0, 64)), F("dense", ff=48)),
            L("parallel", Par(A(heads=2, kv_heads=2, dim=64, vdim=64, scale=0.11, window=33, rot=Rot(500.0, 32)),
                              Ret(heads=1, dim=64, vdim=64, decay=(0.97,), rot=Rot(1e6, 64))), F("dense", ff=32)),
            L("gla", G(heads=1, dim=64, vdim=128, tau=16.0, rank=16), F("dense", ff=24)))), 16),
        # a width that is no multiple of 4; the first layer alone runs three times; five heads on one KV head with two
        # turning lanes under a window of one key (a token sees itself only); one head of 33 state rows, a rank of 3, no
        # feed-forward; a retention whose lanes do not turn at all; pages of 8
        "C": (MefupelConfig(vocab=97, width=50, norm_eps=1e-4, has_loop=True, loop_start=0, loop_stop=1, loop_times=3, layers=(
            L("attention", A(heads=5, kv_heads=1, dim=6, vdim=10, scale=1.0, window=1, rot=Rot(50.0, 2)), F("dense", ff=11)),
            L("gla", G(heads=1, dim=33, vdim=5, tau=1.0, rank=3)),
            L("parallel", Par(A(heads=3, kv_heads=3, dim=10, vdim=10, scale=0.3, window=20, rot=Rot(30.0, 10)),
                              Ret(heads=2, dim=5, vdim=7, decay=(0.999, 0.75), rot=Rot(10.0, 0))), F("dense", ff=9)))), 8),
    }


LENGTHS = {"A": [40, 75, 150, 33, 2, 17, 64], "B": [1, 7, 33, 64, 170, 97, 3], "C": [50, 3, 77, 31, 9]}
REL_TOL = {"float32": 2e-5, "bfloat16": 3e-2}


def hand_made(cfg, tensors, seed):
    """The random tensors, changed so that a fault shows: sharp softmaxes (single keys, often far ones or ones at a
    window's edge, carry the rows), sinks that take a real share, decays spread from fast to slow, and an activation
    in which all four numbers matter."""
    g = torch.Generator().manual_seed(seed)
    out = dict(tensors)
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}.mix."
        if layer.type == "attention":
            out[p + "q"] = tensors[p + "q"] * 12.0
            out[p + "k"] = tensors[p + "k"] * 12.0
        elif layer.type == "parallel":
            n = tensors[p + "left.sink"].numel()
            out[p + "left.sink"] = torch.linspace(-1.5, 2.5, n)
            out[p + "left.q.norm"] = tensors[p + "left.q.norm"] * 2.5
            out[p + "left.k.norm"] = tensors[p + "left.k.norm"] * 2.5
        elif layer.type == "gla":
            n = tensors[p + "a2.b"].numel()
            out[p + "a2.b"] = torch.linspace(-2.0, 7.0, n)[torch.randperm(n, generator=g)]
            out[p + "a2"] = tensors[p + "a2"] * 20.0
        if layer.mlp is not None:
            out[f"l{i}.mlp.act"] = torch.tensor([0.9, -0.4, 0.3, 0.05])
    out["loop.step"] = tensors["loop.step"] * 5.0 if "loop.step" in tensors else None
    return {k: v.to(torch.bfloat16) for k, v in out.items() if v is not None}


@pytest.fixture(scope="module")
def mefupel_dirs(tmp_path_factory):
    from vllm_cpp_b200 import write_random_model
    from vllm_cpp_b200.weights.safetensors_io import read_safetensors, write_safetensors
    out = {}
    for i, (name, (cfg, _)) in enumerate(configs().items()):
        d = tmp_path_factory.mktemp(f"mefupel_{name}")
        write_random_model(cfg, 41 + i, d, dtype="bfloat16")
        tensors = {k: v.float() for k, v in read_safetensors(d / "model.safetensors").items()}
        write_safetensors(d / "model.safetensors", hand_made(cfg, tensors, 5 + i), {"format": "pt"})
        # the rank of the decay's projection is not a key of a model folder's configuration: the tensors say it
        c = json.loads((d / "config.json").read_text())
        for layer in c["layers"]:
            layer["mixer"].pop("rank", None)
        (d / "config.json").write_text(json.dumps(c))
        out[name] = d
    return out


class Oracle:
    def __init__(self, dirs):
        self.models = {n: P.read_model(d) for n, d in dirs.items()}
        self.cache = {}

    def __call__(self, name, tokens):
        key = (name, tuple(tokens))
        if key not in self.cache:
            self.cache[key] = P.forward(*self.models[name], list(tokens)).numpy()
        return self.cache[key]


@pytest.fixture(scope="module")
def oracle(mefupel_dirs):
    return Oracle(mefupel_dirs)


def requests_of(name):
    vocab = configs()[name][0].vocab
    return {f"r{i}": random_tokens(vocab, n, 11 * i + len(name)) for i, n in enumerate(LENGTHS[name])}


# -------------------------------------------------------------------------- without a GPU


def test_config_reads_every_size_and_constant():
    from vllm_cpp_b200 import ConfigError
    from vllm_cpp_b200.config.mefupel import MefupelConfig
    d = {"architecture": "Mefupel", "vocab": 50, "width": 24, "norm": {"eps": 3e-4}, "loop": {"start": 1, "stop": 3, "times": 4},
         "layers": [{"type": "attention", "mlp": None,
                     "mixer": {"heads": 6, "kv_heads": 3, "dim": 10, "vdim": 14, "scale": 0.5, "mask": {"size": 7},
                               "rot": {"base": 777.0, "dims": 6}}},
                    {"type": "gla", "mlp": {"kind": "dense", "ff": 31}, "mixer": {"heads": 4, "dim": 6, "vdim": 9, "tau": 12.5}},
                    {"type": "parallel", "mlp": {"kind": "dense", "ff": 5},
                     "mixer": {"left": {"heads": 2, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.25, "mask": {"size": 3},
                                        "rot": {"base": 9.0, "dims": 4}},
                               "right": {"heads": 2, "dim": 6, "vdim": 12, "decay": [0.5, 0.875], "rot": {"base": 11.0, "dims": 2}}}},
                    {"type": "gla", "mlp": None, "mixer": {"heads": 1, "dim": 2, "vdim": 2, "tau": 1}}]}
    cfg = MefupelConfig.from_dict(d)
    assert (cfg.vocab, cfg.width, cfg.norm_eps) == (50, 24, 3e-4)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times, cfg.has_loop) == (1, 3, 4, True)
    assert cfg.runs() == ((0, None), (1, 0), (2, None), (1, 1), (2, None), (1, 2), (2, None), (1, 3), (2, None), (3, None))
    a, b, c, e = cfg.layers
    m = a.mixer
    assert (m.heads, m.kv_heads, m.dim, m.vdim, m.scale, m.window, m.rot.base, m.rot.dims, a.mlp) == (6, 3, 10, 14, 0.5, 7, 777.0, 6, None)
    assert (b.mixer.heads, b.mixer.dim, b.mixer.vdim, b.mixer.tau, b.mixer.rank, b.mlp.kind, b.mlp.ff) == (4, 6, 9, 12.5, 0, "dense", 31)
    l, r = c.mixer.left, c.mixer.right
    assert (l.heads, l.kv_heads, l.dim, l.vdim, l.scale, l.window, l.rot.base, l.rot.dims) == (2, 1, 8, 8, 0.25, 3, 9.0, 4)
    assert (r.heads, r.dim, r.vdim, r.decay, r.rot.base, r.rot.dims) == (2, 6, 12, (0.5, 0.875), 11.0, 2)
    assert MefupelConfig.from_dict(cfg.to_dict()) == cfg
    # what is left out is off: no repetition (and no vector per pass), an attention over all earlier tokens
    bare = MefupelConfig.from_dict({k: v for k, v in d.items() if k != "loop"})
    assert (bare.has_loop, bare.runs()) == (False, ((0, None), (1, None), (2, None), (3, None)))
    assert MefupelConfig.from_dict(dict(d, loop=None)).runs() == bare.runs()
    unmasked = dict(d["layers"][0], mixer={k: v for k, v in d["layers"][0]["mixer"].items() if k != "mask"})
    assert MefupelConfig.from_dict(dict(d, layers=[unmasked], loop=None)).layers[0].mixer.window == 0
    layer = d["layers"]
    for bad in ({"layers": []}, {"layers": [dict(layer[0], type="other")]}, {"loop": {"start": 2, "stop": 5, "times": 2}},
                {"layers": [dict(layer[0], mixer=dict(layer[0]["mixer"], kv_heads=4))], "loop": None},
                {"layers": [dict(layer[0], mixer=dict(layer[0]["mixer"], rot={"base": 5.0, "dims": 3}))], "loop": None},
                {"layers": [dict(layer[0], mixer=dict(layer[0]["mixer"], rot={"base": 5.0, "dims": 12}))], "loop": None},
                {"layers": [dict(layer[2], mixer=dict(layer[2]["mixer"], right=dict(layer[2]["mixer"]["right"], decay=[0.5])))], "loop": None},
                {"layers": [dict(layer[2], mixer=dict(layer[2]["mixer"], left=dict(layer[2]["mixer"]["left"], vdim=6)))], "loop": None},
                {"layers": [dict(layer[1], mlp={"kind": "routed", "ff": 3})], "loop": None}, {"vocab": None}):
        with pytest.raises(ConfigError):
            MefupelConfig.from_dict(dict(d, **bad))


def test_model_folder_is_recognised_and_names_its_tensors(tmp_path):
    from vllm_cpp_b200.models import expected_tensors, load_config
    cfg, _ = configs()["A"]
    (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
    assert load_config(tmp_path) == cfg
    s = {t.name: tuple(t.shape) for t in expected_tensors(cfg)}
    assert s["embed"] == s["head"] == (150, 48) and s["final.norm"] == (48,) and s["loop.step"] == (2, 48)
    assert s["l0.norm1"] == (48,) and not any(k.startswith("l0.norm2") for k in s)
    assert s["l0.mix.q"] == s["l0.mix.k"] == (12, 48) and s["l0.mix.v"] == s["l0.mix.g"] == (20, 48) and s["l0.mix.o"] == (48, 20)
    assert s["l0.mix.a1"] == (5, 48) and s["l0.mix.a2"] == (12, 5) and s["l0.mix.a2.b"] == (12,) and s["l0.mix.norm"] == (10,)
    assert s["l0.mlp.up"] == (40, 48) and s["l0.mlp.down"] == (48, 40) and s["l0.mlp.act"] == (4,)
    assert s["l1.mix.left.q"] == (32, 48) and s["l1.mix.left.k"] == (16, 48) and "l1.mix.left.v" not in s
    assert s["l1.mix.left.q.norm"] == (32,) and s["l1.mix.left.k.norm"] == (16,) and s["l1.mix.left.sink"] == (4,)
    assert s["l1.mix.left.o"] == (48, 32) and s["l1.mix.left.out"] == s["l1.mix.right.out"] == (48,)
    assert s["l1.mix.right.q"] == s["l1.mix.right.k"] == (18, 48) and s["l1.mix.right.v"] == s["l1.mix.right.g"] == (12, 48)
    assert s["l1.mix.right.o"] == (48, 12)
    assert s["l2.mix.q"] == (32, 48) and s["l2.mix.k"] == (16, 48) and s["l2.mix.v"] == (12, 48) and s["l2.mix.o"] == (48, 24)
    assert not any(k.startswith("l2.mlp") for k in s)                       # a layer without a feed-forward
    b, _ = configs()["B"]
    assert "loop.step" not in {t.name for t in expected_tensors(b)}         # no repetition, no vector per pass
    # without the optional key the rank is whatever the tensors have
    from vllm_cpp_b200.config.mefupel import MefupelConfig
    c = cfg.to_dict()
    del c["layers"][0]["mixer"]["rank"]
    s = {t.name: tuple(t.shape) for t in expected_tensors(MefupelConfig.from_dict(c))}
    assert s["l0.mix.a1"] == (-1, 48) and s["l0.mix.a2"] == (12, -1)


def test_a_size_that_only_the_tensors_know_is_checked_when_they_are_bound():
    from vllm_cpp_b200.weights.loader import TensorSpec, WeightError, WeightStore
    specs = [TensorSpec("a1", (-1, 8)), TensorSpec("a2", (6, -1))]
    WeightStore({"a1": torch.zeros(3, 8), "a2": torch.zeros(6, 3)}, torch.float32, "cpu").check(specs)
    WeightStore({"a1": torch.zeros(5, 8), "a2": torch.zeros(6, 3)}, torch.float32, "cpu").check(specs)    # (the part compares the two)
    with pytest.raises(WeightError):
        WeightStore({"a1": torch.zeros(3, 9), "a2": torch.zeros(6, 3)}, torch.float32, "cpu").check(specs)
    with pytest.raises(WeightError):
        WeightStore({"a1": torch.zeros(3, 8, 1), "a2": torch.zeros(6, 3)}, torch.float32, "cpu").check(specs)


def test_what_a_layer_run_keeps_per_request():
    """Every run of a layer, a repeated one too, has pages and states of its own."""
    import vllm_cpp_b200.models as models
    cfg, _ = configs()["A"]
    model = models.build_model(cfg, torch.float32, "cpu")
    assert [(r.layer, r.opens) for r in model.order] == [(0, None), (1, 0), (2, None), (3, None), (1, 1), (2, None), (3, None)]
    specs = model.cache_specs()
    st = specs[0]
    assert (st.kind, st.shape, st.dtype) == ("state", (2, 10, 6), "float32")
    for run in (1, 4):      # the parallel mixer: the left branch's pages, then the right branch's state
        kv, rs = specs[(run, 0)], specs[(run, 1)]
        assert (kv.kind, kv.num_kv_heads, kv.head_dim, kv.window, kv.v_head_dim) == ("kv", 2, 8, 9, 0)
        assert (rs.kind, rs.shape) == ("state", (3, 4, 6))
    for run in (2, 5):
        kv = specs[run]
        assert (kv.kind, kv.num_kv_heads, kv.head_dim, kv.window, kv.v_head_dim) == ("kv", 2, 8, 5, 6)
    assert specs[3].shape == specs[6].shape == (3, 4, 4)


def test_oracle_mechanisms_by_hand():
    pos = torch.tensor([0, 3])
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0]], [[1.0, 2.0, 3.0, 4.0, 5.0]]], dtype=F64)
    f = [1.0, 10.0 ** -0.5]          # base^(-2i / dims), i = 0, 1
    # halves: lane 0 with lane 2, lane 1 with lane 3; the fifth lane passes
    h = P.rotate(x, pos, 10.0, 4, "half")
    assert torch.equal(h[0], x[0])
    c0, s0, c1, s1 = math.cos(3 * f[0]), math.sin(3 * f[0]), math.cos(3 * f[1]), math.sin(3 * f[1])
    want = torch.tensor([1 * c0 - 3 * s0, 2 * c1 - 4 * s1, 3 * c0 + 1 * s0, 4 * c1 + 2 * s1, 5.0], dtype=F64)
    torch.testing.assert_close(h[1, 0], want)
    # neighbours: lane 0 with lane 1, lane 2 with lane 3
    n = P.rotate(x, pos, 10.0, 4, "interleaved")
    want = torch.tensor([1 * c0 - 2 * s0, 2 * c0 + 1 * s0, 3 * c1 - 4 * s1, 4 * c1 + 3 * s1, 5.0], dtype=F64)
    torch.testing.assert_close(n[1, 0], want)
    torch.testing.assert_close(P.rotate(n, pos, 10.0, 4, "interleaved", sign=-1.0), x)
    # a window of two keys and a sink: position 2 sees keys 1 and 2
    q = torch.tensor([[[1.0]], [[1.0]], [[2.0]]], dtype=F64)
    k = torch.tensor([[[5.0]], [[1.0]], [[0.5]]], dtype=F64)
    v = torch.tensor([[[1.0, 0.0]], [[0.0, 1.0]], [[1.0, 1.0]]], dtype=F64)
    o = P.window_softmax_attention(q, k, v, 0.5, 2, sink=torch.tensor([0.25], dtype=F64))
    e1, e2, es = math.exp(0.5 * 2 * 1.0), math.exp(0.5 * 2 * 0.5), math.exp(0.25)
    torch.testing.assert_close(o[2, 0], torch.tensor([e2 / (e1 + e2 + es), (e1 + e2) / (e1 + e2 + es)], dtype=F64))
    o = P.window_softmax_attention(q, k, v, 0.5, 0)
    e0 = math.exp(0.5 * 2 * 5.0)
    torch.testing.assert_close(o[2, 0], torch.tensor([(e0 + e2) / (e0 + e1 + e2), (e1 + e2) / (e0 + e1 + e2)], dtype=F64))
    # the decay acts on the rows of the key channels
    out, S = P.decayed_state_scan(torch.tensor([[1.0, 1.0], [1.0, 0.0]], dtype=F64), torch.tensor([[1.0, 2.0], [3.0, 4.0]], dtype=F64),
                                  torch.tensor([[1.0], [10.0]], dtype=F64), torch.tensor([[0.5, 0.25], [0.5, 0.25]], dtype=F64))
    torch.testing.assert_close(S, torch.tensor([[0.5 * 1.0 + 30.0], [0.25 * 2.0 + 40.0]], dtype=F64))
    torch.testing.assert_close(out, torch.tensor([[3.0], [30.5]], dtype=F64))
    z = torch.tensor([[1.0, -2.0]], dtype=F64)
    r2, r4, r6 = math.sqrt(2.5), math.sqrt(8.5), math.sqrt(32.5)
    want = torch.tensor([[2 * 1 / r2 + 3 * 1 / r4 + 4 * 1 / r6 + 5, 2 * -2 / r2 + 3 * 4 / r4 + 4 * -8 / r6 + 5]], dtype=F64)
    torch.testing.assert_close(P.polynorm(z, [2.0, 3.0, 4.0, 5.0], 0.0), want)
    assert P.passes({"layers": [0, 1, 2], "loop": {"start": 0, "stop": 2, "times": 2}}) == [(0, 0), (1, None), (0, 1), (1, None), (2, None)]


# -------------------------------------------------------------------------- on the GPU: each kernel alone


def dev():
    return torch.device("cuda:0")


def i32(x):
    return torch.tensor(x, dtype=torch.int32, device=dev())


def f32(x):
    return None if x is None else x.float().contiguous().to(dev())


def entries_of(lengths):
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
@pytest.mark.parametrize("W,n_terms,S,out_dtype", [(6, 1, 1, torch.float32), (50, 2, 2, torch.bfloat16), (320, 2, 3, torch.float32),
                                                   (2500, 4, 1, torch.bfloat16), (64, 0, 1, torch.float32), (13000, 1, 2, torch.float32),
                                                   (12288, 2, 1, torch.bfloat16)])
def test_pending_results_are_added_and_normed_in_one_pass(W, n_terms, S, out_dtype):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(W + n_terms)
    T, eps = 7, 1e-5
    x = torch.randn(T, W, generator=g, dtype=F64)
    terms = [torch.randn(T, W, generator=g, dtype=F64) for _ in range(n_terms)]
    first, vec, gain = torch.randn(T, W, generator=g, dtype=F64), torch.randn(W, generator=g, dtype=F64), torch.randn(W, generator=g, dtype=F64)
    tol = TOL32 if out_dtype == torch.float32 else TOL16
    for extras in (False, True):
        want = x + sum(terms) + (first + vec if extras else 0)
        resid = f32(x)
        out = torch.empty(T, W, dtype=out_dtype, device=dev())
        ops.sum_add_rmsnorm(resid, [partial_sums(t, S if k == 0 else 1, g) for k, t in enumerate(terms)], f32(gain), eps, out,
                            row_extra=f32(first) if extras else None, vec_extra=f32(vec) if extras else None)
        torch.testing.assert_close(resid.double().cpu(), want, **TOL32)
        torch.testing.assert_close(out.double().cpu(), P.rms(want, eps) * gain, **tol)
        # on a list of rows the stream stays as it is
        resid, rows = f32(x), i32([5, 0, 5])
        out = torch.full((3, W), float("nan"), dtype=out_dtype, device=dev())
        ops.sum_add_rmsnorm(resid, [f32(t) for t in terms], f32(gain), eps, out, rows, f32(first) if extras else None,
                            f32(vec) if extras else None)
        torch.testing.assert_close(out.double().cpu(), (P.rms(want, eps) * gain)[[5, 0, 5]], **tol)
        assert torch.equal(resid.cpu(), x.float())
        # the additions alone
        resid = f32(x)
        ops.sum_add_rmsnorm(resid, [f32(t) for t in terms], None, 0.0, None, None, f32(first) if extras else None, f32(vec) if extras else None)
        torch.testing.assert_close(resid.double().cpu(), want, **TOL32)


@gpu
@pytest.mark.parametrize("W,n,S", [(6, 2, 1), (50, 2, 2), (200, 1, 3), (1000, 3, 1), (4096, 2, 2), (77, 4, 1), (6144, 2, 1)])
def test_results_of_mixers_side_by_side_are_normed_and_averaged(W, n, S):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(W * n)
    T, eps = 9, 1e-5
    ys = [torch.randn(T, W, generator=g, dtype=F64) * (10.0 ** b) for b in range(n)]      # results of very different size
    gains = [torch.randn(W, generator=g, dtype=F64) for _ in range(n)]
    out = torch.full((T, W), float("nan"), device=dev())
    ops.branch_norm_mean([partial_sums(y, S, g) for y in ys], [f32(w) for w in gains], eps, out)
    want = sum(P.rms(y, eps) * w for y, w in zip(ys, gains)) / n
    torch.testing.assert_close(out.double().cpu(), want, atol=1e-4, rtol=1e-4)


@gpu
@pytest.mark.parametrize("F,S,dtype", [(5, 1, torch.float32), (40, 2, torch.bfloat16), (256, 1, torch.float32), (3000, 3, torch.float32),
                                       (14336, 1, torch.bfloat16), (12288, 1, torch.bfloat16)])
def test_normed_polynomial_activation(F, S, dtype):
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(F)
    T, eps = 6, 1e-5
    z = torch.randn(T, F, generator=g, dtype=F64) * 1.7
    if S == 1:
        z[2] *= 1e-3    # a row so small that eps decides (as partial sums of ordinary size it would lose its digits on the way in)
    coef = torch.tensor([0.8, -0.5, 0.25, 0.1], dtype=F64)
    out = torch.empty(T, F, dtype=dtype, device=dev())
    ops.polynorm(partial_sums(z, S, g), f32(coef), eps, out)
    torch.testing.assert_close(out.double().cpu(), P.polynorm(z, coef, eps), **(TOL32 if dtype == torch.float32 else TOL16))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,vd,rot,pairing,whole,from_keys,turn_values,S", [
    (4, 2, 8, 6, 4, "interleaved", False, False, True, 1), (2, 1, 64, 64, 64, "interleaved", False, False, True, 2),
    (4, 2, 8, 8, 4, "half", True, True, False, 1), (6, 3, 80, 80, 40, "half", True, True, False, 3),
    (5, 1, 6, 10, 2, "interleaved", False, False, True, 1), (3, 3, 10, 10, 0, "half", True, True, False, 2),
    (2, 2, 16, 16, 16, "half", False, False, False, 1)])
def test_norm_rotation_and_store_ahead_of_attention(dtype, nh, nkv, hd, vd, rot, pairing, whole, from_keys, turn_values, S):
    """Queries to their buffer, keys and values to the tokens' places in the pages -- in both page layouts, at near and far
    positions, with rows that are stored nowhere."""
    from vllm_cpp_b200 import ops
    g = torch.Generator().manual_seed(nh * 31 + hd)
    T, ps, n_pages, eps, base = 6, 4, 5, 1e-5, 37.0
    pos = [0, 1, 5, 5000, 33, 2]
    slots = [3, 17, -1, 8, 0, 19]
    C = nh * hd + nkv * hd + (0 if from_keys else nkv * vd)
    u = torch.randn(T, C, generator=g, dtype=F64)
    gq, gk = (1 + 0.3 * torch.randn(nh * hd, generator=g, dtype=F64), 1 + 0.3 * torch.randn(nkv * hd, generator=g, dtype=F64)) if whole else (None, None)
    freq = f32(P.frequencies(base, rot)) if rot else None
    vfreq = f32(P.frequencies(base, vd)) if turn_values else None
    q_out = torch.full((T, nh * hd), float("nan"), dtype=dtype, device=dev())
    if vd == hd:
        pages = torch.full((n_pages, 2, nkv, ps, hd), float("nan"), dtype=dtype, device=dev())
    else:
        pages = torch.full((n_pages, nkv * ps * (hd + vd)), float("nan"), dtype=dtype, device=dev())
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    ops.qkv_rope_store(partial_sums(u, S, g), f32(gq), f32(gk), eps, i32(pos), freq, vfreq, i32(slots), q_out, pages, nh, nkv, hd, vd,
                       status, rot=rot, interleaved=pairing == "interleaved", values_from_keys=from_keys)
    assert int(status.item()) == 0
    P_ = torch.tensor(pos)
    q, k = u[:, :nh * hd], u[:, nh * hd:nh * hd + nkv * hd]
    v = k.view(T, nkv, hd) if from_keys else u[:, nh * hd + nkv * hd:].view(T, nkv, vd)
    if whole:
        q, k = P.rms(q, eps) * gq, P.rms(k, eps) * gk
    q = P.rotate(q.reshape(T, nh, hd), P_, base, rot, pairing)
    k = P.rotate(k.reshape(T, nkv, hd), P_, base, rot, pairing)
    if turn_values:
        v = P.rotate(v, P_, base, vd, pairing)
    tol = TOL32 if dtype == torch.float32 else TOL16
    if dtype == torch.float32:
        tol = dict(atol=3e-3, rtol=1e-4)     # (an angle is a 32-bit product: at position 5,000 it is good to 2e-4)
    torch.testing.assert_close(q_out.double().cpu().view(T, nh, hd), q, **tol)
    flat = pages.double().cpu().view(n_pages, -1)
    keys = flat[:, :nkv * ps * hd].view(n_pages, nkv, ps, hd)
    vals = flat[:, nkv * ps * hd:].view(n_pages, nkv, ps, vd)
    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for t, s in enumerate(slots):
        if s < 0:
            continue
        written[s // ps, s % ps] = True
        torch.testing.assert_close(keys[s // ps, :, s % ps], k[t], **tol)
        torch.testing.assert_close(vals[s // ps, :, s % ps], v[t], **tol)
    assert bool(torch.isnan(keys[~written[:, None, :].expand(-1, nkv, -1)]).all())       # nothing else was touched
    # and the heads' sums turned back
    if turn_values:
        o = torch.randn(T, nh, vd, generator=g, dtype=F64)
        buf = P.rotate(o, P_, base, vd, pairing).reshape(T, nh * vd).to(dtype).to(dev())
        ops.rotate_heads(buf, i32(pos), vfreq, heads=nh, width=vd, dims=vd, interleaved=pairing == "interleaved", sign=-1.0)
        torch.testing.assert_close(buf.double().cpu().view(T, nh, vd), o, **(dict(atol=5e-3, rtol=1e-3) if dtype == torch.float32 else TOL16))


PORTION_STEPS = [(3, 1), (1, 1), (2, 7), (1, 2), (9, 1), (1, 0), (2, 2), (1, 1), (1, 1), (1, 1), (16, 1), (1, 17)]
DECODE_STEPS = [(4, 2)] + [(1, 1)] * 45
# portions of several staged batches each (the kernels stage 8 or 16 tokens at a time), ending on, before and behind a batch's edge
LONG_STEPS = [(37, 16), (1, 33), (48, 5), (17, 32), (8, 9), (70, 1)]


def run_in_steps(W, steps, one_step, seed):
    """Two requests (in slots 2 and 0 of three) cut as ``steps`` says, two rows of padding behind every step;
    ``one_step(rows, qs, ql, slots, ctx_len, gen)`` -> that step's result rows.  Returns the requests' inputs and results."""
    g = torch.Generator().manual_seed(seed)
    total = [sum(s[0] for s in steps), sum(s[1] for s in steps)]
    seqs = [torch.randn(n, W, generator=g, dtype=F64) for n in total]
    got, at = [[], []], [0, 0]
    for n0, n1 in steps:
        lens = [n0, n1]
        rows = torch.cat([seqs[r][at[r]:at[r] + lens[r]] for r in range(2)] + [torch.full((2, W), float("nan"), dtype=F64)])
        qs, ql = entries_of(lens)
        o = one_step(rows, qs, ql, i32([2, 0]), i32([at[0] + n0, at[1] + n1]), g).double().cpu()
        got[0].append(o[:n0]); got[1].append(o[n0:n0 + n1])
        at = [at[0] + n0, at[1] + n1]
    return seqs, [torch.cat(x) for x in got]


def check_decayed(H, d, dv, rank, tau, S, steps, dtype=torch.float32):
    from vllm_cpp_b200 import ops
    W, eps = 24, 1e-5
    g = torch.Generator().manual_seed(H * 100 + d)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F64)
    qk, inner = H * d, H * dv
    w = {"q": rnd(qk, W), "k": rnd(qk, W) * 0.3, "v": rnd(inner, W), "g": rnd(inner, W) * 0.5, "a1": rnd(rank, W), "a2": rnd(qk, rank),
         "a2.b": torch.linspace(-3.0, 8.0, qk, dtype=F64), "norm": 1 + 0.2 * rnd(dv), "o": torch.eye(inner, dtype=F64)}
    w_in = torch.cat([w[n] for n in ("q", "k", "v", "g")])
    state = torch.zeros(3, H, dv, d, device=dev())
    state[1] = float("nan")

    def one_step(rows, qs, ql, slots, ctx_len, gen):
        T = rows.shape[0]
        u = partial_sums(rows @ w_in.T, S, gen)
        z = partial_sums((rows @ w["a1"].T) @ w["a2"].T, min(S, 2), gen)
        o = torch.full((T, inner), float("nan"), device=dev())
        ops.matrix_rnn("decayed", u, state, qs, ql, slots, 2, o, heads=H, d=d, dv=dv, q_col=0, k_col=qk, v_col=2 * qk, z=z,
                       f_bias=f32(w["a2.b"]), tau=tau)
        out = torch.empty(T, inner, device=dev(), dtype=dtype)
        ops.head_norm_gate(o, f32(w["norm"]), eps, qs, ql, 2, H, dv, out, gate=u, gate_col=2 * qk + inner)
        return out

    seqs, got = run_in_steps(W, steps, one_step, d * 7 + dv)
    m = {"heads": H, "dim": d, "vdim": dv, "tau": tau}
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else TOL16
    for r in range(2):
        torch.testing.assert_close(got[r], P.gla(seqs[r], w, m, eps), **tol)
    assert bool(torch.isnan(state[1]).all())        # the neighbour's slot is untouched


@gpu
@pytest.mark.parametrize("H,d,dv,rank,tau,S", [(2, 6, 10, 5, 8.0, 1), (1, 33, 5, 3, 1.0, 2), (3, 16, 8, 16, 16.0, 3), (4, 40, 56, 12, 10.0, 1),
                                               (1, 128, 128, 8, 4.0, 1), (2, 1, 3, 1, 2.0, 2), (1, 270, 40, 7, 32.0, 1)])
def test_decayed_linear_recurrence_in_portions_equals_the_whole(H, d, dv, rank, tau, S):
    check_decayed(H, d, dv, rank, tau, S, PORTION_STEPS)


@gpu
@pytest.mark.parametrize("H,d,dv,rank,tau,S", [(2, 128, 48, 16, 16.0, 1), (1, 270, 11, 4, 3.0, 1), (3, 20, 66, 6, 8.0, 2), (2, 3, 280, 2, 1.5, 1)])
def test_decayed_linear_recurrence_in_long_portions(H, d, dv, rank, tau, S):
    check_decayed(H, d, dv, rank, tau, S, LONG_STEPS)


@gpu
def test_decayed_linear_recurrence_decoding_token_by_token_and_in_bfloat16():
    check_decayed(3, 40, 72, 12, 6.0, 2, DECODE_STEPS)
    check_decayed(2, 16, 24, 4, 8.0, 1, PORTION_STEPS, dtype=torch.bfloat16)


def check_retention(H, d, dv, rot, pairing, decay, S, steps, dtype=torch.float32):
    from vllm_cpp_b200 import ops
    W, eps, base = 24, 1e-5, 61.0
    g = torch.Generator().manual_seed(H * 100 + d + rot)
    rnd = lambda *shape: torch.randn(*shape, generator=g, dtype=F64)
    qk, inner = H * d, H * dv
    w = {"q": rnd(qk, W), "k": rnd(qk, W), "v": rnd(inner, W), "g": rnd(inner, W) * 0.5, "o": torch.eye(inner, dtype=F64)}
    w_in = torch.cat([w[n] for n in ("q", "k", "v", "g")])
    state = torch.zeros(3, H, dv, d, device=dev())
    state[1] = float("nan")
    freq = f32(P.frequencies(base, rot)) if rot else None
    dec = f32(torch.tensor(decay, dtype=F64))

    def one_step(rows, qs, ql, slots, ctx_len, gen):
        T = rows.shape[0]
        u = partial_sums(rows @ w_in.T, S, gen)
        o = torch.full((T, inner), float("nan"), device=dev())
        ops.matrix_rnn("retention", u, state, qs, ql, slots, 2, o, heads=H, d=d, dv=dv, q_col=0, k_col=qk, v_col=2 * qk, decay=dec,
                       ctx_len=ctx_len, freq=freq, rot=rot, interleaved=pairing == "interleaved")
        out = torch.empty(T, inner, device=dev(), dtype=dtype)
        ops.head_norm_gate(o, None, eps, qs, ql, 2, H, dv, out, gate=u, gate_col=2 * qk + inner)
        return out

    seqs, got = run_in_steps(W, steps, one_step, d * 5 + dv)
    tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else TOL16
    for r in range(2):
        T = seqs[r].shape[0]
        h, positions = seqs[r], torch.arange(T)
        q = P.rotate((h @ w["q"].T).view(T, H, d), positions, base, rot, pairing)
        k = P.rotate((h @ w["k"].T).view(T, H, d), positions, base, rot, pairing) * d ** -0.5
        v = (h @ w["v"].T).view(T, H, dv)
        o = torch.stack([P.decayed_state_scan(q[:, i], k[:, i], v[:, i], torch.full((T, d), decay[i], dtype=F64))[0] for i in range(H)], 1)
        want = P.rms(o, eps).reshape(T, inner) * P.silu(h @ w["g"].T)
        torch.testing.assert_close(got[r], want, **tol)
        if pairing == "half":       # the oracle's own mixer says the same
            m = {"heads": H, "dim": d, "vdim": dv, "decay": list(decay), "rot": {"base": base, "dims": rot}}
            torch.testing.assert_close(P.retention(h, w, m, eps, positions), want)
    assert bool(torch.isnan(state[1]).all())


@gpu
@pytest.mark.parametrize("H,d,dv,rot,pairing,decay,S", [
    (2, 6, 10, 4, "half", (0.9, 0.5), 1), (1, 33, 5, 0, "half", (0.999,), 2), (3, 16, 8, 16, "half", (0.97, 1.0, 0.25), 3),
    (2, 24, 40, 24, "half", (0.9375, 0.998), 1), (1, 128, 96, 64, "interleaved", (0.98,), 1), (2, 2, 3, 2, "interleaved", (0.7, 0.8), 2),
    (1, 270, 40, 100, "half", (0.995,), 1)])
def test_retention_in_portions_equals_the_whole(H, d, dv, rot, pairing, decay, S):
    check_retention(H, d, dv, rot, pairing, decay, S, PORTION_STEPS)


@gpu
@pytest.mark.parametrize("H,d,dv,rot,pairing,decay,S", [(2, 128, 48, 128, "half", (0.99, 0.9), 1), (1, 270, 11, 8, "half", (0.97,), 1),
                                                        (3, 20, 66, 20, "interleaved", (0.5, 0.9, 0.99), 2)])
def test_retention_in_long_portions(H, d, dv, rot, pairing, decay, S):
    check_retention(H, d, dv, rot, pairing, decay, S, LONG_STEPS)


@gpu
def test_retention_decoding_token_by_token_and_in_bfloat16():
    check_retention(2, 64, 64, 64, "half", (0.99, 0.9), 2, DECODE_STEPS)
    check_retention(2, 16, 24, 8, "half", (0.95, 0.8), 1, PORTION_STEPS, dtype=torch.bfloat16)


# -------------------------------------------------------------------------- attention with a learned sink, alone


class _Group:
    def __init__(self, table):
        self.block_table = table


class _Ctx:
    """What paged_attention asks of a step, for entries laid out by hand."""

    def __init__(self, lens, ctxs, table):
        import vllm_cpp_b200.workspace  # noqa: F401
        self.device = dev()
        self.host_q_len, self.host_ctx_len = list(lens), list(ctxs)
        self.host_q_start = np.concatenate([[0], np.cumsum(lens)])[:-1].tolist()
        self.q_start, self.q_len, self.ctx_len = i32(self.host_q_start), i32(lens), i32(ctxs)
        self.slots = i32(list(range(len(lens))))
        self.status = torch.zeros(1, dtype=torch.int32, device=dev())
        self.groups = [_Group(table)]
        self.T, self.E = int(sum(lens)), len(lens)
        self._plans = {}

    def plan(self, key, make):
        if key not in self._plans:
            self._plans[key] = make()
        return self._plans[key]


class _Kv:
    group = 0

    def __init__(self, pages):
        self.pages = pages


def attention_by_hand(nh, nkv, hd, dtype, window, sink, ctxs, lens, make_hot=None, ps=16, seed=0):
    """Entries of ``lens`` new tokens whose contexts end at ``ctxs``: random keys and values laid into pages in a scrambled
    order, the attention of the new tokens' queries by the engine and by the plain implementation."""
    from vllm_cpp_b200.parts.window_attention import paged_attention
    g = torch.Generator().manual_seed(seed + nh * 7 + hd)
    E = len(lens)
    max_blocks = max(-(-c // ps) for c in ctxs)
    n_pages = E * max_blocks + 3
    order = torch.randperm(n_pages, generator=g).tolist()
    table = torch.zeros(E, max_blocks, dtype=torch.int32)
    pages = torch.full((n_pages, 2, nkv, ps, hd), float("nan"), dtype=F64)
    qs, wants = [], []
    scale = 0.3
    for e in range(E):
        n = ctxs[e]
        k = torch.randn(n, nkv, hd, generator=g, dtype=F64)
        v = torch.randn(n, nkv, hd, generator=g, dtype=F64)
        q = torch.randn(n, nh, hd, generator=g, dtype=F64)
        if make_hot is not None:
            make_hot(e, q, k, v)
        k, v, q = (t.to(dtype).double() for t in (k, v, q))       # what the cache and the query buffer hold
        for b in range(-(-n // ps)):
            page = order.pop()
            table[e, b] = page
            m = min(ps, n - b * ps)
            pages[page, 0, :, :m] = k[b * ps:b * ps + m].transpose(0, 1)
            pages[page, 1, :, :m] = v[b * ps:b * ps + m].transpose(0, 1)
        want = P.window_softmax_attention(q, k, v, scale, window, sink=sink)
        qs.append(q[n - lens[e]:])
        wants.append(want[n - lens[e]:])
    ctx = _Ctx(lens, ctxs, table.to(dev()))
    qbuf = torch.cat(qs).reshape(-1, nh * hd).to(dtype).to(dev())
    out = torch.full((ctx.T, nh * hd), float("nan"), dtype=dtype, device=dev())
    paged_attention(ctx, _Kv(pages.to(dtype).to(dev())), qbuf, out, nh=nh, nkv=nkv, hd=hd, vd=hd, scale=scale, window=window,
                    sink=f32(sink) if sink is not None else False)
    assert int(ctx.status.item()) == 0
    return out.double().cpu().view(-1, nh, hd), torch.cat(wants)


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(4, 2, 8, 9), (6, 3, 80, 50), (2, 1, 64, 33), (8, 4, 64, 0), (2, 2, 128, 40), (5, 1, 6, 1)])
def test_attention_with_a_learned_sink_on_a_mixed_batch(dtype, nh, nkv, hd, window):
    """First tokens, single tokens behind short and long contexts, portions that cross page borders and a window's edge."""
    sink = torch.linspace(-2.0, 3.0, nh, dtype=F64)
    lens = [1, 1, 1, 7, 40, 1, 130]
    ctxs = [1, 17, 700, 7, 95, 64, 200]
    got, want = attention_by_hand(nh, nkv, hd, dtype, window, sink, ctxs, lens)
    torch.testing.assert_close(got, want, **(dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else TOL16))


@gpu
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd", [16, 64])
def test_one_key_or_the_sink_decides_the_row(dtype, hd):
    """A key whose score stands out, placed just inside and just outside the window and far back among hundreds, in a
    prompt portion and behind a single token; and scores so low that the sink takes nearly all the weight."""
    W = 24
    sink = torch.tensor([0.5, -1.0], dtype=F64)
    for length, n_new in ((300, 1), (300, 60)):
        for back in (0, W - 1, W, 250):       # how far behind the last query the hot key lies
            def hot(e, q, k, v, back=back):
                n = q.shape[0]
                q[n - 1] *= 0.1
                k[n - 1 - back] = q[n - 1, :1].expand(k.shape[1], -1) * 400.0          # its score with the last query stands out
                v[n - 1 - back] = 5.0
            got, want = attention_by_hand(2, 2, hd, dtype, W, sink, [length], [n_new], make_hot=hot)
            torch.testing.assert_close(got, want, **(dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else TOL16))
            seen = back < W
            assert (abs(float(want[-1, 0, 0]) - 5.0) < 0.5) == seen, (back, want[-1, 0, 0])
            # without a window the far key is seen as well
            got, want = attention_by_hand(2, 2, hd, dtype, 0, sink, [length], [n_new], make_hot=hot)
            torch.testing.assert_close(got, want, **(dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else TOL16))
            assert abs(float(want[-1, 0, 0]) - 5.0) < 0.5

    def cold(e, q, k, v):
        q *= 0.0
        v += 3.0
    big = torch.tensor([12.0, 0.0], dtype=F64)
    got, want = attention_by_hand(2, 2, hd, dtype, 8, big, [50, 9], [1, 9], make_hot=cold)
    torch.testing.assert_close(got, want, **(dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else TOL16))
    assert float(want[0, 0].abs().max()) < 1e-3 and float(want[0, 1].abs().max()) > 1.0     # head 0 gives nearly all to its sink


# -------------------------------------------------------------------------- whole models through bin/trace_run


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
REPLAYS = ([(n, "float32", m) for n in "ABC" for m in MODES] + [(n, "bfloat16", m) for n in "ABC" for m in ("whole", "tail", "portions", "mixed")])


@gpu
@pytest.mark.parametrize("name,dtype,mode", REPLAYS)
def test_replay(name, dtype, mode, mefupel_dirs, oracle, tmp_path):
    """Whole prompts; the last 32 tokens one by one; portions of changing size down to two tokens; up to four live
    requests with pages and slots used again -- the last two also as serving asks (logits of an entry's last token
    only: captured steps), all over a NaN-filled cache."""
    requests = requests_of(name)
    trace = MODES[mode](requests)
    out = R.run_trace(mefupel_dirs[name], dtype, trace, tmp_path / "out", configs()[name][1], extra_args=["--poison"])
    worst = compare(name, dtype, trace, out, requests, oracle)
    print(f"{name} {dtype} {mode}: worst relative error {worst:.3e}, pool {trace.max_tokens} tokens, {len(trace.steps)} steps")


@gpu
def test_replay_modes_agree_with_each_other(mefupel_dirs, tmp_path):
    """Cutting and batching change the logits by rounding only."""
    for name in ("A", "B"):
        requests = requests_of(name)
        vocab = configs()[name][0].vocab
        rows = {}
        for mode in ("whole", "mixed", "portions"):
            trace = MODES[mode](requests)
            out = R.run_trace(mefupel_dirs[name], "float32", trace, tmp_path / (name + mode), configs()[name][1])
            for step, want in enumerate(trace.wanted):
                got = R.read_step(out, step, vocab)
                for i, key in enumerate(want):
                    rows.setdefault(key, {})[mode] = got[i]
        worst = max(np.abs(v["whole"] - v[m]).max() / np.abs(v["whole"]).max() for v in rows.values() for m in ("mixed", "portions"))
        assert worst < 2e-5, (name, worst)


@gpu
def test_long_decoding(mefupel_dirs, oracle, tmp_path):
    """A short prompt, then 250 tokens one by one: the states carried through 250 steps, every window passing over decoded
    tokens and pages' borders, pages given back as the windows pass."""
    for name in ("A", "B"):
        toks = random_tokens(configs()[name][0].vocab, 260, 99)
        trace = R.tail_one_by_one({"long": toks}, tail=250)
        out = R.run_trace(mefupel_dirs[name], "float32", trace, tmp_path / name, configs()[name][1], extra_args=["--poison"])
        compare(name, "float32", trace, out, {"long": toks}, oracle)


# -------------------------------------------------------------------------- generation through the engine's entry point


@gpu
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_scheduler(name, mefupel_dirs):
    """Several prompts at once through LLM.generate (scheduler, portions under a small token budget, captured decoding
    steps, device-side sampling at temperature 0) against the plain implementation's greedy continuation."""
    from vllm_cpp_b200 import LLM
    cfg, w = P.read_model(mefupel_dirs[name])
    vocab, page = configs()[name][0].vocab, configs()[name][1]
    prompts = [random_tokens(vocab, n, 3 + n) for n in (5, 41, 18, 70, 2)]
    llm = LLM(str(mefupel_dirs[name]), dtype="float32", page_size=page, max_tokens=page * 64, max_num_seqs=3, max_step_tokens=32,
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
