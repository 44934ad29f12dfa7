"""Python face of the CUDA kernels in ``csrc/kernels`` (loaded through ctypes).

Each function takes torch CUDA tensors, checks shapes and dtypes, and launches
on torch's current stream.  There is no CPU fallback and no library fallback:
if the kernel library cannot be built or loaded, importing a kernel raises.
"""
from __future__ import annotations

import ctypes
import functools
import math
import struct
from ctypes import c_float, c_int, c_longlong, c_void_p

import torch

from .csrc import build as _build

F32, BF16 = 0, 1
STATUS_BITS = {1: "token id outside the vocabulary", 2: "page id outside the pool",
               4: "a bounded wait inside a kernel gave up", 8: "position outside the rotary table",
               16: "shared memory did not start on the boundary a kernel's tiles need",
               32: "a work item names a partial-result row outside the buffer it was given"}
ITEM_INTS = 6

_lib = None


class KernelError(RuntimeError):
    pass


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return F32
    if t.dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"unsupported element type {t.dtype} (float32 or bfloat16)")


def lib():
    """The loaded kernel library; built on first use."""
    global _lib
    if _lib is None:
        path = _build.build_kernels()
        try:
            L = ctypes.CDLL(str(path))
        except OSError as e:
            raise KernelError(f"cannot load the CUDA kernel library {path}: {e}") from e
        L.vcb_last_error.restype = ctypes.c_char_p
        _declare(L)
        _lib = L
    return _lib


def _declare(L):
    P, I, LL, F = c_void_p, c_int, c_longlong, c_float
    sigs = {
        "vcb_embed_gather": [P, I, P, P, I, I, I, P, P],
        "vcb_add_rmsnorm": [P, P, I, I, LL, P, I, F, P, I, P, I, I, P],
        "vcb_swiglu": [P, I, I, LL, P, I, I, I, P],
        "vcb_qknorm_rope_kvwrite": [P, I, I, LL, I, P, P, I, I, F, P, I, P, P, P, P, LL, I, I, I, I, I, I, I, I, I, P, P],
        "vcb_gemm_bf16_tn": [P, P, P, I, I, I, I, LL, LL, LL, I, LL, P, P],
        "vcb_gemm_bf16_tn_shape": [P, P, P, I, I, I, I, LL, LL, LL, I, LL, I, I, P, P],
        "vcb_gemm_effective_splits": [I, I],
        "vcb_gemm_set_pairs": [I],
        "vcb_gemm_bf16_swiglu": [P, P, P, I, I, I, LL, LL, LL, I, I, P, P],
        "vcb_gemm_bf16_qkv": [P, P, I, I, LL, LL, P, P, LL, I, I, P, P, P, I, P, P, I, I, F, I, I, P, P],
        "vcb_sgemm_tn": [P, P, P, I, I, I, LL, LL, LL, P],
        "vcb_gemm_bf16_plain": [P, P, P, I, I, I, I, LL, LL, LL, P],
        "vcb_attn_paged": [P, P, I, P, LL, P, P, I, P, P, P, P, I, I, P, P, I, I, I, I, I, I, F, P, P],
        "vcb_attn_paged_ex": [P, P, I, P, LL, P, P, I, P, P, P, P, I, I, P, P, I, I, I, I, I, I, F, I, P, P, I, F, P, I, P, P, P],
        "vcb_embed_sinusoid": [P, I, P, P, P, P, I, I, I, P, P],
        "vcb_causal_conv": [P, I, LL, LL, P, P, P, LL, P, P, P, I, I, I, I, I, P, P, I, P, I, P],
        "vcb_embed_scaled_pos": [P, I, P, P, P, I, F, P, I, I, I, I, P, P],
        "vcb_postnorm_add_norm": [P, P, I, LL, LL, P, P, P, F, P, P, I, I, I, P, F, P, I, P, I, P],
        "vcb_qkv_wholenorm_store": [P, I, LL, LL, P, P, F, P, P, P, I, I, I, I, I, I, P, P, LL, I, I, I, P, P],
        "vcb_gated_act": [P, I, LL, LL, P, P, I, I, I, I, P],
        "vcb_softcap": [P, LL, F, P],
        "vcb_ssm_scan": [P, I, LL, LL, I, P, I, LL, P, P, P, P, LL, P, P, P, I, I, I, I, I, I, I, I, P, P, P, P],
        "vcb_gated_group_norm": [P, P, I, LL, LL, P, F, P, P, I, I, I, I, P, I, P],
        "vcb_moe_route": [P, I, LL, LL, P, P, I, I, I, I, I, P, P, P],
        "vcb_hyper_mix_norm": [P, P, P, I, LL, LL, P, P, P, P, F, P, I, P, I, I, I, I, P],
        "vcb_token_shift": [P, P, P, LL, P, P, P, I, I, I, P, I, P],
        "vcb_latent_norm_rope_store": [P, I, LL, LL, P, P, F, P, P, F, P, P, P, LL, I, I, I, I, I, I, I, I, P, P],
        "vcb_head_linear": [P, I, I, LL, LL, I, I, P, I, P, I, LL, I, I, I, I, I, I, P],
        "vcb_rope_rows": [P, I, LL, LL, I, I, P, P, F, P, I, LL, I, I, I, I, I, I, P],
        "vcb_matrix_rnn": [I, P, I, LL, LL, P, LL, I, I, I, I, I, P, P, P, P, P, LL, P, P, P, I, I, I, I, I, I, P,
                           P, I, LL, LL, F, P, P, P, I, I, P],
        "vcb_sum_add_rmsnorm": [P, I, P, P, P, P, P, P, P, F, P, I, P, I, I, P],
        "vcb_branch_norm_mean": [I, P, P, P, P, P, F, P, I, I, P],
        "vcb_polynorm": [P, I, LL, LL, P, F, P, I, I, I, P],
        "vcb_qkv_rope_store": [P, I, LL, LL, P, P, F, P, P, P, P, P, P, LL, I, I, I, I, I, I, I, I, I, I, I, I, P, P],
        "vcb_rotate_heads": [P, I, P, P, F, I, I, I, I, I, P],
        "vcb_head_norm_gate": [P, P, I, LL, LL, I, P, F, P, P, I, I, I, I, P, I, P],
        "vcb_moe_route_grouped": [P, I, LL, LL, P, I, I, F, P, P, I, I, I, I, P, P, P],
        "vcb_moe_group": [P, I, I, I, I, P, P, P, P],
        "vcb_moe_gather": [P, LL, I, P, P, I, I, I, P, P],
        "vcb_gemm_bf16_grouped": [P, P, P, I, I, I, I, I, I, LL, LL, LL, P, I, P, P],
        "vcb_moe_gemm": [P, LL, P, I, P, P, P, I, I, P, I, I, I, I, P],
        "vcb_moe_combine": [P, P, P, I, P, I, LL, LL, P, P, I, I, I, P, P],
        "vcb_conv_state_update": [P, I, LL, LL, P, P, LL, P, P, P, I, I, I, P],
        "vcb_qkv_conv_norm_store": [P, I, LL, LL, P, P, P, LL, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P, LL, I, I, I, I, P, P],
        "vcb_gated_norm_add": [P, P, I, LL, LL, P, I, LL, LL, P, P, F, P, P, I, I, I, P, I, P],
        "vcb_bias_act": [P, I, LL, LL, P, P, I, I, I, I, P],
        "vcb_scatter_i32": [P, P, P, P, I, LL, P],
        "vcb_selftest_wait_timeout": [LL, P, P, P],
        "vcb_state_reset": [P, I, LL, LL, LL, I, I, P, P, P, I, ctypes.c_uint, P, P],
        "vcb_attn_mma": [P, P, P, LL, P, P, I, P, P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, F, P, I, I, P],
        "vcb_attn_mma_ex": [P, P, P, LL, P, P, I, P, P, P, P, I, I, P, P, P, P, I, I, I, I, I, I, F, I, P, P, F, P, I, P, P, I, I, P],
        "vcb_attn_mma_supported": [I, I],
        "vcb_attn_mma_max_clusters": [I, I, I],
        "vcb_attn_mma_fused_supported": [I, I, I],
        "vcb_attn_mma_decode_fused": [P, I, LL, P, P, I, I, F, P, I, P, P, P, LL, P, P, I, P, P, P, P, I, P, P, P, P, I, I,
                                      I, I, I, I, F, P, I, P],
        "vcb_attn_tc": [P, P, P, LL, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, P, P, P],
        "vcb_attn_tc_ex": [P, P, P, LL, P, P, I, P, P, P, P, I, I, I, I, I, I, I, F, I, P, P, F, P, I, P, P, P, P],
        "vcb_attn_tc_supported": [I, I, I],
        "vcb_attn_stream": [P, P, P, LL, P, P, I, P, P, P, I, P, I, I, I, I, I, I, F, P, I, P],
        "vcb_attn_stream_supported": [I, I, I, I, I],
        "vcb_attn_merge": [P, P, P, P, I, I, I, I, I, P],
        "vcb_sample": [P, LL, I, I, P, P, P, P],
        "vcb_sample_split": [P, LL, I, I, P, P, P, P, I, P, P],
        "vcb_count_tokens": [P, P, P, I, I, I, P],
    }
    for name, args in sigs.items():
        fn = getattr(L, name)
        fn.argtypes = args
        fn.restype = c_int


_num_sms = None


def num_sms() -> int:
    """Streaming multiprocessors of the current device, asked once (148 on a B200); where there is no device
    -- the host-side tests of the planning arithmetic -- the B200's count."""
    global _num_sms
    if _num_sms is None:
        _num_sms = torch.cuda.get_device_properties(torch.cuda.current_device()).multi_processor_count \
            if torch.cuda.is_available() else 148
    return _num_sms


launch_count = 0   # kernels of this library launched so far (every launcher starts exactly one)


def _call(name: str, *args):
    global launch_count
    L = lib()
    launch_count += 1
    fn = getattr(L, name)
    # ctypes takes arguments beyond the declared ones without a word and passes them as 32-bit integers: a pointer or
    # a stream handle would lose its upper half
    if fn.argtypes is None or len(fn.argtypes) != len(args):
        raise KernelError(f"{name}: {len(args)} arguments for a declaration of {0 if fn.argtypes is None else len(fn.argtypes)}")
    rc = fn(*args)
    if rc != 0:
        raise KernelError(L.vcb_last_error().decode() or f"{name} failed with code {rc}")


_held_stream: int | None = None   # the stream handle for the launches inside hold_stream(), asked for once


def _stream() -> int:
    return _held_stream if _held_stream is not None else torch.cuda.current_stream().cuda_stream


class hold_stream:
    """Within this context every launch goes to the stream that is current on entry, without asking torch for it
    again (three microseconds a launch, a quarter of a launch's host time).  Not to be held across a change of
    the current stream: a graph capture, for one, must start outside it."""

    def __enter__(self):
        global _held_stream
        self._outer = _held_stream
        _held_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _held_stream
        _held_stream = self._outer
        return False


def _p(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _need(t: torch.Tensor, name: str, dtype=None, contiguous=True):
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor (there is no CPU path)")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, found {t.dtype}")
    if contiguous and not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")


def check_status(status: torch.Tensor, where: str = "step") -> None:
    """Reads the device status word (a synchronising copy) and raises on any set bit."""
    v = int(status.item())
    if v:
        status.zero_()
        what = [msg for bit, msg in STATUS_BITS.items() if v & bit]
        raise KernelError(f"{where}: a kernel reported: " + "; ".join(what))


# --------------------------------------------------------------------------


def embed_gather(table, ids, out, status):
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    T, H = out.shape
    V = table.shape[0]
    assert table.shape[1] == H and ids.numel() >= T
    _call("vcb_embed_gather", _p(table), _dt(table), _p(ids), _p(out), T, H, V, _p(status), _stream())


def add_rmsnorm(resid, delta, weight, eps, out, rows=None):
    """resid [T,H] f32 (updated in place with the deltas unless ``rows`` is given);
    delta None, [T,H] or [S,T,H]; out [n,H] in the activation dtype."""
    _need(resid, "resid", torch.float32); _need(weight, "weight"); _need(out, "out")
    T, H = resid.shape
    S, stride, dptr, ddt = 0, 0, None, F32
    if delta is not None:
        _need(delta, "delta")
        if delta.dim() == 2:
            delta = delta.unsqueeze(0)
        S = delta.shape[0]
        assert delta.shape[1] >= T and delta.shape[2] == H, (delta.shape, resid.shape)
        stride, dptr, ddt = delta.stride(0), delta.data_ptr(), _dt(delta)
    n = T if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    assert out.shape[0] >= n and out.shape[1] == H and weight.numel() == H
    _call("vcb_add_rmsnorm", _p(resid), dptr, ddt, S, stride, _p(weight), _dt(weight), float(eps), _p(out), _dt(out),
          _p(rows), n, H, _stream())


def _partials(t: torch.Tensor, name: str):
    """[T, W] or [S, T, W] (S partial sums to be added) -> (S, stride between partials)."""
    _need(t, name)
    if t.dim() == 2:
        return 1, 0
    return t.shape[0], t.stride(0)


def swiglu(gate_up, out):
    """out[t, i] = silu(gate_up[t, 2i]) * gate_up[t, 2i+1]: gate and up alternate along a row.
    gate_up [T, 2I] or [S, T, 2I] (32-bit partial sums); out [T, I]."""
    S, stride = _partials(gate_up, "gate_up"); _need(out, "out")
    T, I2 = gate_up.shape[-2:]
    assert out.shape == (T, I2 // 2)
    _call("vcb_swiglu", _p(gate_up), _dt(gate_up), S, stride, _p(out), _dt(out), T, I2 // 2, _stream())


def qknorm_rope_kvwrite(qkv, q_weight, k_weight, eps, cos_sin, positions, slot_map, q_out, pages, nh, nkv, hd,
                        status, has_kv=True, use_norm=True, rotary_dim=None, interleaved=False):
    """qkv [T, W] or [S, T, W] (32-bit partial sums); pages: one layer's [num_pages, 2, nkv, page_size, hd];
    slot_map int32 [T] = page * page_size + offset or -1.  ``rotary_dim`` (default: hd) lanes of a head are
    rotated, paired (i, i + rotary_dim/2) or, with ``interleaved``, (2i, 2i+1); cos_sin is [positions, rotary_dim]."""
    rotary_dim = hd if rotary_dim is None else int(rotary_dim)
    S, stride = _partials(qkv, "qkv")
    _need(cos_sin, "cos_sin", torch.float32); _need(positions, "positions", torch.int32); _need(q_out, "q_out")
    T = qkv.shape[-2]
    width = (nh + (2 * nkv if has_kv else 0)) * hd
    assert qkv.shape[-1] == width, (qkv.shape, width)
    if cos_sin.shape[1] != rotary_dim:
        raise KernelError(f"the table of angles has {cos_sin.shape[1]} columns, {rotary_dim} lanes are to be rotated")
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight"); wdt = _dt(q_weight)
        if has_kv:
            _need(k_weight, "k_norm weight", q_weight.dtype)
    page_stride = page_size = num_pages = 0
    if has_kv:
        _need(pages, "pages", q_out.dtype); _need(slot_map, "slot_map", torch.int32)
        num_pages, two, nkv_p, page_size, hd_p = pages.shape
        assert two == 2 and nkv_p == nkv and hd_p == hd
        page_stride = pages.stride(0)
    _call("vcb_qknorm_rope_kvwrite", _p(qkv), _dt(qkv), S, stride, _dt(q_out), _p(q_weight), _p(k_weight), wdt,
          int(use_norm), float(eps), _p(cos_sin), cos_sin.shape[0], _p(positions), _p(slot_map), _p(q_out), _p(pages),
          page_stride, max(page_size, 1), num_pages, nh, nkv, hd, T, int(has_kv), rotary_dim, int(bool(interleaved)),
          _p(status), _stream())


def gemm_bf16_plain(x, w, out):
    """out[T,N] = x[T,K] . w[N,K]^T for bfloat16 operands of any inner size (no TMA alignment needed)."""
    _need(x, "x", torch.bfloat16, contiguous=False); _need(w, "w", torch.bfloat16, contiguous=False); _need(out, "out")
    T, K = x.shape
    N = w.shape[0]
    assert w.shape[1] == K and out.shape == (T, N) and x.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    _call("vcb_gemm_bf16_plain", _p(x), _p(w), _p(out), _dt(out), T, N, K, x.stride(0), w.stride(0), out.stride(0), _stream())


def gemm_tma_ok(x, w) -> bool:
    """Whether the tcgen05/TMA product can address these operands (16-byte rows and bases)."""
    K = x.shape[1]
    return (K % 8 == 0 and x.stride(0) % 8 == 0 and w.stride(0) % 8 == 0 and x.data_ptr() % 16 == 0
            and w.data_ptr() % 16 == 0)


def gemm_effective_splits(K: int, splits: int) -> int:
    """The number of k-slices the kernel makes of ``splits`` asked for: whole 64-wide k-blocks, none empty
    (the arithmetic of vcb_gemm_effective_splits, here without a call into the library)."""
    total_kb = -(-K // 64)
    splits = max(1, min(int(splits), total_kb))
    per = -(-total_kb // splits)
    return -(-total_kb // per)


GEMM_SHAPES = ("n16", "n32", "n64", "n128", "n256", "m256_n192", "m256_n256", "pair", "m256_n160")   # unit shapes of the kernel, by index


def gemm_set_pairs(mode: int) -> None:
    """Which products of more than 128 tokens without k-slices run on pairs of blocks (``cta_group::2``: one MMA
    spans 256 features on two SMs, each block loads its half of the token tile): 0 none, 1 those whose units fill
    the pairs' rounds no worse than the single-block kernel's fill the SMs' (the default, which
    ``VLLM_CPP_B200_GEMM_PAIRS`` overrides), 2 all that can.  Process-wide."""
    lib().vcb_gemm_set_pairs(int(mode))


def gemm_bf16_tn(w, x, out, splits, status, shape=-1, after_small_kernel=False):
    """out[z, t, m] = sum over k-slice z of w[m, k] x[t, k]   (tcgen05 + TMA; w [M,K], x [T,K] bfloat16).
    out: [T, M] (bfloat16 or float32, one slice) or [S, T, M] float32 with S = gemm_effective_splits(K, splits).
    ``shape`` forces one of GEMM_SHAPES (an index) whatever the sizes; -1 lets the kernel choose.
    ``after_small_kernel``: the kernel before this one in the stream is a short one (a norm, the SiLU-gate): a decode
    product then asks further weight tiles into L2 while it waits for it (VLLM_CPP_B200_GEMM_PREFETCH)."""
    _need(w, "w", torch.bfloat16, contiguous=False); _need(x, "x", torch.bfloat16, contiguous=False); _need(out, "out")
    M, K = w.shape
    T = x.shape[0]
    assert x.shape[1] == K and w.stride(1) == 1 and x.stride(1) == 1
    S = gemm_effective_splits(K, splits)
    if out.dim() == 2:
        assert S == 1 and out.shape == (T, M)
        ldc, sstride = out.stride(0), 0
    else:
        assert out.shape == (S, T, M) and out.dtype == torch.float32
        ldc, sstride = out.stride(1), out.stride(0)
    _call("vcb_gemm_bf16_tn_shape", _p(w), _p(x), _p(out), _dt(out), M, T, K, w.stride(0), x.stride(0), ldc, S, sstride,
          int(shape), int(bool(after_small_kernel)), _p(status), _stream())


def gemm_bf16_swiglu(w_gate_up, x, out, status, shape=-1, after_small_kernel=False):
    """out[t, i] = silu(gate_i . x_t) * (up_i . x_t) with gate_i in row 2i and up_i in row 2i+1 of w_gate_up: the
    product and the SiLU-gate in one kernel (adjacent accumulator lanes are paired in the epilogue).
    ``shape`` and ``after_small_kernel`` as in gemm_bf16_tn."""
    _need(w_gate_up, "w_gate_up", torch.bfloat16); _need(x, "x", torch.bfloat16, contiguous=False)
    _need(out, "out", torch.bfloat16)
    I2, K = w_gate_up.shape
    T = x.shape[0]
    assert I2 % 2 == 0 and x.shape[1] == K and x.stride(1) == 1 and out.shape == (T, I2 // 2)
    _call("vcb_gemm_bf16_swiglu", _p(w_gate_up), _p(x), _p(out), I2 // 2, T, K, w_gate_up.stride(0), x.stride(0),
          out.stride(0), int(shape), int(bool(after_small_kernel)), _p(status), _stream())


def gemm_qkv_rope(w_qkv, x, q_out, pages, slot_map, positions, cos_sin, q_weight, k_weight, eps, nh, nkv, status,
                  use_norm=True):
    """The stacked q, k, v projection of a prompt portion with what :func:`qknorm_rope_kvwrite` does in its epilogue
    (head_dim 128, the whole head rotated in half-split pairs): per-head norm of queries and keys, rotation, queries to
    ``q_out`` [T, nh * 128], keys and values to the tokens' slots of ``pages`` (None: a layer that stores none; then
    ``w_qkv`` holds the query rows only).  No k-slices, so for more than 128 tokens; 32-bit from the product's sums on."""
    _need(w_qkv, "w_qkv", torch.bfloat16); _need(x, "x", torch.bfloat16, contiguous=False); _need(q_out, "q_out", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32); _need(positions, "positions", torch.int32)
    M, K = w_qkv.shape
    T = x.shape[0]
    assert x.shape[1] == K and x.stride(1) == 1 and q_out.shape == (T, nh * 128) and cos_sin.shape[1] == 128
    page_stride = page_size = num_pages = 0
    if pages is not None:
        _need(pages, "pages", torch.bfloat16); _need(slot_map, "slot_map", torch.int32)
        num_pages, two, nkv_p, page_size, hd_p = pages.shape
        assert two == 2 and nkv_p == nkv and hd_p == 128 and M == (nh + 2 * nkv) * 128
        page_stride = pages.stride(0)
    else:
        assert M == nh * 128
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight")
        wdt = _dt(q_weight)
        if pages is not None:
            _need(k_weight, "k_norm weight", q_weight.dtype)
    _call("vcb_gemm_bf16_qkv", _p(w_qkv), _p(x), T, K, w_qkv.stride(0), x.stride(0), _p(q_out), _p(pages), page_stride,
          page_size, num_pages, _p(slot_map), _p(positions), _p(cos_sin), cos_sin.shape[0], _p(q_weight), _p(k_weight), wdt,
          int(use_norm), float(eps), nh, nkv, _p(status), _stream())


def sgemm_tn(a, b, out):
    """out[M,N] = a[M,K] . b[N,K]^T in true 32-bit."""
    _need(a, "a", torch.float32, contiguous=False); _need(b, "b", torch.float32, contiguous=False)
    _need(out, "out", torch.float32, contiguous=False)
    M, K = a.shape
    N = b.shape[0]
    assert b.shape[1] == K and out.shape == (M, N)
    assert a.stride(1) == 1 and b.stride(1) == 1 and out.stride(1) == 1
    _call("vcb_sgemm_tn", _p(a), _p(b), _p(out), M, N, K, a.stride(0), b.stride(0), out.stride(0), _stream())


def attn_paged(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, rows_max, part_o, part_ml,
               nh, nkv, hd, window, status, table_row=None):
    """block_table int32 [rows, max_blocks]; entry e reads row ``table_row[e]`` (row e when table_row is None)."""
    _need(q, "q"); _need(out, "out", q.dtype); _need(pages, "pages", q.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_paged", _p(q), _p(out), _dt(q), _p(pages), pages.stride(0), _p(block_table), _p(table_row), block_table.shape[1],
          _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, rows_max, _p(part_o), _p(part_ml), nh, nkv, hd,
          page_size, num_pages, int(window or 0), 1.0 / math.sqrt(hd), _p(status), _stream())


def _sink_scores(sink, nh):
    """``sink`` as the attention wrappers take it (False, True, or a float32 tensor [nh] of scores) -> the tensor or None."""
    if not torch.is_tensor(sink):
        return None
    _need(sink, "sink", torch.float32)
    assert sink.numel() == nh
    return sink


def kv_page_views(pages, nkv, hd, hd_v):
    """(page_size, num_pages) of one cache's pages, laid out either [pages, 2, nkv, page_size, hd] or, where values
    have another head size than keys, [pages, nkv * page_size * (hd + hd_v)]: keys first, then values."""
    if pages.dim() == 5:
        num_pages, two, nkv_p, page_size, hd_p = pages.shape
        assert two == 2 and nkv_p == nkv and hd_p == hd == hd_v, (pages.shape, nkv, hd, hd_v)
        return page_size, num_pages
    assert pages.dim() == 2 and pages.shape[1] % (nkv * (hd + hd_v)) == 0, (pages.shape, nkv, hd, hd_v)
    return pages.shape[1] // (nkv * (hd + hd_v)), pages.shape[0]


def attn_window_bias(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, rows_max, part_o, part_ml,
                     nh, nkv, hd, window, status, table_row=None, *, scale, keep_first=0, dist_a=None, dist_b=None, hd_v=None,
                     softcap=0.0, slope=None, sink=False):
    """:func:`attn_paged` with its options: scores scaled by ``scale``; with a window, the first ``keep_first`` keys of
    a request stay visible; ``dist_a``/``dist_b`` (float32 [nh]): a_h ln(1 + b_h (pos - j)) is taken off key j's
    score; values of head size ``hd_v`` (``pages`` then [num_pages, nkv * page_size * (hd + hd_v)]); ``softcap`` c > 0:
    the scaled score becomes c tanh(s / c); ``slope`` (float32 [nh]): slope_h (pos - j) is taken off after the cap;
    ``sink``: a silent key of score 0 and no value takes part in every softmax; given as a float32 tensor [nh], the
    silent key's score per head (not scaled)."""
    hd_v = hd if hd_v is None else int(hd_v)
    sink_value = sink if torch.is_tensor(sink) else None
    if sink_value is not None:
        _need(sink_value, "sink", torch.float32); assert sink_value.numel() == nh
    _need(q, "q"); _need(out, "out", q.dtype); _need(pages, "pages", q.dtype)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    page_size, num_pages = kv_page_views(pages, nkv, hd, hd_v)
    if dist_a is not None:
        _need(dist_a, "dist_a", torch.float32); _need(dist_b, "dist_b", torch.float32)
        assert dist_a.numel() == nh and dist_b.numel() == nh
    if slope is not None:
        _need(slope, "slope", torch.float32)
        assert slope.numel() == nh
    _call("vcb_attn_paged_ex", _p(q), _p(out), _dt(q), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, rows_max, _p(part_o), _p(part_ml),
          nh, nkv, hd, page_size, num_pages, int(window or 0), float(scale), int(keep_first or 0), _p(dist_a), _p(dist_b),
          hd_v, float(softcap or 0.0), _p(slope), int(sink_value is not None or bool(sink)), _p(sink_value), _p(status), _stream())


def embed_sinusoid(table, ids, positions, inv_freq, out, status):
    """out[t] = table[ids[t]] + s(positions[t]) with s(p)[2i] = sin(p * inv_freq[i]), s(p)[2i+1] = cos(p * inv_freq[i])."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(positions, "positions", torch.int32)
    _need(inv_freq, "inv_freq", torch.float32); _need(out, "out", torch.float32)
    T, H = out.shape
    assert table.shape[1] == H and ids.numel() >= T and positions.numel() >= T and inv_freq.numel() >= (H + 1) // 2
    _call("vcb_embed_sinusoid", _p(table), _dt(table), _p(ids), _p(positions), _p(inv_freq), _p(out), T, H, table.shape[0],
          _p(status), _stream())


def _rows_in(t: torch.Tensor, name: str):
    """A 32-bit [T, C] or [S, T, C] operand (rows may be strided) -> (S, stride between partial sums, row stride)."""
    _need(t, name, torch.float32, contiguous=False)
    assert t.stride(-1) == 1
    if t.dim() == 2:
        return 1, 0, t.stride(0)
    return t.shape[0], t.stride(0), t.stride(1)


def causal_conv(x, weight, state, q_start, q_len, slots, n_entries, out_conv=None, out_copy=None, bias=None,
                add_input=False, out_bias=None, act=None):
    """Per channel, over the tokens of each entry: out_conv[t] = sum_j weight[:, j] x[t - taps + 1 + j] (+ x[t] with
    ``add_input``), the taps - 1 inputs before an entry's first row read from ``state`` [slots, taps - 1, C] (32-bit)
    at the entry's slot; out_copy[t] = x[t].  x: 32-bit [T, C] or [S, T, C] partial sums, ``bias`` [C] added.
    ``weight`` None: no convolution.  Rows outside every entry are left alone.  The state row of an entry that brought
    one token is brought up to date as well; entries of more tokens need :func:`conv_state_update` afterwards.
    ``out_bias`` [C] is added to the convolution's result, then ``act`` ("silu" or None) is applied to it."""
    S, ss, ld = _rows_in(x, "x")
    T, C = x.shape[-2:]
    if out_bias is not None:
        _need(out_bias, "out_bias", torch.float32); assert out_bias.numel() == C
    if act not in (None, "silu"):
        raise KernelError(f"causal_conv: activation '{act}' (None or 'silu')")
    taps = 0 if weight is None else weight.shape[1]
    if weight is not None:
        _need(weight, "weight", torch.float32); assert weight.shape[0] == C
    if taps > 1:
        _need(state, "state", torch.float32); assert state.shape[1:] == (taps - 1, C), (state.shape, taps, C)
    dt = None
    for o in (out_conv, out_copy):
        if o is not None:
            _need(o, "out"); assert o.shape == (T, C); dt = _dt(o)
    assert dt is not None
    _call("vcb_causal_conv", _p(x), S, ss, ld, _p(bias), _p(weight), _p(state) if taps > 1 else None,
          state.stride(0) if taps > 1 else 0, _p(q_start), _p(q_len), _p(slots), n_entries, T, C, taps, int(bool(add_input)),
          _p(out_conv), _p(out_copy), dt, _p(out_bias), 1 if act == "silu" else 0, _stream())


def conv_state_update(x, state, q_start, q_len, slots, n_entries, bias=None):
    """After :func:`causal_conv` (or :func:`qkv_conv_norm_store`): the state row of each entry of two tokens or more
    holds the last taps - 1 inputs its request has seen (older ones move up where the entry brought fewer).  Entries of
    one token were brought up to date by the convolving kernel."""
    S, ss, ld = _rows_in(x, "x")
    C = x.shape[-1]
    _need(state, "state", torch.float32)
    taps = state.shape[1] + 1
    assert state.shape[2] == C
    _call("vcb_conv_state_update", _p(x), S, ss, ld, _p(bias), _p(state), state.stride(0), _p(q_start), _p(q_len), _p(slots),
          n_entries, C, taps, _stream())


def qkv_conv_norm_store(qkv, bias, weight, state, q_start, q_len, slots, slot_map, n_entries, q_out, pages, nh, nkv, hd,
                        hd_v, eps, status, use_norm=True, has_kv=True):
    """The stacked q, k, v projection ``qkv`` (32-bit [T, C] or [S, T, C], C = nh hd + nkv (hd + hd_v)) with ``bias``
    [C]; a causal convolution per channel (``weight`` [C, taps] or None) whose earlier inputs come from ``state``;
    every query and key head divided by its root mean square (``eps`` inside the root); queries to ``q_out``
    [T, nh hd], keys and values to the tokens' slots of ``pages`` (see :func:`kv_page_views`).  ``state`` as in
    :func:`causal_conv`."""
    S, ss, ld = _rows_in(qkv, "qkv")
    T, C = qkv.shape[-2:]
    assert C == nh * hd + (nkv * (hd + hd_v) if has_kv else 0), (C, nh, nkv, hd, hd_v)
    taps = 0 if weight is None else weight.shape[1]
    if weight is not None:
        _need(weight, "weight", torch.float32); assert weight.shape[0] == C
    if taps > 1:
        _need(state, "state", torch.float32); assert state.shape[1:] == (taps - 1, C)
    _need(q_out, "q_out"); assert q_out.shape == (T, nh * hd)
    page_size = num_pages = page_stride = 0
    if has_kv:
        _need(pages, "pages", q_out.dtype); _need(slot_map, "slot_map", torch.int32)
        page_size, num_pages = kv_page_views(pages, nkv, hd, hd_v)
        page_stride = pages.stride(0)
    _call("vcb_qkv_conv_norm_store", _p(qkv), S, ss, ld, _p(bias), _p(weight), _p(state) if taps > 1 else None,
          state.stride(0) if taps > 1 else 0, _p(q_start), _p(q_len), _p(slots), _p(slot_map), n_entries, T, taps, nh, nkv, hd,
          hd_v, int(bool(use_norm)), float(eps), _p(q_out), _p(pages) if has_kv else None, page_stride, max(page_size, 1),
          num_pages, int(bool(has_kv)), _dt(q_out), _p(status), _stream())


def gated_norm_add(resid, y, gate, gate_bias, weight, eps, q_start, q_len, n_entries, out_cast=None):
    """resid[t] += weight * n(y[t] * sigmoid(gate[t] + gate_bias)), n(v) = v / sqrt(mean(v^2) + eps); ``gate`` None: no
    gate.  y, gate: 32-bit [T, H] or [S, T, H] partial sums (rows may be strided).  ``out_cast``: the new rows once more."""
    _need(resid, "resid", torch.float32); _need(weight, "weight", torch.float32)
    T, H = resid.shape
    Sy, ssy, ldy = _rows_in(y, "y")
    assert y.shape[-1] == H and y.shape[-2] >= T
    Sg = ssg = ldg = 0
    if gate is not None:
        Sg, ssg, ldg = _rows_in(gate, "gate")
        assert gate.shape[-1] == H and gate.shape[-2] >= T
        if gate_bias is not None:
            _need(gate_bias, "gate_bias", torch.float32)
    if out_cast is not None:
        _need(out_cast, "out_cast"); assert out_cast.shape == (T, H)
    _call("vcb_gated_norm_add", _p(resid), _p(y), Sy, ssy, ldy, _p(gate), Sg, ssg, ldg, _p(gate_bias) if gate is not None else None,
          _p(weight), float(eps), _p(q_start), _p(q_len), n_entries, T, H, _p(out_cast), _dt(out_cast) if out_cast is not None else F32,
          _stream())


ACTIVATIONS = {"gelu": 0, "gelu_erf": 0, "gelu_tanh": 1, "silu": 2, "relu2": 3}
ELEMENTWISE = dict(ACTIVATIONS, identity=4)    # what bias_act takes: the activations, and the sums as they are


def bias_act(x, out, kind: str, bias=None):
    """out = act(x + bias): x 32-bit [T, C] or [S, T, C] partial sums; ``kind`` one of ACTIVATIONS, or "identity" (the
    sums themselves, added up and in ``out``'s type)."""
    S, ss, ld = _rows_in(x, "x")
    T, C = x.shape[-2:]
    _need(out, "out"); assert out.shape == (T, C)
    if kind not in ELEMENTWISE:
        raise KernelError(f"activation '{kind}' is not one of {sorted(ELEMENTWISE)}")
    _call("vcb_bias_act", _p(x), S, ss, ld, _p(bias), _p(out), _dt(out), T, C, ELEMENTWISE[kind], _stream())


def embed_scaled_pos(table, ids, positions, pos_table, scale, out, status):
    """out[t] = scale * table[ids[t]] + pos_table[positions[t]] (32-bit); ``pos_table`` None: the scaled row alone."""
    _need(table, "table"); _need(ids, "ids", torch.int32); _need(out, "out", torch.float32)
    T, H = out.shape
    assert table.shape[1] == H and ids.numel() >= T
    P = 0
    if pos_table is not None:
        _need(pos_table, "pos_table"); _need(positions, "positions", torch.int32)
        assert pos_table.shape[1] == H and positions.numel() >= T
        P = pos_table.shape[0]
    _call("vcb_embed_scaled_pos", _p(table), _dt(table), _p(ids), _p(positions) if pos_table is not None else None,
          _p(pos_table), _dt(pos_table) if pos_table is not None else F32, float(scale),
          _p(out), T, H, table.shape[0], P, _p(status), _stream())


def postnorm_add_norm(resid, y, post_weight, eps, q_start, q_len, n_entries, *, y_bias=None, layer_scale=None,
                      next_weight=None, next_eps=None, out=None, rows=None):
    """resid[t] += layer_scale * post_weight * n(y[t] + y_bias), n(v) = v / sqrt(mean(v^2) + eps), for the rows of the
    step's entries; then out[t] = next_weight * n'(resid[t]) with ``next_eps`` inside its root.  y: 32-bit [T, H] or
    [S, T, H] partial sums, or None (nothing is added: a plain norm).  ``rows`` (int32): only those rows, the stream is
    left as it is and ``out`` is [len(rows), H]."""
    _need(resid, "resid", torch.float32)
    T, H = resid.shape
    Sy = ssy = ldy = 0
    if y is not None:
        Sy, ssy, ldy = _rows_in(y, "y")
        assert y.shape[-1] == H and y.shape[-2] >= T
        _need(post_weight, "post_weight", torch.float32)
    for name, t in (("y_bias", y_bias), ("layer_scale", layer_scale), ("next_weight", next_weight)):
        if t is not None:
            _need(t, name, torch.float32); assert t.numel() == H
    n = T
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = rows.numel()
    if out is not None:
        _need(out, "out"); assert out.shape == (n, H) and next_weight is not None
    _call("vcb_postnorm_add_norm", _p(resid), _p(y), Sy, ssy, ldy, _p(y_bias) if y is not None else None, _p(post_weight),
          _p(layer_scale), float(eps), _p(q_start), _p(q_len), n_entries, T, H, _p(next_weight),
          float(eps if next_eps is None else next_eps), _p(out), _dt(out) if out is not None else F32, _p(rows), n, _stream())


def qkv_wholenorm_store(qkv, q_weight, k_weight, eps, q_start, q_len, slot_map, n_entries, q_out, pages, nh, nkv, hd, hd_v,
                        status):
    """The stacked q, k, v projection ``qkv`` (32-bit [T, C] or [S, T, C], C = nh hd + nkv (hd + hd_v)): all of a token's
    query lanes divided by their common root mean square and multiplied by ``q_weight`` [nh hd], its key lanes likewise
    with ``k_weight`` [nkv hd] (both None: no norm); queries to ``q_out``, keys and values to the tokens' slots of
    ``pages`` (see :func:`kv_page_views`)."""
    S, ss, ld = _rows_in(qkv, "qkv")
    T, C = qkv.shape[-2:]
    assert C == nh * hd + nkv * (hd + hd_v), (C, nh, nkv, hd, hd_v)
    if q_weight is not None:
        _need(q_weight, "q_weight", torch.float32); _need(k_weight, "k_weight", torch.float32)
        assert q_weight.numel() == nh * hd and k_weight.numel() == nkv * hd
    _need(q_out, "q_out"); assert q_out.shape == (T, nh * hd)
    _need(pages, "pages", q_out.dtype); _need(slot_map, "slot_map", torch.int32)
    page_size, num_pages = kv_page_views(pages, nkv, hd, hd_v)
    _call("vcb_qkv_wholenorm_store", _p(qkv), S, ss, ld, _p(q_weight), _p(k_weight), float(eps), _p(q_start), _p(q_len),
          _p(slot_map), n_entries, T, nh, nkv, hd, hd_v, _p(q_out), _p(pages), pages.stride(0), page_size, num_pages,
          _dt(q_out), _p(status), _stream())


def gated_act(x, out, kind: str, bias=None):
    """out[t, i] = act(x[t, i] + bias[i]) * (x[t, I + i] + bias[I + i]): x 32-bit [T, 2 I] or [S, T, 2 I] partial sums,
    the gate's columns first; ``kind`` one of ACTIVATIONS."""
    S, ss, ld = _rows_in(x, "x")
    T, I2 = x.shape[-2:]
    _need(out, "out"); assert out.shape == (T, I2 // 2) and I2 % 2 == 0
    if kind not in ACTIVATIONS:
        raise KernelError(f"activation '{kind}' is not one of {sorted(ACTIVATIONS)}")
    if bias is not None:
        _need(bias, "bias", torch.float32); assert bias.numel() == I2
    _call("vcb_gated_act", _p(x), S, ss, ld, _p(bias), _p(out), _dt(out), T, I2 // 2, ACTIVATIONS[kind], _stream())


def softcap(z, cap):
    """z <- cap * tanh(z / cap), in place (32-bit)."""
    _need(z, "z", torch.float32)
    _call("vcb_softcap", _p(z), z.numel(), float(cap), _stream())


SSM_STAGE = 16     # tokens the recurrence stages at a time; a chunk is a multiple of it


def ssm_scan(u, dt_col, xbc, dt_bias, rate, skip, state, q_start, q_len, slots, n_entries, heads, P, N, groups, y, *,
             chunk, n_chunks, scratch=None, chunk_decay=None):
    """S <- exp(-rate_h dt) S + dt B x^T, y = S^T C + skip_h x per head over the step's entries, the state carried in
    ``state`` [slots, heads, P, N] (32-bit).  ``u``: 32-bit sums [T, C] or [S, T, C] whose column ``dt_col + h`` is head
    h's raw dt (softplus(dt + dt_bias_h) is taken here); ``xbc`` [T, heads P + 2 groups N]: x, then B, then C, in the
    compute dtype; ``y`` [T, heads P] 32-bit.  Entries are cut into chunks of ``chunk`` tokens; ``n_chunks`` bounds their
    number over the step; with ``scratch`` [n_chunks, heads, P, N] and ``chunk_decay`` [n_chunks, heads] entries of more
    than one chunk run their chunks side by side (without them every entry must fit one chunk)."""
    S, ss, ld = _rows_in(u, "u")
    _need(xbc, "xbc", contiguous=False); _need(state, "state", torch.float32); _need(y, "y", torch.float32)
    for name, t in (("dt_bias", dt_bias), ("rate", rate), ("skip", skip)):
        _need(t, name, torch.float32); assert t.numel() == heads
    T = u.shape[-2]
    assert xbc.stride(1) == 1 and xbc.shape == (T, heads * P + 2 * groups * N) and y.shape == (T, heads * P)
    assert state.shape[1:] == (heads, P, N) and chunk % SSM_STAGE == 0
    multi = scratch is not None
    if multi:
        _need(scratch, "scratch", torch.float32); _need(chunk_decay, "chunk_decay", torch.float32)
        assert scratch.numel() >= n_chunks * heads * P * N and chunk_decay.numel() >= n_chunks * heads
    global launch_count
    _call("vcb_ssm_scan", _p(u), S, ss, ld, int(dt_col), _p(xbc), _dt(xbc), xbc.stride(0), _p(dt_bias), _p(rate), _p(skip),
          _p(state), state.stride(0), _p(q_start), _p(q_len), _p(slots), n_entries, heads, P, N, groups, int(chunk),
          int(n_chunks), int(multi), _p(scratch), _p(chunk_decay), _p(y), _stream())
    if multi:
        launch_count += 2   # three kernels


def gated_group_norm(y, z, weight, eps, q_start, q_len, n_entries, parts, out):
    """out = weight * n_g(y * silu(z)): y 32-bit [T, C]; z 32-bit sums [T, >= C] or [S, T, >= C] whose first C columns
    gate y; the row is cut into ``parts`` equal pieces, each divided by its own root mean square."""
    _need(y, "y", torch.float32); _need(weight, "weight", torch.float32); _need(out, "out")
    T, C = y.shape
    S, ss, ld = _rows_in(z, "z")
    assert z.shape[-1] >= C and z.shape[-2] >= T and out.shape == (T, C) and weight.numel() == C
    _call("vcb_gated_group_norm", _p(y), _p(z), S, ss, ld, _p(weight), float(eps), _p(q_start), _p(q_len), n_entries, T, C,
          int(parts), _p(out), _dt(out), _stream())


@functools.lru_cache(maxsize=None)
def moe_tile_rows() -> int:
    """Rows of a tile of the experts' products: every expert's (token, choice) pairs are padded to a multiple of it."""
    return int(lib().vcb_moe_tile_rows())


def moe_tiles_cap(n_pairs: int, n_experts: int, tile_rows: int | None = None) -> int:
    """The most tiles of ``tile_rows`` rows (default: the plain product's) that ``n_pairs`` pairs can fill when each of
    ``n_experts`` experts pads its own to whole tiles."""
    return min(n_pairs, n_experts) + n_pairs // (tile_rows or moe_tile_rows())


def moe_route(logits, q_start, q_len, n_entries, top, sel_e, sel_w, softmax_weights=False):
    """Per row of the step's entries: the ``top`` largest of the router's ``logits`` (32-bit [T, E] or [S, T, E]) ->
    ``sel_e`` [T, top] int32 (-1 in rows outside every entry) and ``sel_w`` [T, top]: sigmoid(logit), or the softmax over
    the chosen logits."""
    S, ss, ld = _rows_in(logits, "logits")
    T, E = logits.shape[-2:]
    _need(sel_e, "sel_e", torch.int32); _need(sel_w, "sel_w", torch.float32)
    assert sel_e.numel() == T * top and sel_w.numel() == T * top
    _call("vcb_moe_route", _p(logits), S, ss, ld, _p(q_start), _p(q_len), n_entries, T, E, int(top), int(bool(softmax_weights)),
          _p(sel_e), _p(sel_w), _stream())


def moe_group(sel_e, n_experts, tiles_cap, pos_of, src_of, tile_expert, tile_rows=None):
    """Sorts the pairs by expert into tiles of ``tile_rows`` rows (default: the plain product's; see csrc/kernels/moe.cu)."""
    for name, t in (("sel_e", sel_e), ("pos_of", pos_of), ("src_of", src_of), ("tile_expert", tile_expert)):
        _need(t, name, torch.int32)
    A = sel_e.numel()
    tile_rows = int(tile_rows or moe_tile_rows())
    assert pos_of.numel() == A and src_of.numel() == tiles_cap * tile_rows and tile_expert.numel() == tiles_cap
    _call("vcb_moe_group", _p(sel_e), A, int(n_experts), int(tiles_cap), tile_rows, _p(pos_of), _p(src_of), _p(tile_expert),
          _stream())


GROUPED_TILE_ROWS = (16, 32, 64, 128, 256)     # token tiles of the grouped tensor-core product


def moe_gather(x, src_of, sel_w, top, out):
    """out[pos] = x[token of the pair at sorted row pos] * sel_w[pair] (None: as it is), zeros where no pair sits."""
    _need(x, "x", contiguous=False); _need(out, "out", x.dtype); _need(src_of, "src_of", torch.int32)
    rows, K = out.shape
    assert x.shape[1] == K and x.stride(1) == 1 and src_of.numel() == rows
    _call("vcb_moe_gather", _p(x), x.stride(0), _dt(x), _p(src_of), _p(sel_w), int(top), rows, K, _p(out), _stream())


def gemm_grouped_ok(x, w) -> bool:
    """Whether the grouped tensor-core product can address these operands (bfloat16, 16-byte rows and bases)."""
    return (x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.shape[1] % 8 == 0 and x.stride(0) % 8 == 0
            and x.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0 and w.is_contiguous())


def gemm_bf16_grouped(w, x, tile_expert, tile_rows, out, status, act=None):
    """out[r, :] = act(w[tile_expert[r // tile_rows]] . x[r]) over the sorted rows (tcgen05 + TMA): w [E, N, K] bfloat16,
    x [tiles * tile_rows, K] bfloat16, out [tiles * tile_rows, N] bfloat16 or float32; tiles whose expert is -1 are
    skipped.  ``act``: None, "silu" or "relu2"."""
    _need(w, "w", torch.bfloat16); _need(x, "x", torch.bfloat16, contiguous=False); _need(out, "out")
    _need(tile_expert, "tile_expert", torch.int32)
    E, N, K = w.shape
    tiles = tile_expert.numel()
    assert tile_rows in GROUPED_TILE_ROWS and x.shape == (tiles * tile_rows, K) and out.shape == (tiles * tile_rows, N)
    if act not in (None, "silu", "relu2"):
        raise KernelError(f"gemm_bf16_grouped: activation '{act}' (None, 'silu' or 'relu2')")
    _call("vcb_gemm_bf16_grouped", _p(w), _p(x), _p(out), _dt(out), E, N, tiles, int(tile_rows), K, K, x.stride(0), out.stride(0),
          _p(tile_expert), 0 if act is None else ACTIVATIONS[act], _p(status), _stream())


def moe_gemm(x, w, tile_expert, out, *, src_of=None, sel_w=None, top=1, act=None):
    """The experts' product over the sorted tiles: w [E, N, K]; with ``src_of`` x is the tokens' rows [T, K], read through
    the sorted order and multiplied by the pairs' ``sel_w`` (None: as they are); without it x is [tiles * rows, K] in
    sorted order.  ``act``: out [tiles * rows, N] in the compute dtype after that activation; None: 32-bit sums."""
    _need(x, "x", w.dtype, contiguous=False); _need(w, "w"); _need(tile_expert, "tile_expert", torch.int32)
    E, N, K = w.shape
    tiles = tile_expert.numel()
    assert x.shape[1] == K and x.stride(1) == 1 and out.shape == (tiles * moe_tile_rows(), N)
    _need(out, "out", w.dtype if act is not None else torch.float32)
    if act is not None and act not in ACTIVATIONS:
        raise KernelError(f"activation '{act}' is not one of {sorted(ACTIVATIONS)}")
    _call("vcb_moe_gemm", _p(x), x.stride(0), _p(w), _dt(w), _p(tile_expert), _p(src_of), _p(sel_w), int(top),
          int(src_of is not None), _p(out), N, K, ACTIVATIONS[act] if act is not None else -1, tiles, _stream())


def moe_combine(y, pos_of, top, q_start, q_len, n_entries, out, shared=None, sel_w=None):
    """out[t] = shared[t] + sum over the token's pairs of y[pos_of[t, k]] (times sel_w[t, k] if given), k in order."""
    _need(y, "y", torch.float32); _need(pos_of, "pos_of", torch.int32); _need(out, "out", torch.float32)
    T, W = out.shape
    S = ss = ld = 0
    if shared is not None:
        S, ss, ld = _rows_in(shared, "shared")
        assert shared.shape[-1] == W and shared.shape[-2] >= T
    _call("vcb_moe_combine", _p(y), _p(pos_of), _p(sel_w), int(top), _p(shared), S, ss, ld, _p(q_start), _p(q_len), n_entries,
          T, W, _p(out), _stream())


def attn_merge(part_o, part_ml, dec_rows, out, n_dec, nh, hd, nslices):
    _need(part_o, "part_o", torch.float32); _need(part_ml, "part_ml", torch.float32)
    _need(dec_rows, "dec_rows", torch.int32); _need(out, "out")
    _call("vcb_attn_merge", _p(part_o), _p(part_ml), _p(dec_rows), _p(out), _dt(out), n_dec, nh, hd, nslices, _stream())


def sample(logits, params, counts, out, no_nucleus=False):
    """logits [R,V] f32; params [R,8] int32 records (see sampling.cu); counts [slots,V] int32 or None.
    ``no_nucleus``: no row has top_p < 1, so the vocabulary can be dealt to several blocks per row."""
    _need(logits, "logits", torch.float32, contiguous=False); _need(params, "params", torch.int32)
    _need(out, "out", torch.int32)
    R, V = logits.shape
    assert logits.stride(1) == 1 and params.shape == (R, 8) and out.numel() >= R
    if counts is not None:
        _need(counts, "counts", torch.int32)
        assert counts.shape[1] == V
    nb = max(1, min(64, 2 * num_sms() // max(R, 1), V // 2048))
    if no_nucleus and nb > 1:
        global launch_count
        from . import workspace
        part_v = workspace.empty((R * nb,), torch.float32, logits.device)
        part_i = workspace.empty((R * nb,), torch.int32, logits.device)
        _call("vcb_sample_split", _p(logits), logits.stride(0), R, V, _p(params), _p(counts), _p(part_v), _p(part_i),
              nb, _p(out), _stream())
        launch_count += 1   # two kernels
        return
    _call("vcb_sample", _p(logits), logits.stride(0), R, V, _p(params), _p(counts), _p(out), _stream())


def count_tokens(ids, slots, counts, n, slot_bias=0):
    """counts[slots[t] - slot_bias, ids[t]] += 1 for tokens whose slot entry less the bias is >= 0."""
    _need(ids, "ids", torch.int32); _need(slots, "slots", torch.int32); _need(counts, "counts", torch.int32)
    _call("vcb_count_tokens", _p(ids), _p(slots), _p(counts), n, counts.shape[1], slot_bias, _stream())


def scatter_i32(dst, idx, val, count, capacity):
    """dst.flat[idx[i]] = val[i] for i < min(count[0], capacity); count is a device int32."""
    _need(dst, "dst", torch.int32); _need(idx, "idx", torch.int32); _need(val, "val", torch.int32)
    _need(count, "count", torch.int32)
    _call("vcb_scatter_i32", _p(dst), _p(idx), _p(val), _p(count), capacity, dst.numel(), _stream())


def state_reset(state, slots, q_len, ctx_len, n_entries, value, status):
    """state [caches, slots, ...]: the rows of the requests whose entries start at position 0 (ctx_len == q_len > 0)
    are filled with ``value``; all on the device (a captured step includes it)."""
    _need(state, "state"); _need(slots, "slots", torch.int32); _need(q_len, "q_len", torch.int32); _need(ctx_len, "ctx_len", torch.int32)
    if state.dim() < 2:
        raise KernelError("a state tensor is [caches, slots, ...]")
    n_caches, num_slots = state.shape[0], state.shape[1]
    row = state[0, 0].numel()
    if state.dtype == torch.float32:
        bits = struct.unpack("<I", struct.pack("<f", float(value)))[0]
    elif state.dtype == torch.bfloat16:
        bits = struct.unpack("<I", struct.pack("<f", float(torch.tensor(float(value)).to(torch.bfloat16).float())))[0] >> 16
    elif state.dtype == torch.int32:
        bits = int(value) & 0xFFFFFFFF
    else:
        raise KernelError(f"state of type {state.dtype} (float32, bfloat16 or int32)")
    _call("vcb_state_reset", _p(state), state.element_size(), state.stride(0), state.stride(1), row, n_caches, num_slots,
          _p(slots), _p(q_len), _p(ctx_len), n_entries, bits, _p(status), _stream())


def selftest_wait_timeout(limit_clocks: int, status: torch.Tensor) -> list[int]:
    """Lets the kernels' bounded mbarrier wait run out on a barrier nothing arrives at (see csrc/kernels/selftest.cu)
    and returns [the wait's answer, the abort flag seen by another warp, a later wait's answer, whether that one
    returned at once]; the status word gets the wait-timeout bit."""
    _need(status, "status", torch.int32)
    out = torch.full((4,), -1, dtype=torch.int32, device=status.device)
    _call("vcb_selftest_wait_timeout", int(limit_clocks), _p(status), _p(out), _stream())
    return out.tolist()


def attn_mma_supported(dtype: torch.dtype, hd: int) -> bool:
    """Whether the tensor-core attention kernel takes this element type and head size."""
    return bool(lib().vcb_attn_mma_supported(BF16 if dtype == torch.bfloat16 else F32, hd))


def attn_mma_fused_supported(dtype: torch.dtype, hd: int, page_size: int) -> bool:
    """Whether decoded tokens can be attended straight from the stacked q, k, v projection (attn_mma_decode_fused)."""
    return bool(lib().vcb_attn_mma_fused_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size))


def attn_mma_decode_fused(qkv, q_weight, k_weight, eps, cos_sin, slot_map, out, pages, block_table, q_start,
                          q_len, ctx_len, items, n_items, part_o, part_ml, slice_counters, dec_rows, nh, nkv, hd, window,
                          status, table_row=None, use_norm=True, cluster=0):
    """Attention of single decoded tokens straight from the stacked projection ``qkv`` [S, T, (nh + 2 nkv) hd]
    (32-bit k-slice partial sums): each block norms and rotates its own query heads, and the blocks that read the
    token's own position store its key and value in the cache first -- what qknorm_rope_kvwrite and attn_mma do
    in two kernels.  Items: one token each, as for :func:`attn_mma` with rows_max 16; a token's position is its
    entry's context length less one."""
    _need(qkv, "qkv", torch.float32); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    _need(cos_sin, "cos_sin", torch.float32); _need(slot_map, "slot_map", torch.int32)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len), ("items", items)):
        _need(t, name, torch.int32)
    assert qkv.dim() == 3 and qkv.shape[2] == (nh + 2 * nkv) * hd and cos_sin.shape[1] == hd
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    wdt = F32
    if use_norm:
        _need(q_weight, "q_norm weight"); _need(k_weight, "k_norm weight", q_weight.dtype)
        wdt = _dt(q_weight)
    _call("vcb_attn_mma_decode_fused", _p(qkv), qkv.shape[0], qkv.stride(0), _p(q_weight), _p(k_weight), wdt, int(use_norm),
          float(eps), _p(cos_sin), cos_sin.shape[0], _p(slot_map), _p(out), _p(pages), pages.stride(0),
          _p(block_table), _p(table_row), block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items,
          _p(part_o), _p(part_ml), _p(slice_counters), _p(dec_rows), nh, nkv, hd, page_size, num_pages, int(window or 0),
          1.0 / math.sqrt(hd), _p(status), int(cluster), _stream())


@functools.lru_cache(maxsize=None)
def attn_mma_max_clusters(hd: int, cluster: int, deep: bool) -> int:
    """How many clusters of ``cluster`` blocks of the decode attention kernel run at once on this device (``deep``: the
    variant with the ring of six stages, which has an SM to itself).  -1 when the driver does not say."""
    return int(lib().vcb_attn_mma_max_clusters(hd, cluster, int(deep)))


def attn_tc_supported(dtype: torch.dtype, hd: int, page_size: int) -> bool:
    """Whether the tcgen05 attention kernel for prompt portions takes this element type, head size and page size."""
    return bool(lib().vcb_attn_tc_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size))


def attn_tc(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, nh, nkv, hd, window, status,
            table_row=None, work=None, scale=None, keep_first=0, dist_a=None, dist_b=None, softcap=0.0, slope=None, sink=False):
    """Attention of prompt portions on tcgen05 tensor cores (bfloat16, head_dim 64 or 128, pages of 8 to 64
    tokens), with the options of :func:`attn_window_bias` (``scale``, ``keep_first``, ``dist_a``/``dist_b``, ``softcap``,
    ``slope``, ``sink``).
    Items as for :func:`attn_paged` with one key slice and at most 128 rows each.  ``work``: two int32
    zeros, zero again when the kernel is through (the queue its blocks take their units from); launches that share
    them must follow one another on a stream.  Made on the spot when not given."""
    if work is None:
        work = torch.zeros(2, dtype=torch.int32, device=q.device)
    _need(work, "work", torch.int32)
    sink_value = _sink_scores(sink, nh)
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    if dist_a is not None:
        _need(dist_a, "dist_a", torch.float32); _need(dist_b, "dist_b", torch.float32)
        assert dist_a.numel() == nh and dist_b.numel() == nh
    if slope is not None:
        _need(slope, "slope", torch.float32); assert slope.numel() == nh
    _call("vcb_attn_tc_ex", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, nh, nkv, hd, page_size,
          num_pages, int(window or 0), 1.0 / math.sqrt(hd) if scale is None else float(scale), int(keep_first or 0),
          _p(dist_a), _p(dist_b), float(softcap or 0.0), _p(slope), int(sink_value is not None or bool(sink)), _p(sink_value),
          _p(status), _p(work), _stream())


def attn_mma(q, out, pages, block_table, q_start, q_len, ctx_len, items, n_items, rows_max, part_o, part_ml,
             nh, nkv, hd, window, status, table_row=None, allow_tma=True, slice_counters=None, dec_rows=None,
             cluster=0, scale=None, keep_first=0, dist_a=None, dist_b=None, softcap=0.0, slope=None, sink=False):
    """Tensor-core variant of :func:`attn_paged` (bfloat16, head_dim 64 or 128; rows_max 16 or 128), with the
    options of :func:`attn_window_bias` (``scale``, default 1/sqrt(hd); ``keep_first``; ``dist_a``/``dist_b``;
    ``softcap``, ``slope``, ``sink``).
    With ``slice_counters`` (int32 zeros, one per decoded token and KV head group, left at zero again) and
    ``dec_rows``, the block that finishes a token's last key slice merges the slices itself; with ``cluster`` = the
    number of slices per token (2 to 8) as well, the slices' blocks run as a cluster and merge through shared memory."""
    sink_value = _sink_scores(sink, nh)
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_start", q_start), ("q_len", q_len), ("ctx_len", ctx_len),
                    ("items", items)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    if dist_a is not None:
        _need(dist_a, "dist_a", torch.float32); _need(dist_b, "dist_b", torch.float32)
        assert dist_a.numel() == nh and dist_b.numel() == nh
    if slope is not None:
        _need(slope, "slope", torch.float32); assert slope.numel() == nh
    _call("vcb_attn_mma_ex", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_start), _p(q_len), _p(ctx_len), _p(items), n_items, rows_max, _p(part_o),
          _p(part_ml), _p(slice_counters), _p(dec_rows), nh, nkv, hd, page_size, num_pages, int(window or 0),
          1.0 / math.sqrt(hd) if scale is None else float(scale), int(keep_first or 0), _p(dist_a), _p(dist_b),
          float(softcap or 0.0), _p(slope), int(sink_value is not None or bool(sink)), _p(sink_value), _p(status), int(allow_tma),
          int(cluster), _stream())


def attn_stream_supported(dtype: torch.dtype, hd: int, page_size: int, nh: int, nkv: int) -> bool:
    """Whether :func:`attn_stream` takes these sizes (bfloat16, head_dim 64 or 128, pages of 8 to 64 tokens, at
    most 16 query heads a KV head)."""
    return bool(lib().vcb_attn_stream_supported(BF16 if dtype == torch.bfloat16 else F32, hd, page_size, nh, nkv))


def attn_stream(q, out, pages, block_table, q_len, ctx_len, items, n_dec, dec_rows, nh, nkv, hd, window, status,
                table_row=None, blocks=0):
    """Single decoded tokens, many of them: persistent blocks walk the (token, KV head) pairs, all keys of a pair in
    one block, the loading warp running ahead from pair to pair.  ``items`` [n_dec, 6] as for :func:`attn_mma` with
    one slice; ``dec_rows`` [n_dec] the tokens' rows of ``q`` and ``out``; entries with q_len 0 are skipped.
    ``blocks``: how many blocks to run on (0: two an SM, or one where the head group is large)."""
    _need(q, "q", torch.bfloat16); _need(out, "out", torch.bfloat16); _need(pages, "pages", torch.bfloat16)
    for name, t in (("block_table", block_table), ("q_len", q_len), ("ctx_len", ctx_len), ("items", items),
                    ("dec_rows", dec_rows)):
        _need(t, name, torch.int32)
    num_pages, two, nkv_p, page_size, hd_p = pages.shape
    assert two == 2 and nkv_p == nkv and hd_p == hd
    _call("vcb_attn_stream", _p(q), _p(out), _p(pages), pages.stride(0), _p(block_table), _p(table_row),
          block_table.shape[1], _p(q_len), _p(ctx_len), _p(items), n_dec, _p(dec_rows), nh, nkv, hd, page_size,
          num_pages, int(window or 0), 1.0 / math.sqrt(hd), _p(status), int(blocks), _stream())


# --------------------------------------------------------------------------  a look at a step from inside
_timeline = None
_TL_ROLE_EVERY, _TL_ROLE_BLOCKS, _TL_ROLES, _TL_ROLE_MARKS = 37, 8, 3, 2048     # as in kernels/common.cuh
_TL_ROLE_WORDS = _TL_ROLE_BLOCKS * _TL_ROLES * _TL_ROLE_MARKS * 2
TIMELINE_KERNELS = {1: "gemm", 2: "attn_decode", 3: "add_rmsnorm", 4: "qknorm_rope", 5: "swiglu", 6: "attn_tc", 7: "other"}


def timeline_begin(capacity: int = 1 << 18) -> None:
    """Starts recording the kernels' timeline marks (a library built with VLLM_CPP_B200_TIMELINE=1 only): thread 0 of
    every block notes when the block starts, when its wait for the kernel before it ends, and when it ends."""
    global _timeline
    L = lib()
    if not hasattr(L, "vcb_timeline_set_gemm"):
        raise KernelError("this kernel library was built without timeline marks (build with VLLM_CPP_B200_TIMELINE=1)")
    _timeline = torch.zeros(2 + 4 * capacity + _TL_ROLE_WORDS, dtype=torch.int64, device="cuda")
    _timeline[1] = capacity
    torch.cuda.synchronize()
    for unit in ("gemm", "attn_mma", "attn_tc", "attn_stream", "elementwise"):
        fn = getattr(L, f"vcb_timeline_set_{unit}")
        fn.argtypes, fn.restype = [c_void_p], c_int
        if fn(_timeline.data_ptr()) != 0:
            raise KernelError("could not hand the timeline buffer to the kernels")


def timeline_end():
    """Stops recording; returns the records as a list of dicts (t_ns, clock, kernel, phase, sm, tile, block, grid), by
    time.  The marks of the roles inside a block (phases from 10 on; they have a ``role``, a tile number and the SM's
    clock, but no time: t_ns 0) come first."""
    global _timeline
    L = lib()
    torch.cuda.synchronize()
    for unit in ("gemm", "attn_mma", "attn_tc", "attn_stream", "elementwise"):
        getattr(L, f"vcb_timeline_set_{unit}")(None)
    buf = _timeline.cpu().numpy()
    _timeline = None
    n = int(min(buf[0], buf[1]))
    rec = buf[2:2 + 4 * n].reshape(n, 4)
    out = [dict(t_ns=int(r[0]), clock=int(r[1]), kernel=TIMELINE_KERNELS.get(int(r[2]) >> 32, "?"), phase=(int(r[2]) >> 24) & 0xFF,
                sm=int(r[2]) & 0xFF, tile=0, block=int(r[3]) & 0xFFFFFFFF, grid=int(r[3]) >> 32) for r in rec]
    # the logs of the roles inside a block: (clock, tag) pairs per (recording block, role)
    logs = buf[2 + 4 * int(buf[1]):].reshape(_TL_ROLE_BLOCKS, _TL_ROLES, _TL_ROLE_MARKS, 2)
    for b in range(_TL_ROLE_BLOCKS):
        for role in range(_TL_ROLES):
            for clock, tag in logs[b, role]:
                tag = int(tag) & 0xFFFFFFFFFFFFFFFF
                if tag >> 63:
                    out.append(dict(t_ns=0, clock=int(clock), kernel=TIMELINE_KERNELS.get((tag >> 48) & 0xFF, "?"), phase=(tag >> 32) & 0xFFFF,
                                    sm=-1, tile=tag & 0xFFFFFFFF, block=b * _TL_ROLE_EVERY, grid=0, role=role))
    out.sort(key=lambda d: d["t_ns"])
    return out


# -------------------------------------------------------------------------- several residual streams, token shift


def hyper_mix_norm(streams, *, init=None, y=None, mix=None, outw=None, inw=None, gain=None, eps=0.0, out=None, rows=None):
    """One pass over the S residual streams ``streams`` [S, T, W] (32-bit): the write-back of the sublayer before
    (``y``: 32-bit [T, W] or [Sy, T, W] partial sums; x_r <- sum_s mix[s, r] x_s + outw[r] y, ``mix`` and ``outw`` None:
    the identity and ones), then the read-out for the one ahead (u = sum_r inw[r] x_r, ``inw`` None: the plain sum) and
    its norm ``gain`` * u / sqrt(mean(u^2) + eps) into ``out`` [n, W] (32-bit or the compute dtype; ``gain`` None: no
    read-out).  ``init`` [T, W]: the step's first sublayer -- every stream starts as that row.  ``rows`` (int32): only
    those rows are read out, and the streams are left as they are."""
    _need(streams, "streams", torch.float32)
    S, T, W = streams.shape
    Sy = ys = ldy = 0
    if y is not None:
        Sy, ys, ldy = _rows_in(y, "y")
        assert y.shape[-1] == W and y.shape[-2] >= T
    for name, t, n in (("mix", mix, S * S), ("outw", outw, S), ("inw", inw, S), ("gain", gain, W)):
        if t is not None:
            _need(t, name, torch.float32); assert t.numel() == n, (name, t.shape, n)
    if init is not None:
        _need(init, "init", torch.float32); assert init.shape == (T, W)
    n = T
    if rows is not None:
        _need(rows, "rows", torch.int32)
        n = rows.numel()
    if out is not None:
        _need(out, "out"); assert out.shape[0] >= n and out.shape[1] == W
    _call("vcb_hyper_mix_norm", _p(streams), _p(init), _p(y), Sy, ys, ldy, _p(mix), _p(outw), _p(inw), _p(gain), float(eps),
          _p(out), _dt(out) if out is not None else F32, _p(rows), n, T, W, S, _stream())


def token_shift(h, mu, state, q_start, q_len, slots, n_entries, out):
    """out[t] = h[t] + (h[t-1] - h[t]) * mu per channel over each entry's rows (32-bit ``h`` [T, W]); the row before an
    entry's first is the request's ``state`` [slots, W] (32-bit), which then takes the entry's last row of ``h``."""
    _need(h, "h", torch.float32); _need(mu, "mu", torch.float32); _need(state, "state", torch.float32, contiguous=False)
    _need(out, "out")
    T, W = h.shape
    assert mu.numel() == W and out.shape == (T, W) and state.shape[-1] == W and state.stride(-1) == 1
    _call("vcb_token_shift", _p(h), _p(mu), _p(state), state.stride(0), _p(q_start), _p(q_len), _p(slots), n_entries, T, W,
          _p(out), _dt(out), _stream())


# -------------------------------------------------------------------------- attention through a latent


def latent_norm_rope_store(u, q_gain, kv_gain, eps, positions, freq, gain, slot_map, cq_out, pages, page_size, q_rank,
                           kv_rank, rot, status, v_width=None):
    """From the stacked down projections ``u`` (32-bit [T, q_rank + kv_rank + rot] or partial sums): the normed query
    latent to ``cq_out`` [T, q_rank]; the normed key/value latent c and the rotated shared key part into the token's
    cache row.  A page is one flat row: [page_size, kv_rank + rot] key rows [c | k_rot], then [page_size, v_width]
    value rows [c | zeros] (``v_width`` None: kv_rank lanes, c alone).  ``freq`` [rot / 2] 32-bit; cos and sin are
    multiplied by ``gain``."""
    v_width = int(kv_rank if v_width is None else v_width)
    S, ss, ld = _rows_in(u, "u")
    T = u.shape[-2]
    assert u.shape[-1] == q_rank + kv_rank + rot and rot % 2 == 0
    _need(cq_out, "cq_out"); _need(pages, "pages", cq_out.dtype); _need(positions, "positions", torch.int32)
    _need(slot_map, "slot_map", torch.int32); _need(q_gain, "q_gain", torch.float32); _need(kv_gain, "kv_gain", torch.float32)
    if rot:
        _need(freq, "freq", torch.float32); assert freq.numel() == rot // 2
    assert cq_out.shape == (T, q_rank) and q_gain.numel() == q_rank and kv_gain.numel() == kv_rank
    assert pages[0].numel() == page_size * (kv_rank + rot + v_width), (pages.shape, page_size, kv_rank, rot, v_width)
    _call("vcb_latent_norm_rope_store", _p(u), S, ss, ld, _p(q_gain), _p(kv_gain), float(eps), _p(positions), _p(freq),
          float(gain), _p(slot_map), _p(cq_out), _p(pages), pages.stride(0), int(page_size), pages.shape[0], int(q_rank),
          int(kv_rank), int(rot), v_width, T, _dt(cq_out), _p(status), _stream())


def head_linear(x, m, out, *, heads, n_in, n_out, in_head_stride, in_off=0, out_head_stride, out_off=0):
    """out[t, h * out_head_stride + out_off + j] = sum_c m[h, j, c] x[t, h * in_head_stride + in_off + c]: every head
    meets a small matrix of its own.  ``x``: 32-bit [T, C] / [S, T, C] partial sums, or one [T, C] buffer of the compute
    dtype; ``m`` [heads, n_out, n_in]; sums are 32-bit."""
    _need(m, "m"); _need(out, "out", contiguous=False)
    assert m.shape == (heads, n_out, n_in) and out.stride(-1) == 1
    if x.dtype == torch.float32:
        S, ss, ld = _rows_in(x, "x")
    else:
        _need(x, "x", contiguous=False); assert x.dim() == 2 and x.stride(1) == 1
        S, ss, ld = 1, 0, x.stride(0)
    T = x.shape[-2]
    assert (heads - 1) * in_head_stride + in_off + n_in <= x.shape[-1]
    assert (heads - 1) * out_head_stride + out_off + n_out <= out.shape[-1] and out.shape[0] >= T
    _call("vcb_head_linear", _p(x), _dt(x), S, ss, ld, int(in_head_stride), int(in_off), _p(m), _dt(m), _p(out), _dt(out),
          out.stride(0), int(out_head_stride), int(out_off), T, int(heads), int(n_in), int(n_out), _stream())


def rope_rows(x, positions, freq, gain, out, *, heads, dims, width, in_head_stride, in_off=0, out_head_stride, out_off=0):
    """Copies ``width`` lanes of every head's slice of the 32-bit sums ``x`` into ``out``, the first ``dims`` of them
    rotated: lane i pairs with lane i + dims/2, the angle is position * freq[i], cos and sin times ``gain``."""
    S, ss, ld = _rows_in(x, "x")
    T = x.shape[-2]
    _need(out, "out", contiguous=False); _need(positions, "positions", torch.int32)
    if dims:
        _need(freq, "freq", torch.float32); assert freq.numel() == dims // 2
    assert out.stride(-1) == 1 and dims % 2 == 0
    assert (heads - 1) * in_head_stride + in_off + width <= x.shape[-1]
    assert (heads - 1) * out_head_stride + out_off + width <= out.shape[-1]
    _call("vcb_rope_rows", _p(x), S, ss, ld, int(in_head_stride), int(in_off), _p(positions), _p(freq), float(gain), _p(out),
          _dt(out), out.stride(0), int(out_head_stride), int(out_off), T, int(heads), int(dims), int(width), _stream())


# -------------------------------------------------------------------------- recurrences with a matrix state per head


def matrix_rnn(mode, u, state, q_start, q_len, slots, n_entries, out, *, heads, d, dv, q_col, k_col, v_col, x=None,
               kv_heads=None, b_col=0, a_col=0, dt_bias=None, rate=None, f_bias=None, lower=None, z=None, tau=1.0, decay=None,
               ctx_len=None, freq=None, rot=0, interleaved=False):
    """A recurrence over each entry's tokens whose state S [d, dv] per head lies in ``state`` [slots, heads, dv, d] (32-bit, a value column's rows in a run), ``out`` [T, heads dv].

    ``mode`` "delta": S <- g S; w = beta (v - S^T k); S <- S + k w^T; o = S^T q.  q, k, v are columns ``q_col``,
    ``k_col``, ``v_col`` of ``x`` [T, C] (32-bit, convolved and activated; q and k of ``kv_heads`` heads, made unit
    vectors here, q times d^(-1/2)); beta = sigmoid(u[:, b_col + h]), g = exp(-rate_h softplus(u[:, a_col + h] + dt_bias_h)).
    ``mode`` "gated": S <- diag(f) S + (1 - f) v^T; o = S^T q with q = silu(u[:, q_col ...]), f = lower + (1 - lower)
    sigmoid(u[:, k_col ...] + f_bias), v = u[:, v_col ...].
    ``mode`` "decayed": S <- diag(f) S + k v^T; o = S^T q with q = u[:, q_col ...] d^(-1/2), k = u[:, k_col ...],
    v = u[:, v_col ...] and f = sigmoid(z + f_bias)^(1 / tau), ``z`` [T, heads d] the 32-bit sums of a projection of its own.
    ``mode`` "retention": S <- decay_h S + k v^T; o = S^T q with q, k, v columns of u, the first ``rot`` lanes of every q
    and k head turned by position * freq[i] (lanes paired in halves, or ``interleaved``), k then times d^(-1/2);
    positions from ``ctx_len``.
    ``u``: the projection's 32-bit sums ([S, T, C] partials)."""
    S, ss, ld = _rows_in(u, "u")
    _need(state, "state", torch.float32, contiguous=False); _need(out, "out", torch.float32)
    assert state.shape[1:] == (heads, dv, d) and state[0].is_contiguous() and out.shape[1] == heads * dv
    m = {"delta": 0, "gated": 1, "decayed": 2, "retention": 3}[mode]
    ldx = 0
    zS = zss = zld = 0
    if m == 0:
        _need(x, "x", torch.float32, contiguous=False); assert x.stride(1) == 1
        ldx = x.stride(0)
        for name, t in (("dt_bias", dt_bias), ("rate", rate)):
            _need(t, name, torch.float32); assert t.numel() == heads
    elif m == 1:
        for name, t in (("f_bias", f_bias), ("lower", lower)):
            _need(t, name, torch.float32); assert t.numel() == heads * d
    elif m == 2:
        zS, zss, zld = _rows_in(z, "z")
        _need(f_bias, "f_bias", torch.float32); assert f_bias.numel() == heads * d and z.shape[-1] == heads * d
        assert z.shape[-2] >= out.shape[0] and tau > 0
    else:
        _need(decay, "decay", torch.float32); assert decay.numel() == heads
        _need(ctx_len, "ctx_len", torch.int32)
        if rot:
            _need(freq, "freq", torch.float32); assert freq.numel() == rot // 2
    _call("vcb_matrix_rnn", m, _p(u), S, ss, ld, _p(x), ldx, int(q_col), int(k_col), int(v_col), int(b_col), int(a_col),
          _p(dt_bias), _p(rate), _p(f_bias), _p(lower), _p(state), state.stride(0), _p(q_start), _p(q_len), _p(slots),
          n_entries, int(out.shape[0]), int(heads), int(kv_heads or heads), int(d), int(dv), _p(out),
          _p(z), zS, zss, zld, 1.0 / float(tau), _p(decay), _p(ctx_len), _p(freq), int(rot), int(bool(interleaved)), _stream())


def head_norm_gate(o, weight, eps, q_start, q_len, n_entries, heads, dv, out, gate=None, gate_col=0):
    """out[t, h] = weight * o[t, h] / sqrt(mean(o[t, h]^2) + eps) (* silu(gate[t, gate_col + h dv ...]) with a gate):
    every head of the 32-bit ``o`` [T, heads dv] by its own root mean square, one gain [dv] for all heads (None: no gain)."""
    _need(o, "o", torch.float32); _need(out, "out")
    T = o.shape[0]
    assert o.shape == (T, heads * dv) and out.shape == o.shape
    if weight is not None:
        _need(weight, "weight", torch.float32); assert weight.numel() == dv
    S = ss = ld = 0
    if gate is not None:
        S, ss, ld = _rows_in(gate, "gate")
        assert gate_col + heads * dv <= gate.shape[-1]
    _call("vcb_head_norm_gate", _p(o), _p(gate), S, ss, ld, int(gate_col), _p(weight), float(eps), _p(q_start), _p(q_len),
          n_entries, T, int(heads), int(dv), _p(out), _dt(out), _stream())


def moe_route_grouped(logits, correction, n_groups, keep, weight_scale, q_start, q_len, n_entries, top, sel_e, sel_w):
    """The router that chooses by sigmoid(logit) + ``correction`` among the experts of the ``keep`` best of ``n_groups``
    equal groups of neighbours (a group's score: the sum of its two largest choice scores; ``n_groups`` <= 1: all
    experts are open); a chosen expert's weight is sigmoid(logit) * ``weight_scale``."""
    S, ss, ld = _rows_in(logits, "logits")
    T, E = logits.shape[-2:]
    _need(sel_e, "sel_e", torch.int32); _need(sel_w, "sel_w", torch.float32)
    if correction is not None:
        _need(correction, "correction", torch.float32); assert correction.numel() == E
    assert sel_e.numel() == T * top and sel_w.numel() == T * top
    _call("vcb_moe_route_grouped", _p(logits), S, ss, ld, _p(correction), int(n_groups or 1), int(keep or 0), float(weight_scale),
          _p(q_start), _p(q_len), n_entries, T, E, int(top), _p(sel_e), _p(sel_w), _stream())


# -------------------------------------------------------------------------- sublayers side by side on one normed input


def _terms(tensors, name):
    """A list of 32-bit [T, C] or [S, T, C] operands -> the four ctypes arrays a kernel that adds them all reads."""
    n = len(tensors)
    ptrs, counts, sstr, lds = (c_void_p * n)(), (c_int * n)(), (c_longlong * n)(), (c_longlong * n)()
    for k, t in enumerate(tensors):
        S, ss, ld = _rows_in(t, name)
        ptrs[k], counts[k], sstr[k], lds[k] = t.data_ptr(), S, ss, ld
    return ptrs, counts, sstr, lds


def sum_add_rmsnorm(resid, terms, gain, eps, out, rows=None, row_extra=None, vec_extra=None):
    """resid[t] += sum of ``terms`` (up to four 32-bit results, each [T, H] or [S, T, H] partial sums) + row_extra[t] +
    vec_extra, then out = gain * resid[t] / sqrt(mean(resid[t]^2) + eps), in one pass.  ``gain`` 32-bit [H]; ``out`` None:
    the additions alone.  With ``rows`` (int32 indices) only those rows are made and the stream is left alone."""
    _need(resid, "resid", torch.float32)
    T, H = resid.shape
    terms = [t for t in terms if t is not None]
    for t in terms:
        assert t.shape[-1] == H and t.shape[-2] >= T, (t.shape, resid.shape)
    for name, t, numel in (("row_extra", row_extra, None), ("vec_extra", vec_extra, H), ("gain", gain, H)):
        if t is not None:
            _need(t, name, torch.float32)
            assert numel is None or t.numel() == numel
    if row_extra is not None:
        assert row_extra.shape[-1] == H and row_extra.shape[0] >= T
    n = T if rows is None else rows.numel()
    if rows is not None:
        _need(rows, "rows", torch.int32)
    if out is not None:
        _need(out, "out"); assert out.shape[0] >= n and out.shape[1] == H and gain is not None
    ptrs, counts, sstr, lds = _terms(terms, "term")
    _call("vcb_sum_add_rmsnorm", _p(resid), len(terms), ptrs, counts, sstr, lds, _p(row_extra), _p(vec_extra), _p(gain), float(eps),
          _p(out), _dt(out) if out is not None else F32, _p(rows), n, H, _stream())


def branch_norm_mean(results, gains, eps, out):
    """out[t] = 1/N sum_b gains[b] * results[b][t] / sqrt(mean(results[b][t]^2) + eps): N results (32-bit [T, H] or
    [S, T, H] partial sums) of mixers that read one input, each normed over the width with its own gain, averaged."""
    _need(out, "out", torch.float32)
    T, H = out.shape
    assert len(results) == len(gains) and 1 <= len(results) <= 4
    for g in gains:
        _need(g, "gain", torch.float32); assert g.numel() == H
    for r in results:
        assert r.shape[-1] == H and r.shape[-2] >= T
    ptrs, counts, sstr, lds = _terms(results, "result")
    gp = (c_void_p * len(gains))(*[g.data_ptr() for g in gains])
    _call("vcb_branch_norm_mean", len(results), ptrs, counts, sstr, lds, gp, float(eps), _p(out), T, H, _stream())


def polynorm(u, coef, eps, out):
    """out[t] = a n(z) + b n(z^2) + c n(z^3) + e with z = u[t] (32-bit sums [T, F] or [S, T, F]), powers lane by lane,
    n(v) = v / sqrt(mean(v^2) + eps) over the F lanes, and (a, b, c, e) = ``coef`` (float32 [4] on the device)."""
    S, ss, ld = _rows_in(u, "u")
    T, Fw = u.shape[-2:]
    _need(coef, "coef", torch.float32); _need(out, "out")
    assert coef.numel() == 4 and out.shape == (T, Fw)
    _call("vcb_polynorm", _p(u), S, ss, ld, _p(coef), float(eps), _p(out), _dt(out), T, Fw, _stream())


# -------------------------------------------------------------------------- rotary attention with its options as parameters


def qkv_rope_store(qkv, q_gain, k_gain, eps, positions, freq, vfreq, slot_map, q_out, pages, nh, nkv, hd, vd, status, *,
                   rot, interleaved=False, values_from_keys=False):
    """From the stacked projection's 32-bit sums ``qkv`` ([T, C] or [S, T, C]; C = nh hd + nkv hd + nkv vd, or without the
    value columns where ``values_from_keys``: the keys as projected are the values): with ``q_gain`` [nh hd] / ``k_gain``
    [nkv hd] all of a token's query (key) lanes divided by their root mean square times the gain; the first ``rot`` lanes
    of every q and k head turned by position * freq[i], pairs (i, i + rot/2) or ``interleaved`` (2i, 2i+1); with
    ``vfreq`` [vd/2] every value head turned likewise over all its lanes; queries to ``q_out``, keys and values to the
    tokens' slots of ``pages`` (see :func:`kv_page_views`)."""
    S, ss, ld = _rows_in(qkv, "qkv")
    T, C = qkv.shape[-2:]
    assert C == nh * hd + nkv * hd + (0 if values_from_keys else nkv * vd), (C, nh, nkv, hd, vd)
    if q_gain is not None:
        _need(q_gain, "q_gain", torch.float32); _need(k_gain, "k_gain", torch.float32)
        assert q_gain.numel() == nh * hd and k_gain.numel() == nkv * hd
    _need(positions, "positions", torch.int32); _need(slot_map, "slot_map", torch.int32)
    if rot:
        _need(freq, "freq", torch.float32); assert freq.numel() == rot // 2
    if vfreq is not None:
        _need(vfreq, "vfreq", torch.float32); assert vfreq.numel() == vd // 2 and vd % 2 == 0
    _need(q_out, "q_out"); assert q_out.shape == (T, nh * hd)
    _need(pages, "pages", q_out.dtype)
    page_size, num_pages = kv_page_views(pages, nkv, hd, vd)
    _call("vcb_qkv_rope_store", _p(qkv), S, ss, ld, _p(q_gain), _p(k_gain), float(eps), _p(positions), _p(freq), _p(vfreq),
          _p(slot_map), _p(q_out), _p(pages), pages.stride(0), page_size, num_pages, nh, nkv, hd, vd, int(rot), vd,
          int(bool(interleaved)), int(bool(values_from_keys)), T, _dt(q_out), _p(status), _stream())


def rotate_heads(x, positions, freq, *, heads, width, dims, interleaved=False, sign=1.0):
    """x [T, heads * width] in place: the first ``dims`` lanes of every head turned by sign * position * freq[i]."""
    _need(x, "x"); _need(positions, "positions", torch.int32); _need(freq, "freq", torch.float32)
    T = x.shape[0]
    assert x.shape[1] == heads * width and freq.numel() == dims // 2
    _call("vcb_rotate_heads", _p(x), _dt(x), _p(positions), _p(freq), float(sign), T, int(heads), int(width), int(dims),
          int(bool(interleaved)), _stream())
