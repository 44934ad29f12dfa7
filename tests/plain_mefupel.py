"""A plain, slow implementation of the Mefupel design: float64, whole sequences, one function per mechanism.

It shares no code with the package: its own reading of config.json's keys, its own loops.  A model is a dict of the
configuration (as config.json holds it) and a dict name -> float64 tensor.  ``forward`` returns the logits of every
position and, if asked, the residual stream after every layer run.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch

from plain_qwen3 import read_safetensors

F64 = torch.float64


def read_model(model_dir):
    model_dir = Path(model_dir)
    return json.loads((model_dir / "config.json").read_text()), read_safetensors(model_dir / "model.safetensors")


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def one_plus_norm(x, w, eps):
    """The layers' norm: the gain is stored around zero."""
    return rms(x, eps) * (1.0 + w)


def silu(z):
    return z * torch.sigmoid(z)


def frequencies(base, dims):
    return torch.tensor([float(base) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)


def rotate(x, positions, base, dims, pairing, sign=1.0):
    """x [T, heads, n]: the first ``dims`` lanes of every head turn by sign * position * f_i; pairing "half" pairs lane
    i with lane i + dims / 2, "interleaved" lane 2i with lane 2i + 1."""
    if dims == 0:
        return x
    half = dims // 2
    ang = sign * positions.to(F64)[:, None, None] * frequencies(base, dims)[None, None, :]
    c, s = torch.cos(ang), torch.sin(ang)
    out = x.clone()
    if pairing == "half":
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * c - v * s
        out[..., half:dims] = v * c + u * s
    else:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * c - v * s
        out[..., 1:dims:2] = v * c + u * s
    return out


def window_softmax_attention(q, k, v, scale, window, sink=None):
    """q [T, H, d], k [T, G, d], v [T, G, dv] -> [T, H, dv].  Position i sees j with 0 <= i - j < window (window 0 or
    None: every j <= i).  ``sink`` [H]: exp(sink_h) joins the denominator, with no value."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=F64)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1) if window else 0
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            m = s.max() if sink is None else torch.maximum(s.max(), sink[h])
            e = torch.exp(s - m)
            den = e.sum() + (0.0 if sink is None else torch.exp(sink[h] - m))
            out[i, h] = (e / den) @ v[lo:i + 1, g]
    return out


def rotary_attention(h, w, m, positions):
    """The mixer "attention": interleaved rotation of q and k, values rotated by their own position over all their
    lanes and the heads' sums turned back by the query's position."""
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    rot = m["rot"]
    base, dims = float(rot["base"]), int(rot["dims"])
    q = (h @ w["q"].T).view(T, H, d)
    k = (h @ w["k"].T).view(T, G, d)
    v = (h @ w["v"].T).view(T, G, dv)
    q = rotate(q, positions, base, dims, "interleaved")
    k = rotate(k, positions, base, dims, "interleaved")
    v = rotate(v, positions, base, dv, "interleaved")
    o = window_softmax_attention(q, k, v, float(m["scale"]), int((m.get("mask") or {}).get("size") or 0))
    o = rotate(o, positions, base, dv, "interleaved", sign=-1.0)
    return o.reshape(T, H * dv) @ w["o"].T


def sink_attention(h, w, m, eps, positions):
    """The left branch: keys double as values (as projected), q and k normed over the whole projection, rotated in
    halves, softmax with a learned sink per head."""
    T = h.shape[0]
    H, G, d = int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    rot = m["rot"]
    base, dims = float(rot["base"]), int(rot["dims"])
    q = h @ w["q"].T
    k = h @ w["k"].T
    v = k.view(T, G, d)
    q = (rms(q, eps) * w["q.norm"]).view(T, H, d)
    k = (rms(k, eps) * w["k.norm"]).view(T, G, d)
    q = rotate(q, positions, base, dims, "half")
    k = rotate(k, positions, base, dims, "half")
    o = window_softmax_attention(q, k, v, float(m["scale"]), int((m.get("mask") or {}).get("size") or 0), sink=w["sink"])
    return o.reshape(T, H * d) @ w["o"].T


def decayed_state_scan(q, k, v, decay, state=None):
    """S_t = diag(decay_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t for one head: q, k [T, d], v [T, dv], decay [T, d]."""
    T, d = q.shape
    S = torch.zeros(d, v.shape[1], dtype=F64) if state is None else state.clone()
    out = torch.zeros(T, v.shape[1], dtype=F64)
    for t in range(T):
        S = decay[t][:, None] * S + torch.outer(k[t], v[t])
        out[t] = S.T @ q[t]
    return out, S


def gla(h, w, m, eps):
    """Gated linear attention: a decay per key channel from a low-rank projection."""
    T = h.shape[0]
    H, d, dv, tau = int(m["heads"]), int(m["dim"]), int(m["vdim"]), float(m["tau"])
    q = (h @ w["q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    z = (h @ w["a1"].T) @ w["a2"].T + w["a2.b"]
    alpha = torch.sigmoid(z).pow(1.0 / tau).view(T, H, d)
    o = torch.stack([decayed_state_scan(q[:, i], k[:, i], v[:, i], alpha[:, i])[0] for i in range(H)], 1)
    o = rms(o, eps) * w["norm"]
    return (o.reshape(T, H * dv) * silu(h @ w["g"].T)) @ w["o"].T


def retention(h, w, m, eps, positions):
    """The right branch: linear attention with one fixed decay per head, q and k rotated in halves."""
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    rot = m["rot"]
    base, dims = float(rot["base"]), int(rot["dims"])
    q = rotate((h @ w["q"].T).view(T, H, d), positions, base, dims, "half")
    k = rotate((h @ w["k"].T).view(T, H, d), positions, base, dims, "half") * d ** -0.5
    v = (h @ w["v"].T).view(T, H, dv)
    outs = []
    for i in range(H):
        decay = torch.full((T, d), float(m["decay"][i]), dtype=F64)
        outs.append(decayed_state_scan(q[:, i], k[:, i], v[:, i], decay)[0])
    o = rms(torch.stack(outs, 1), eps)
    return (o.reshape(T, H * dv) * silu(h @ w["g"].T)) @ w["o"].T


def parallel_mixer(h, w, m, eps, positions):
    left = sink_attention(h, sub(w, "left."), m["left"], eps, positions)
    right = retention(h, sub(w, "right."), m["right"], eps, positions)
    return 0.5 * (rms(left, eps) * w["left.out"] + rms(right, eps) * w["right.out"])


def polynorm(z, coef, eps):
    a, b, c, e = (float(x) for x in coef)
    return a * rms(z, eps) + b * rms(z * z, eps) + c * rms(z * z * z, eps) + e


def feed_forward(h, w, eps):
    return polynorm(h @ w["up"].T, w["act"], eps) @ w["down"].T


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def passes(cfg):
    """[(layer, number of the pass it opens or None)] in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop.get("times", 1))
    runs = [(i, None) for i in range(a)]
    for t in range(times):
        runs += [(i, t if i == a else None) for i in range(a, b)]
    return runs + [(i, None) for i in range(b, n)]


def forward(cfg, tensors, tokens, want_layers=False):
    eps = float(cfg["norm"]["eps"])
    ids = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(ids))
    x0 = tensors["embed"][ids]
    x = x0.clone()
    after = []
    for i, opens in passes(cfg):
        if opens is not None:
            if opens > 0:
                x = x + x0
            x = x + tensors["loop.step"][opens]
        layer = cfg["layers"][i]
        w = sub(tensors, f"l{i}.")
        h = one_plus_norm(x, w["norm1"], eps)
        mw, m = sub(w, "mix."), layer["mixer"]
        if layer["type"] == "attention":
            y = rotary_attention(h, mw, m, positions)
        elif layer["type"] == "gla":
            y = gla(h, mw, m, eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(h, mw, m, eps, positions)
        else:
            raise ValueError(f"layer type {layer['type']}")
        if layer.get("mlp") is not None:
            y = y + feed_forward(h, sub(w, "mlp."), eps)
        x = x + y
        after.append(x.clone())
    logits = one_plus_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    return (logits, torch.stack(after)) if want_layers else logits


def greedy(cfg, tensors, prompt, n_new):
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, tensors, seq)[-1].argmax()))
    return seq[len(prompt):]
