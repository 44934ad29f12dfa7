"""A plain, slow implementation of the Fifudra design: float64, whole sequences, one function per mechanism.

It shares no code with the package: its own reading of config.json's keys, its own loops.  A model is a dict of the
configuration (as config.json holds it) and a dict name -> float64 tensor.  ``forward`` returns the logits of every
position and, if asked, the sum of the residual streams after every layer run.
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


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def silu(z):
    return z * torch.sigmoid(z)


def token_shift(h, mu, before=None):
    """h [T, W] -> h + (previous row - h) * mu; the row before the first is ``before`` (zeros if None)."""
    first = torch.zeros_like(h[:1]) if before is None else before.reshape(1, -1)
    prev = torch.cat([first, h[:-1]], 0)
    return h + (prev - h) * mu


def hyper_read(streams, w_in):
    """streams [S, T, W], w_in [S] -> [T, W]."""
    return torch.einsum("s,stw->tw", w_in, streams)


def hyper_write(streams, y, w_mix, w_out):
    """new[t] = sum_s mix[s, t] old[s] + out[t] y, all streams from the old ones."""
    return torch.einsum("sr,stw->rtw", w_mix, streams) + w_out[:, None, None] * y[None]


def yarn_frequencies(rot):
    """The per-pair frequencies and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    half = dims // 2
    f = [base ** (-2.0 * i / dims) for i in range(half)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(orig / (2 * math.pi * turns)) / (2 * math.log(base))

    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    out = []
    for i in range(half):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(f[i] / factor * ramp + f[i] * (1 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, freqs, gain):
    """x [T, ..., dims]: lane i pairs with lane i + dims / 2."""
    half = freqs.numel()
    ang = positions.to(F64)[:, None] * freqs[None, :]
    while ang.dim() < x.dim():
        ang = ang.unsqueeze(1)
    c, s = torch.cos(ang) * gain, torch.sin(ang) * gain
    u, v = x[..., :half], x[..., half:2 * half]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., 2 * half:]], -1)


def latent_attention(h, w, m, eps, pos0=0):
    """h [T, W]; w: the mixer's tensors by short name; m: the mixer's sizes."""
    T = h.shape[0]
    H, d, r, dv, kr = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(pos0, pos0 + T)
    freqs, gain = yarn_frequencies(m["rot"])
    cq = rms_norm(h @ w["dq"].T, w["dq.norm"], eps)
    q = (cq @ w["uq"].T).view(T, H, d + r)
    q_plain, q_rot = q[..., :d], rotate(q[..., d:], pos, freqs, gain)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :kr], w["dkv.norm"], eps)
    k_rot = rotate(down[:, kr:], pos, freqs, gain)          # [T, r], shared by the heads
    k_plain = (c @ w["uk"].T).view(T, H, d)
    v = (c @ w["uv"].T).view(T, H, dv)
    out = torch.zeros(T, H, dv, dtype=F64)
    for i in range(T):
        s = (torch.einsum("hd,jhd->hj", q_plain[i], k_plain[:i + 1]) + q_rot[i] @ k_rot[:i + 1].T) * float(m["scale"])
        p = torch.softmax(s, -1)
        out[i] = torch.einsum("hj,jhv->hv", p, v[:i + 1])
    return out.reshape(T, H * dv) @ w["o"].T


def short_conv(x, taps_w):
    """x [T, C], taps_w [C, taps]: the last column multiplies the current token, zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = torch.cat([torch.zeros(taps - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(taps):
        out += padded[j:j + T] * taps_w[:, j]
    return out


def delta_rule(h, w, m, eps):
    T = h.shape[0]
    H, G, d, dv = int(m["heads"]), int(m["kv_heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(short_conv(h @ w["q"].T, w["q.conv"])).view(T, G, d)
    k = silu(short_conv(h @ w["k"].T, w["k.conv"])).view(T, G, d)
    v = silu(short_conv(h @ w["v"].T, w["v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * d ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(h @ w["b"].T)
    decay = torch.exp(-torch.exp(w["A_log"]) * torch.nn.functional.softplus(h @ w["a"].T + w["dt_bias"]))
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = decay[t, hd] * S
            u = beta[t, hd] * (v[t, hd] - S.T @ k[t, g])
            S = S + torch.outer(k[t, g], u)
            out[t, hd] = S.T @ q[t, g]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w["norm"]
    out = out.reshape(T, H * dv) * silu(h @ w["g"].T)
    return out @ w["o"].T


def hgrn2(h, w, m, eps):
    T = h.shape[0]
    H, d, dv = int(m["heads"]), int(m["dim"]), int(m["vdim"])
    q = silu(h @ w["q"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
    low = w["lower"]
    f = (low + (1 - low) * torch.sigmoid(h @ w["f"].T + w["f.b"])).view(T, H, d)
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = f[t, hd][:, None] * S + torch.outer(1 - f[t, hd], v[t, hd])
            out[t, hd] = S.T @ q[t, hd]
    out = out / torch.sqrt((out * out).mean(-1, keepdim=True) + eps) * w["norm"]
    return out.reshape(T, H * dv) @ w["o"].T


def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, w_router, correction, router, margins=None):
    """-> (chosen experts [T, top], their weights [T, top]).  ``margins`` (a list) receives, per call, the smallest gap
    by which any token's choice was decided: between the last chosen and the first left-out choice score, and between
    the last kept and the first dropped group."""
    E, top = int(router["experts"]), int(router["top"])
    s = torch.sigmoid(h @ w_router.T)
    choice = s + correction
    groups = router.get("groups")
    gap = math.inf
    if groups:
        n, keep = int(groups["count"]), int(groups["keep"])
        per = E // n
        grouped = choice.view(-1, n, per)
        score = grouped.topk(min(2, per), -1).values.sum(-1)
        kept = score.topk(keep, -1).indices
        if keep < n:
            ranked = score.sort(-1, descending=True).values
            gap = min(gap, float((ranked[:, keep - 1] - ranked[:, keep]).min()))
        allowed = torch.zeros(choice.shape[0], n, dtype=torch.bool)
        allowed.scatter_(1, kept, True)
        choice = torch.where(allowed[:, :, None].expand(-1, -1, per).reshape(-1, E), choice,
                             torch.full_like(choice, -math.inf))
    chosen = choice.topk(top, -1).indices
    if top < E:
        ranked = choice.sort(-1, descending=True).values
        gap = min(gap, float((ranked[:, top - 1] - ranked[:, top]).min()))
    if margins is not None:
        margins.append(gap)
    return chosen, s.gather(1, chosen) * float(router.get("scale", 1.0))


def routed_ff(h, w, mlp, margins=None):
    chosen, weight = route(h, w["router"], w["correction"], mlp["router"], margins)
    out = torch.zeros(h.shape[0], w["e0.down"].shape[0], dtype=F64)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weight[t]):
            out[t] += a * gated_ff(h[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
    return out


MIXERS = {"latent_attention": latent_attention, "delta": delta_rule, "hgrn2": hgrn2}


def layer_order(cfg):
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = int(loop["start"]), int(loop["stop"]), int(loop["times"])
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(cfg, tensors, tokens, want_layers=False, margins=None):
    """tokens: a list of ids -> logits [T, vocab] (and [runs, T, W] sums of the streams after every layer run).
    ``margins``: see ``route``."""
    eps = float(cfg["norm"]["eps"])
    x = tensors["embed"][torch.tensor(tokens)] * float(cfg.get("embedding", {}).get("scale", 1.0))
    n_streams = cfg.get("streams")
    streams = x[None].repeat(int(n_streams or 1), 1, 1)
    after = []
    for li in order_runs(cfg):
        layer, p = cfg["layers"][li], f"l{li}."
        t = sub(tensors, p)
        for q, name in ((1, "mixer"), (2, "ff")):
            if q == 2 and layer.get("mlp") is None:
                continue
            if n_streams:
                u = hyper_read(streams, t[f"hc{q}.in"])
            else:
                u = streams[0]
            h = rms_norm(u, t[f"norm{q}"], eps)
            if q == 1:
                h = token_shift(h, t["shift"])
                w = sub(t, "mix.")
                y = (latent_attention(h, w, layer["mixer"], eps) if layer["type"] == "latent_attention"
                     else MIXERS[layer["type"]](h, w, layer["mixer"], eps))
            else:
                w = sub(t, "mlp.")
                y = gated_ff(h, w["gate"], w["up"], w["down"]) if layer["mlp"]["kind"] == "dense" else routed_ff(h, w, layer["mlp"], margins)
            if n_streams:
                streams = hyper_write(streams, y, t[f"hc{q}.mix"], t[f"hc{q}.out"])
            else:
                streams = streams + y[None]
        after.append(streams.sum(0))
    x = rms_norm(streams.sum(0), tensors["final.norm"], eps)
    logits = x @ tensors["embed"].T
    return (logits, torch.stack(after)) if want_layers else logits


def order_runs(cfg):
    return layer_order(cfg)


def greedy(cfg, tensors, prompt, n_new):
    """The greedy continuation (lowest index wins a tie), recomputing the whole sequence for every token."""
    seq = list(prompt)
    for _ in range(n_new):
        seq.append(int(forward(cfg, tensors, seq)[-1].argmax()))
    return seq[len(prompt):]
