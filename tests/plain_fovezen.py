"""A plain, slow implementation of the Fovezen design: whole sequences, no cache, no batching, one function
per mechanism, on the CPU. It is the oracle of the Fovezen tests and shares no code with the engine (its own
reading of config.json, its own loops over tokens).

Notation. A model keeps ``streams`` copies X[s] of the residual stream, all equal to the embedding at the start.
Sublayer q of a layer reads u = sum_s a_q[s] X[s], computes y = f(N(u)) with N(u) = u / sqrt(mean(u^2) + eps) (1 + w),
and rewrites every copy at once: X'[t] = sum_s M_q[s, t] X[s] + b_q[t] y. The model's output is the norm of
sum_s X[s]. Layers ``start .. stop-1`` of ``loop`` run ``times`` times in a row.

Every function takes ``dt`` (float64 for an oracle without rounding of its own, float32 otherwise) and ``rnd``,
applied where a bfloat16 engine stores an operand of a matrix product in 16 bits.
"""
from __future__ import annotations

import json
import math
from typing import Dict, List, Optional

import torch

import plain_model as pm


def ident(t):
    return t


def bf16(t):
    return t.to(torch.bfloat16).to(t.dtype)


def load(model_dir: str):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return pm.read_safetensors_f32(f"{model_dir}/model.safetensors"), cfg


# ------------------------------------------------------------------------------------ small pieces
def unit_rms(x, eps):
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def norm_one_plus(x, w, eps):
    return unit_rms(x, eps) * (1.0 + w.to(x.dtype))


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w.to(x.dtype)


def silu(z):
    return z * torch.sigmoid(z)


def softplus(z):
    return torch.where(z > 30.0, z, torch.log1p(torch.exp(torch.clamp(z, max=30.0))))


def linear(w, h, rnd):
    """W h for every row of h; both operands stored in 16 bits by a bfloat16 engine."""
    return rnd(h) @ rnd(w.to(h.dtype)).T


def short_conv(u, w, bias=None):
    """y_t = bias + sum_j w[:, j] u_(t - taps + 1 + j) per channel, zeros before the first token. u [T, C], w [C, taps]."""
    T, C = u.shape
    taps = w.shape[1]
    y = torch.zeros_like(u) if bias is None else bias.to(u.dtype).expand(T, C).clone()
    for j in range(taps):
        back = taps - 1 - j
        if back < T:
            y[back:] += w[:, j].to(u.dtype) * u[:T - back]
    return y


# ------------------------------------------------------------------------------------ mixers
def mamba2_mixer(W: Dict[str, torch.Tensor], p: str, m: dict, h, eps, dt, rnd):
    """State-space mixer in its scalar-decay form. ``p`` is the tensors' prefix (ending in '.')."""
    H, P, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = H * P
    T = h.shape[0]
    proj = linear(W[p + "in"], h, rnd)
    z, xbc, raw = proj[:, :inner], proj[:, inner:2 * inner + 2 * G * N], proj[:, 2 * inner + 2 * G * N:]
    xbc = silu(short_conv(xbc, W[p + "conv"], W[p + "conv.b"]))
    x = xbc[:, :inner].reshape(T, H, P)
    B = xbc[:, inner:inner + G * N].reshape(T, G, N)
    C = xbc[:, inner + G * N:].reshape(T, G, N)
    step = softplus(raw + W[p + "dt_bias"].to(dt))
    rate = torch.exp(W[p + "A_log"].to(dt))
    skip = W[p + "D"].to(dt)
    y = torch.zeros(T, H, P, dtype=dt)
    for hd in range(H):
        g = hd // (H // G)
        S = torch.zeros(N, P, dtype=dt)
        for t in range(T):
            S = torch.exp(-rate[hd] * step[t, hd]) * S + step[t, hd] * torch.outer(B[t, g], x[t, hd])
            y[t, hd] = S.T @ C[t, g] + skip[hd] * x[t, hd]
    y = y.reshape(T, inner) * silu(z)
    parts = m["norm_groups"]
    y = unit_rms(y.reshape(T, parts, inner // parts), eps).reshape(T, inner) * W[p + "norm"].to(dt)
    return linear(W[p + "o"], y, rnd)


def softmax_attention(q, k, v, scale, rnd, window: Optional[int] = None, softcap: Optional[float] = None):
    """q [T, H, d], k [T, G, d], v [T, G, dv]; position i sees j <= i, and with a window only i - j < window."""
    T, H, d = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[2], dtype=q.dtype)
    qs, ks, vs = rnd(q), rnd(k), rnd(v)
    i = torch.arange(T)
    visible = i[None, :] <= i[:, None]
    if window is not None:
        visible &= (i[:, None] - i[None, :]) < window
    for hd in range(H):
        g = hd // (H // G)
        s = (qs[:, hd] @ ks[:, g].T) * scale
        if softcap is not None:
            s = softcap * torch.tanh(s / softcap)
        s = s.masked_fill(~visible, -math.inf)
        out[:, hd] = rnd(torch.softmax(s, dim=-1)) @ vs[:, g]
    return out


def window_conv_attention(W, p, m, h, eps, dt, rnd):
    """The left branch of a parallel mixer: projections, a short convolution on each, norm per head, capped scores, window."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q, k, v = (linear(W[p + n], h, rnd) for n in ("q", "k", "v"))
    if m.get("conv"):
        q, k, v = (short_conv(u, W[p + n + ".conv"]) for u, n in ((q, "q"), (k, "k"), (v, "v")))
    q = norm_plain(q.reshape(T, H, d), W[p + "q.norm"], eps)
    k = norm_plain(k.reshape(T, G, d), W[p + "k.norm"], eps)
    o = softmax_attention(q, k, v.reshape(T, G, dv), m["scale"], rnd, window=(m.get("mask") or {}).get("size"), softcap=m.get("softcap"))
    return linear(W[p + "o"], o.reshape(T, H * dv), rnd)


def gated_linear_attention(W, p, m, h, eps, dt, rnd):
    """The right branch: a state per head whose rows fade each by its own factor per token."""
    H, d, dv, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    T = h.shape[0]
    q = (linear(W[p + "q"], h, rnd) * d ** -0.5).reshape(T, H, d)
    k = linear(W[p + "k"], h, rnd).reshape(T, H, d)
    v = linear(W[p + "v"], h, rnd).reshape(T, H, dv)
    z = linear(W[p + "a2"], linear(W[p + "a1"], h, rnd), rnd) + W[p + "a2.b"].to(dt)
    alpha = torch.exp(-softplus(-z) / tau).reshape(T, H, d)          # sigmoid(z)^(1/tau)
    o = torch.zeros(T, H, dv, dtype=dt)
    for hd in range(H):
        S = torch.zeros(d, dv, dtype=dt)
        for t in range(T):
            S = alpha[t, hd][:, None] * S + torch.outer(k[t, hd], v[t, hd])
            o[t, hd] = S.T @ q[t, hd]
    o = norm_plain(o, W[p + "norm"], eps).reshape(T, H * dv) * silu(linear(W[p + "g"], h, rnd))
    return linear(W[p + "o"], o, rnd)


def parallel_mixer(W, p, m, h, eps, dt, rnd):
    left = window_conv_attention(W, p + "left.", m["left"], h, eps, dt, rnd)
    right = gated_linear_attention(W, p + "right.", m["right"], h, eps, dt, rnd)
    return 0.5 * (norm_plain(left, W[p + "left.out"], eps) + norm_plain(right, W[p + "right.out"], eps))


def scaled_frequencies(rot: dict, dt):
    dims = rot["dims"]
    f = torch.tensor([rot["base"] ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if sc:
        factor, low, high, original = (float(sc[k]) for k in ("factor", "low", "high", "original"))
        out = []
        for fi in f.tolist():
            wave = 2.0 * math.pi / fi
            if wave < original / high:
                out.append(fi)
            elif wave > original / low:
                out.append(fi / factor)
            else:
                s = (original / wave - low) / (high - low)
                out.append((1.0 - s) * fi / factor + s * fi)
        f = torch.tensor(out, dtype=torch.float64)
    return f.to(dt)


def rotate_half_layout(x, freq, dims):
    """x [T, heads, d]: dimension i is paired with i + dims/2 for i < dims/2; the rest pass."""
    T = x.shape[0]
    angle = torch.arange(T, dtype=x.dtype)[:, None] * freq[None, :]
    c, s = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    a, b = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([a * c - b * s, b * c + a * s, x[..., dims:]], dim=-1)


def rotary_attention(W, p, m, h, eps, dt, rnd):
    """The 'attention' mixer: norm over the whole projection, partial rotation, all earlier keys."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = norm_plain(linear(W[p + "q"], h, rnd), W[p + "q.norm"], eps).reshape(T, H, d)
    k = norm_plain(linear(W[p + "k"], h, rnd), W[p + "k.norm"], eps).reshape(T, G, d)
    v = linear(W[p + "v"], h, rnd).reshape(T, G, dv)
    rot = m.get("rot")
    if rot:
        freq = scaled_frequencies(rot, dt)
        q, k = rotate_half_layout(q, freq, rot["dims"]), rotate_half_layout(k, freq, rot["dims"])
    o = softmax_attention(q, k, v, m["scale"], rnd)
    return linear(W[p + "o"], o.reshape(T, H * dv), rnd)


MIXERS = {"mamba2": mamba2_mixer, "parallel": parallel_mixer, "attention": rotary_attention}


def feed_forward(W, p, f, h, dt, rnd):
    limit = float(f["limit"])
    g = torch.clamp(linear(W[p + "gate"], h, rnd), max=limit)
    u = torch.clamp(linear(W[p + "up"], h, rnd), min=-limit, max=limit)
    return linear(W[p + "down"], g * torch.sigmoid(1.702 * g) * (u + 1.0), rnd)


# ------------------------------------------------------------------------------------ layers and the model
def layer_order(cfg) -> List[int]:
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def sublayer_streams(X, y_fn, W, p, eps, norm_w):
    """X [S, T, D] -> X' with the sublayer's result mixed in. ``p``: '<layer>.hc<q>.'."""
    a, b, M = W[p + "in"].to(X.dtype), W[p + "out"].to(X.dtype), W[p + "mix"].to(X.dtype)
    u = torch.einsum("s,std->td", a, X)
    y = y_fn(norm_one_plus(u, norm_w, eps))
    return torch.einsum("sr,std->rtd", M, X) + b[:, None, None] * y[None]


def forward(W: Dict[str, torch.Tensor], cfg: dict, tokens, dt=torch.float64, rnd=ident, layers_out: Optional[list] = None):
    """Logits [T, vocab] of one sequence. ``layers_out``: a list that receives the stream (the sum of the copies) after every layer run."""
    eps = float(cfg["norm"]["eps"])
    S = cfg.get("streams")
    x = W["embed"].to(dt)[torch.as_tensor(tokens, dtype=torch.long)]
    X = x[None].repeat(S or 1, 1, 1)
    for i in layer_order(cfg):
        layer = cfg["layers"][i]
        p = f"l{i}."
        mix = lambda hh: MIXERS[layer["type"]](W, p + "mix.", layer["mixer"], hh, eps, dt, rnd)
        ff = (lambda hh: feed_forward(W, p + "mlp.", layer["mlp"], hh, dt, rnd)) if layer.get("mlp") else None
        if S:
            X = sublayer_streams(X, mix, W, p + "hc1.", eps, W[p + "norm1"])
            if ff:
                X = sublayer_streams(X, ff, W, p + "hc2.", eps, W[p + "norm2"])
        else:
            X = X + mix(norm_one_plus(X[0], W[p + "norm1"], eps))[None]
            if ff:
                X = X + ff(norm_one_plus(X[0], W[p + "norm2"], eps))[None]
        if layers_out is not None:
            layers_out.append(X.sum(dim=0).clone())
    x = norm_one_plus(X.sum(dim=0), W["final.norm"], eps)
    return linear(W["head"], x, rnd) * float(cfg.get("logit_scale", 1.0))
