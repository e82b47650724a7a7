"""A plain, slow implementation of the Pinorax design: one function per mechanism, whole sequences at once, no cache,
no batching, torch on the CPU in float64.

It takes the configuration as the dictionary that config.json holds and the weights by their checkpoint names, and
shares no code with the engine. Notation: u is a sublayer's input [n, width] for n tokens at positions 0..n-1; a
matrix W is stored [out, in] and applied as u W^T. ``rnd`` rounds at the places where an engine that computes its
matrix products in bfloat16 rounds (the operands of the products and the cached latent); the default rounds nothing.
"""
from __future__ import annotations

import json
import math
import os
import struct
from typing import Dict, List, Optional, Tuple

import numpy as np
import torch

F = torch.float64


def ident(x: torch.Tensor) -> torch.Tensor:
    return x


def bf16(x: torch.Tensor) -> torch.Tensor:
    return x.to(torch.bfloat16).to(F)


# ---------------------------------------------------------------------------------------------- norms
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last dimension, eps inside the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def scalar_norm(x: torch.Tensor, g: torch.Tensor, eps: float) -> torch.Tensor:
    """Unit RMS times one learned number for all coordinates."""
    return unit_rms(x, eps) * g.reshape(())


def weighted_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Unit RMS times a weight per coordinate."""
    return unit_rms(x, eps) * w


# ---------------------------------------------------------------------------------------------- embedding
def embed(tokens: List[int], table: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Row of the token plus the learned vector of its position 0..n-1 (neither is scaled)."""
    n = len(tokens)
    return table[torch.tensor(tokens, dtype=torch.long)] + positions[torch.arange(n)]


# ---------------------------------------------------------------------------------------------- attention
def softmax_with_sink(scores: torch.Tensor, sink: torch.Tensor) -> torch.Tensor:
    """scores [H, n, n] (every j <= i is seen), sink [H]: p_ij = exp(s_ij) / (exp(sink_h) + sum over j' <= i of exp(s_ij'))."""
    H, n, _ = scores.shape
    seen = torch.ones(n, n, dtype=torch.bool).tril()
    s = scores.masked_fill(~seen, -math.inf)
    top = torch.maximum(s.max(-1, keepdim=True).values, sink.view(H, 1, 1))
    e = torch.exp(s - top)
    return e / (e.sum(-1, keepdim=True) + torch.exp(sink.view(H, 1, 1) - top))


def latent_attention(u: torch.Tensor, m: dict, w: Dict[str, torch.Tensor], eps: float, rnd=ident) -> torch.Tensor:
    """q = W_q u; c = N(W_dkv u) with the weight dkv.norm (only c would be cached); per head k = W_uk c and v = W_uv c;
    score = q . k * scale, causal, softmax with the head's sink; the heads' outputs side by side times
    sigmoid(W_g u), then W_o."""
    n = u.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    u = rnd(u)
    q = (u @ w["q"].T).view(n, H, d)
    c = rnd(weighted_norm(u @ w["dkv"].T, w["dkv.norm"], eps))
    k = (c @ w["uk"].T).view(n, H, d)
    v = (c @ w["uv"].T).view(n, H, dv)
    p = softmax_with_sink(torch.einsum("ihd,jhd->hij", q, k) * m["scale"], w["sink"])
    heads = torch.einsum("hij,jhd->ihd", p, v).reshape(n, H * dv)
    gated = heads * torch.sigmoid(u @ w["g"].T)
    return rnd(gated) @ w["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def dense_ff(u: torch.Tensor, w: Dict[str, torch.Tensor], rnd=ident) -> torch.Tensor:
    """W_down (silu(W_gate u + b_gate) * (W_up u + b_up)) + b_down."""
    u = rnd(u)
    g = u @ w["gate"].T + w["gate.b"]
    up = u @ w["up"].T + w["up.b"]
    return rnd(g * torch.sigmoid(g) * up) @ w["down"].T + w["down.b"]


def capped_expert(u: torch.Tensor, gate: torch.Tensor, up: torch.Tensor, down: torch.Tensor, limit: float, rnd=ident) -> torch.Tensor:
    """g = min(W_gate u, limit), v = clamp(W_up u, -limit, limit); W_down (g sigmoid(1.702 g) (v + 1)). No biases."""
    u = rnd(u)
    g = torch.clamp(u @ gate.T, max=limit)
    v = torch.clamp(u @ up.T, min=-limit, max=limit)
    return rnd(g * torch.sigmoid(1.702 * g) * (v + 1.0)) @ down.T


def table_experts(u: torch.Tensor, tokens: List[int], mlp: dict, w: Dict[str, torch.Tensor], rnd=ident) -> torch.Tensor:
    """Each token's experts are row ``token id`` of the table, each with weight 1 / top; a shared expert, when the
    layer has one, runs for every token and is added."""
    top = mlp["router"]["top"]
    out = torch.zeros_like(u)
    for t, tok in enumerate(tokens):
        for e in w["table"][tok].tolist():
            e = int(e)
            out[t] += capped_expert(u[t:t + 1], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], mlp["expert"]["limit"], rnd)[0] / top
    if mlp.get("shared") is not None:
        out = out + capped_expert(u, w["shared.gate"], w["shared.up"], w["shared.down"], mlp["shared"]["limit"], rnd)
    return out


# ---------------------------------------------------------------------------------------------- the layer
def depth_average(results: List[torch.Tensor], a: torch.Tensor) -> torch.Tensor:
    """sum_j a[j] * results[j] over everything so far (results[0] the embedding's output)."""
    assert a.numel() == len(results)
    return sum(a[j] * results[j] for j in range(len(results)))


def softcap(z: torch.Tensor, cap: float) -> torch.Tensor:
    return cap * torch.tanh(z / cap)


def _sub(weights: Dict[str, torch.Tensor], prefix: str) -> Dict[str, torch.Tensor]:
    return {k[len(prefix):]: (v if v.dtype in (torch.int32, torch.int64) else v.to(F)) for k, v in weights.items() if k.startswith(prefix)}


def layer_forward(x: torch.Tensor, tokens: List[int], layer: dict, w: Dict[str, torch.Tensor], eps: float, mult: float, rnd=ident) -> torch.Tensor:
    """One norm, both sublayers read it: x + mult * (mixer(h) + ff(h)). ``w``: the layer's tensors without its prefix."""
    h = scalar_norm(x, w["norm1"], eps)
    y = latent_attention(h, layer["mixer"], _sub(w, "mix."), eps, rnd)
    mlp = layer.get("mlp")
    if mlp is not None:
        ff = _sub(w, "mlp.")
        y = y + (dense_ff(h, ff, rnd) if mlp["kind"] == "dense" else table_experts(h, tokens, mlp, ff, rnd))
    return x + mult * y


def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: List[int], rnd=ident) -> Tuple[torch.Tensor, torch.Tensor]:
    """(logits [n, vocab], the stream that goes on after every layer [layers, n, width])."""
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    x = embed(tokens, weights["embed"].to(F), weights["pos"].to(F))
    results, after = [x], []
    for i, layer in enumerate(config["layers"]):
        w = _sub(weights, f"l{i}.")
        results.append(layer_forward(x, tokens, layer, w, eps, mult, rnd))
        x = depth_average(results, w["dwa"])
        after.append(x)
    logits = rnd(scalar_norm(x, weights["final.norm"].to(F), eps)) @ weights["head"].to(F).T
    return softcap(logits, config["logit_softcap"]), torch.stack(after)


def load(folder: str) -> Tuple[dict, Dict[str, torch.Tensor]]:
    """(config.json as a dictionary, the tensors of model.safetensors by name), read with a reader of its own."""
    with open(os.path.join(folder, "config.json")) as f:
        config = json.load(f)
    with open(os.path.join(folder, "model.safetensors"), "rb") as f:
        n = struct.unpack("<Q", f.read(8))[0]
        header = json.loads(f.read(n))
        data = f.read()
    out = {}
    for name, e in header.items():
        if name == "__metadata__":
            continue
        a, b = e["data_offsets"]
        if e["dtype"] == "BF16":
            bits = np.frombuffer(data[a:b], dtype="<u2").astype(np.uint32) << 16
            t = torch.from_numpy(bits.view(np.float32).copy())
        elif e["dtype"] == "I32":
            t = torch.from_numpy(np.frombuffer(data[a:b], dtype="<i4").copy())
        else:
            t = torch.from_numpy(np.frombuffer(data[a:b], dtype="<f4").copy())
        out[name] = t.view(e["shape"])
    return config, out
