"""Attention over a shared low-rank latent: the cache holds one short row per token instead of keys and values per head."""
from __future__ import annotations

import torch

from ..cache import CacheNeed
from ..config import PartSpec
from ..ops import kernels
from ..ops.linear import Linear
from .registry import POSITION_ENCODINGS, build_part, register_mixer


@register_mixer("latent_attention")
class LatentAttentionMixer:
    """Queries, keys and values are made from two latents of the input u:
    cq = N(W_dq u) (q_rank values, unit RMS times ``q_latent_norm``) and q_h = W_uq,h cq = [q_h^p (dim), q_h^r (rot)];
    [c'; k^r] = W_dkv u with c = N(c') (kv_rank values, unit RMS times ``kv_latent_norm``) and k^r (rot values), one for
    all heads; k_h^p = W_uk,h c and v_h = W_uv,h c. q_h^r and k^r are rotated by the token's position (pairs (2i, 2i+1),
    the position encoding's frequencies and amplitude). score_h(i, j) = (q_h^p(i) . k_h^p(j) + q_h^r(i) . k^r(j)) * scale
    over a window of the last ``window`` positions, softmax (with ``sink`` = "learned" its denominator holds
    exp(``sink``_h) too), out_h = sum_j p_j v_h(j), x += W_o [out_1 .. out_H]. Without a query latent (``q_rank`` None)
    the queries are a product of the input itself, q = W_q u. With ``output_gate`` every value of [out_1 .. out_H] is
    multiplied by sigmoid((W_g u)) of its place before W_o (the gate reads the mixer's input, like the projections).

    The cache holds [c, rotated k^r] per token, kv_rank + rot values, for all heads. The heads' key matrices are applied
    to the queries instead of the cached latents, (W_uk,h^T q_h^p) . c = q_h^p . (W_uk,h c), so a step does work for its
    own tokens only: attention runs with one key/value "head" of kv_rank + rot dimensions whose values are the first
    kv_rank columns of the same rows, and W_uv,h is applied to the attention's output.

    Params: ``hidden_size``, ``num_heads``, ``head_dim`` (dim), ``rotary_dim`` (rot), ``value_dim``, ``q_rank``,
    ``kv_rank``, ``scale``, ``window``, ``norm_eps``, ``position`` (a PartSpec of kind ``rope_on_device`` for rot
    dimensions; None without a rotated part) and optionally ``sink`` ("learned") and ``output_gate``. Weights: ``w_down``
    [q_rank + kv_rank + rot (+ H value_dim), hidden] (rows of W_dq, or of W_q [H (dim + rot)] without a query latent,
    then W_dkv, then W_g with an output gate: everything that reads u is one product), ``q_latent_norm`` [q_rank] and
    ``w_uq`` [H (dim + rot), q_rank] (with a query latent), ``kv_latent_norm`` [kv_rank], ``w_uk`` [H dim, kv_rank], ``w_uv``
    [H value_dim, kv_rank], ``w_o`` [hidden, H value_dim], ``sink`` [H]."""

    graph_safe = True
    takes_then = True

    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = H = int(params["num_heads"])
        self.head_dim, self.rotary_dim = int(params["head_dim"]), int(params["rotary_dim"])
        self.value_dim, self.kv_rank = int(params["value_dim"]), int(params["kv_rank"])
        self.q_rank = int(params["q_rank"]) if params.get("q_rank") else 0          # 0: the queries come from the input itself
        self.output_gate = bool(params.get("output_gate", False))
        self.scale = float(params["scale"])
        self.window = params.get("window")
        self.eps = float(params["norm_eps"])
        D, d, r, dv, qr, kr = self.hidden_size, self.head_dim, self.rotary_dim, self.value_dim, self.q_rank, self.kv_rank
        pos_spec = params.get("position") or PartSpec("none", {})
        self.position = build_part(POSITION_ENCODINGS, "position encoding", pos_spec, {}, build)
        self.freq = getattr(self.position, "freq", None)
        if r > 0 and (self.freq is None or 2 * self.freq.numel() != r or not self.position.interleaved):
            raise ValueError("latent attention: the rotated part needs a 'rope_on_device' encoding of rotary_dim values, interleaved")
        self.amplitude = float(getattr(self.position, "amplitude", 1.0))
        if not kernels.attention_rows_supported(kr + r, kr):
            raise ValueError(f"latent attention: a latent of {kr} + {r} values is not supported by the attention kernel")
        # columns of the first product: queries (or their latent), the key/value latent, the rotated key, the gate
        self.q_cols = qr if qr else H * (d + r)
        self.gate_offset = self.q_cols + kr + r
        self.down_cols = self.gate_offset + (H * dv if self.output_gate else 0)
        shapes = {"w_down": (self.down_cols, D), "kv_latent_norm": (kr,), "w_uk": (H * d, kr), "w_uv": (H * dv, kr),
                  "w_o": (D, H * dv)}
        if qr:
            shapes.update({"q_latent_norm": (qr,), "w_uq": (H * (d + r), qr)})
        if params.get("sink") == "learned":
            shapes["sink"] = (H,)
        elif params.get("sink"):
            raise ValueError(f"latent attention: unknown sink '{params.get('sink')}'")
        for name, shape in shapes.items():
            if tuple(weights[name].shape) != shape:
                raise ValueError(f"latent attention: {name} has shape {tuple(weights[name].shape)}, expected {shape}")
        dt, dev = build.compute_dtype, build.device
        self.w_down = Linear(weights["w_down"], dt, dev, tiles=build.weight_tiles)
        self.w_uq = Linear(weights["w_uq"], dt, dev, tiles=build.weight_tiles) if qr else None
        self.w_o = Linear(weights["w_o"], dt, dev, tiles=build.weight_tiles)
        # a matrix per head: the key matrices transposed, [H, kv_rank, dim], so that both are applied as W[h] x
        self.w_uk_t = weights["w_uk"].view(H, d, kr).transpose(1, 2).to(device=dev, dtype=dt).contiguous()
        self.w_uv = weights["w_uv"].view(H, dv, kr).to(device=dev, dtype=dt).contiguous()
        self.q_latent_norm = weights["q_latent_norm"].to(device=dev, dtype=torch.float32).contiguous() if qr else None
        self.kv_latent_norm = weights["kv_latent_norm"].to(device=dev, dtype=torch.float32).contiguous()
        self.sink = weights["sink"].to(device=dev, dtype=torch.float32).contiguous() if "sink" in shapes else None
        self.dtype = dt

    def cache_need(self):
        return CacheNeed(1, self.kv_rank + self.rotary_dim, self.window, value_dim=0)

    def state_need(self):
        return None

    def launch_key(self, ctx, run):
        H, kr, r = self.num_heads, self.kv_rank, self.rotary_dim
        return (run.cache_layer, run.writes_cache) + kernels.attention_rows_launch_key(ctx, H, 1, kr + r, kr, True, self.dtype)

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        T = xn.shape[0]
        H, d, r, dv, qr, kr = self.num_heads, self.head_dim, self.rotary_dim, self.value_dim, self.q_rank, self.kv_rank
        cache, _ = ctx.pages(run.cache_layer)
        tables = ctx.block_tables(run.cache_layer)
        down = ctx.scratch("latent_down", (T, self.down_cols), torch.float32)
        self.w_down.forward(xn, down)
        cq = ctx.scratch("latent_q", (T, qr), self.dtype) if qr else None
        kernels.latent_store(down, 0, self.q_latent_norm, cq, self.q_cols, self.kv_latent_norm, self.q_cols + kr, self.freq,
                             self.amplitude, self.eps, ctx.positions, ctx.row_req, tables, cache, ctx.page_size,
                             write_cache=run.writes_cache)
        if qr:
            q = ctx.scratch("latent_queries", (T, H * (d + r)), torch.float32)
            self.w_uq.forward(cq, q)
        else:
            q = down            # the queries are the first H (dim + rot) columns of the product
        # the queries as the latent rows see them: [W_uk,h^T q_h^p, rotated q_h^r] per head
        qa = ctx.scratch("latent_queries_absorbed", (T, H * (kr + r)), torch.float32)
        kernels.head_product(q, 0, d + r, self.w_uk_t, qa, 0, kr + r, tail=r, freq=self.freq, amplitude=self.amplitude,
                             positions=ctx.positions)
        ol = ctx.scratch("latent_out", (T, H * kr), torch.float32)
        kernels.attention_rows_of_step(ctx, qa, cache, None, ol, tables, H, 1, kr + r, kr, self.scale, self.window, None, None,
                                       self.sink)
        att = ctx.scratch("att", (T, H * dv), self.dtype)
        # the heads' value matrices; the output gate (its values lie in the first product's columns) in the same kernel
        kernels.head_product(ol, 0, kr, self.w_uv, att, 0, dv, gate=down if self.output_gate else None, gate_offset=self.gate_offset)
        self.w_o.forward(att, x, accumulate=True, then=then)
