"""The attention mixer: grouped-query causal attention over the paged cache."""
from __future__ import annotations

import torch

from ..cache import CacheNeed, StateNeed
from ..config import PartSpec
from ..ops import kernels
from ..ops.linear import Linear
from .registry import POSITION_ENCODINGS, build_part, register_mixer


@register_mixer("attention")
class AttentionMixer:
    """q, k, v = W_qkv xn; position encoding on q and k; k, v stored in the request's pages;
    causal softmax(q k^T * scale) v per head with query head h reading key/value head
    h // (H / Hkv); x += W_o out (src/model/transformer.cpp:389-434).

    Params: ``hidden_size``, ``num_heads``, ``num_kv_heads``, ``head_dim``, ``scale`` (multiplied
    after the dot product), ``window`` (None = all keys) and ``position`` (a PartSpec).
    Weights: ``w_qkv`` [(H+2Hkv)*hd, hidden] and ``w_o`` [hidden, H*hd].

    Options (each absent by default; any of them takes the mixer off the fused [q; k; v] product with
    rotation in its epilogue and onto the 32-bit projection followed by the norm+rotation+store kernel):
    ``values`` = "keys": the model has no value projection; the value rows written to the pages are the key
    projection's raw output, taken ahead of the per-head norm and the rotation (``w_qkv`` then has no value rows). ``qk_norm_eps``: queries and keys are
    normalised per head to unit RMS and multiplied by ``q_norm`` / ``k_norm`` [hd] (shared by the heads)
    before the rotation. ``sink``: the softmax's denominator has one more term, exp(0). ``head_gate``:
    ``w_qkv`` ends with H more rows, and head h's output is multiplied by the sigmoid of its row's product
    with the input. ``out_scale``: a constant on the mixer's output (applied before the output projection).

    Further options, which run the row-form attention kernel (32-bit arithmetic over shared key tiles):
    ``value_dim``: value heads of a width of their own (``w_qkv`` then has Hkv * value_dim value rows, ``w_o``
    H * value_dim columns, and the values have pages of their own). ``qk_norm_weights`` False: the unit-RMS norm of
    queries and keys has no weights. ``distance_slopes`` [H]: slope_h * (i - j) is taken off the score of key j for the
    query at i. ``chunk``: position i sees j <= i only inside its own block of ``chunk`` positions counted from 0
    (pages of earlier blocks are given back). ``sink`` = "learned": the term added to the softmax's denominator is
    exp(``sink``_h) with a weight per head (``sink`` [H]). ``softcap`` c: the scaled score s becomes c tanh(s / c).

    ``qk_norm_wide`` (with ``qk_norm_eps``): the norm runs over the whole query projection at once (all heads' values
    together, ``q_norm`` [H * hd]) and over the whole key projection (``k_norm`` [Hkv * hd]) instead of head by head.
    ``conv_taps`` n: every channel of the [q; k; v] projection passes a causal convolution over the request's last n
    tokens before anything else (``conv`` [channels, n], column n-1 weighs the newest token; no bias, no activation;
    nothing before the first token; one tap is a factor per channel); the request's last n-1 projected rows are state, kept
    in its state slot from ``state_offset`` on."""

    graph_safe = True      # launches depend only on the step's shape: decode steps may be captured in a CUDA graph


    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.scale = float(params["scale"])
        self.window = params.get("window")
        if self.num_heads % self.num_kv_heads:
            raise ValueError("attention: num_heads must be a multiple of num_kv_heads")
        if not kernels.attention_supported(self.head_dim):
            raise ValueError(f"attention: head size {self.head_dim} is not supported by the attention kernels "
                             f"(up to 256)")
        pos_spec = params.get("position") or PartSpec("none", {})
        self.position = build_part(POSITION_ENCODINGS, "position encoding", pos_spec, {}, build)
        self.values_are_keys = params.get("values", "projected") == "keys"
        if params.get("values", "projected") not in ("projected", "keys"):
            raise ValueError(f"attention: unknown source of values '{params.get('values')}'")
        self.qk_norm_eps = params.get("qk_norm_eps")
        self.value_dim = int(params.get("value_dim") or self.head_dim)
        self.chunk = params.get("chunk")
        self.learned_sink = params.get("sink") == "learned"
        self.softcap = float(params["softcap"]) if params.get("softcap") else None
        if self.softcap is not None and not self.softcap > 0:
            raise ValueError("attention: the soft cap of the scores must be positive")
        self.wide_norm = bool(params.get("qk_norm_wide", False))
        self.conv_taps = int(params["conv_taps"]) if params.get("conv_taps") else None
        self.state_offset = 0
        slopes = params.get("distance_slopes")
        if slopes is not None and len(slopes) != self.num_heads:
            raise ValueError("attention: distance_slopes needs one slope per head")
        self.slopes = None if slopes is None else torch.tensor([float(v) for v in slopes], dtype=torch.float32, device=build.device)
        # these options are served by the row-form kernel only
        self.row_form = (self.value_dim != self.head_dim or self.chunk is not None or self.learned_sink or
                         self.slopes is not None or self.softcap is not None)
        self.sink = bool(params.get("sink", False))
        self.head_gate = bool(params.get("head_gate", False))
        self.out_scale = float(params.get("out_scale", 1.0))
        on_device = getattr(self.position, "freq", None) is not None
        self.extended = (self.values_are_keys or self.qk_norm_eps is not None or self.sink or self.head_gate
                         or self.out_scale != 1.0 or on_device or self.row_form or self.conv_taps is not None)
        if self.row_form:
            if self.head_gate or self.out_scale != 1.0 or self.values_are_keys:
                raise ValueError("attention: a gate, an output factor or values taken from the keys cannot be combined with "
                                 "value_dim, chunk, distance_slopes, a soft cap or a learned sink")
            if not kernels.attention_rows_supported(self.head_dim, self.value_dim):
                raise ValueError(f"attention: head size {self.head_dim} with value size {self.value_dim} is not supported")
        if getattr(self.position, "amplitude", 1.0) != 1.0:
            raise ValueError("attention: a rotation whose cos and sin are scaled is not served by this mixer")
        self.sink_weight = None
        if self.learned_sink:
            if tuple(weights["sink"].shape) != (self.num_heads,):
                raise ValueError(f"attention: sink has shape {tuple(weights['sink'].shape)}, expected ({self.num_heads},)")
            self.sink_weight = weights["sink"].to(device=build.device, dtype=torch.float32).contiguous()
        elif self.row_form and self.sink:
            self.sink_weight = torch.zeros(self.num_heads, dtype=torch.float32, device=build.device)      # exp(0) = 1
        if self.extended and getattr(self.position, "cos", None) is not None:
            raise ValueError("attention: with these options the rotation's angles are computed on the device "
                             "(position encoding 'rope_on_device' or 'none')")
        # soft-capped scores alone (equal key and value sizes, nothing else of the row form): prompt portions may run on the
        # tcgen05 kernel and single tokens on the decode kernel, which have the cap
        self.cap_only = (self.softcap is not None and self.value_dim == self.head_dim and self.chunk is None and self.slopes is None
                         and not self.learned_sink and not params.get("sink") and build.compute_dtype is torch.bfloat16)
        self.q_norm = self.k_norm = None
        if self.qk_norm_eps is not None and not params.get("qk_norm_weights", True):
            self.q_norm = self.k_norm = torch.ones(self.head_dim, dtype=torch.float32, device=build.device)
        elif self.qk_norm_eps is not None:
            for name, heads in (("q_norm", self.num_heads), ("k_norm", self.num_kv_heads)):
                n = heads * self.head_dim if self.wide_norm else self.head_dim
                if tuple(weights[name].shape) != (n,):
                    raise ValueError(f"attention: {name} has shape {tuple(weights[name].shape)}, expected ({n},)")
                setattr(self, name, weights[name].to(device=build.device, dtype=torch.float32).contiguous())
        if self.wide_norm and (self.qk_norm_eps is None or not params.get("qk_norm_weights", True)):
            raise ValueError("attention: qk_norm_wide needs qk_norm_eps and weights")
        qkv_rows = (self.num_heads + self.num_kv_heads) * self.head_dim + \
            (0 if self.values_are_keys else self.num_kv_heads * self.value_dim) + (self.num_heads if self.head_gate else 0)
        if tuple(weights["w_qkv"].shape) != (qkv_rows, self.hidden_size):
            raise ValueError(f"attention: w_qkv has shape {tuple(weights['w_qkv'].shape)}, expected "
                             f"({qkv_rows}, {self.hidden_size})")
        if tuple(weights["w_o"].shape) != (self.hidden_size, self.num_heads * self.value_dim):
            raise ValueError(f"attention: w_o has shape {tuple(weights['w_o'].shape)}")
        self.conv = None
        if self.conv_taps is not None:
            if self.head_gate or self.values_are_keys:
                raise ValueError("attention: a convolution of the projections cannot be combined with a head gate or values taken from the keys")
            if not (self.conv_taps <= 17):
                raise ValueError(f"attention: {self.conv_taps} convolution taps are not supported (1 to 17)")
            if tuple(weights["conv"].shape) != (qkv_rows, self.conv_taps):
                raise ValueError(f"attention: conv has shape {tuple(weights['conv'].shape)}, expected ({qkv_rows}, {self.conv_taps})")
            self.conv = weights["conv"].to(device=build.device, dtype=torch.float32).contiguous()
            self.conv_channels = qkv_rows
        self.w_qkv = Linear(weights["w_qkv"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_o = Linear(weights["w_o"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.dtype = build.compute_dtype
        # bfloat16 with a head size the tensor-core kernels are built for; else the general kernel
        self.fast = self.dtype is torch.bfloat16 and not self.row_form and kernels.attention_fast_supported(
            self.head_dim, self.num_heads, self.num_kv_heads)
        self._prefill_rows = {}
        self.cap_fast = self.cap_only and kernels.attention_fast_supported(self.head_dim, self.num_heads, self.num_kv_heads)
        if self.fast or self.cap_fast:
            self.chunk_keys = kernels.attention_chunk_keys()
            self.max_chunks = (build.max_position + self.chunk_keys - 1) // self.chunk_keys

    def prefill_on_tcgen05(self, page_size: int) -> bool:
        """Head sizes 64 and 128 with pages TMA can tile: prompt portions run on the tcgen05 kernel."""
        key = ("tc", page_size)
        if key not in self._prefill_rows:
            self._prefill_rows[key] = kernels.attention_prefill_tc_supported(self.head_dim, self.num_heads,
                                                                             self.num_kv_heads, page_size)
        return self._prefill_rows[key]

    def prefill_rows(self, page_size: int) -> int:
        """Query rows (tokens x heads of a group) per work item of the prefill kernel in use."""
        if page_size not in self._prefill_rows:
            self._prefill_rows[page_size] = 128 if self.prefill_on_tcgen05(page_size) else \
                kernels.attention_prefill_rows(page_size, self.head_dim)
        return self._prefill_rows[page_size]

    def cache_need(self):
        return CacheNeed(self.num_kv_heads, self.head_dim, self.window,
                         value_dim=None if self.value_dim == self.head_dim else self.value_dim, chunk=self.chunk)

    def state_need(self):
        if self.conv is None or self.conv_taps == 1:
            return None
        return StateNeed(((self.conv_taps - 1) * self.conv_channels,), "float32")

    def launch_key(self, ctx, run):
        key = self._launch_key(ctx, run)
        return key + (ctx.n_requests,) if self.conv is not None else key

    def _launch_key(self, ctx, run):
        """What the mixer's launches depend on besides the token count: whose cache it uses, and (tensor-core
        kernels) how many rows are single decoded tokens, how many tiles the prompt portions make and how many
        chunks the longest context of a single token has. Asking also places this step's work lists on the device."""
        if self.row_form:
            key = (run.cache_layer, run.writes_cache) + kernels.attention_rows_launch_key(
                ctx, self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, False, self.dtype)
            if self._cap_tiles_on_tcgen05(ctx):
                key += (ctx.attention_work(128 // (self.num_heads // self.num_kv_heads))[1].shape[0],)
            if self._cap_singles_on_decode(ctx):
                per_tile = kernels.attention_rows_tile_tokens(self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, False)
                key += ((ctx.attention_work(per_tile)[2] + self.chunk_keys - 1) // self.chunk_keys,)
            return key
        if not self._fast_now(ctx):
            return (run.cache_layer, run.writes_cache)
        rows, work, longest = ctx.attention_work(self.prefill_rows(ctx.page_size) // (self.num_heads // self.num_kv_heads))
        return (run.cache_layer, run.writes_cache, rows.numel(), work.shape[0],
                (longest + self.chunk_keys - 1) // self.chunk_keys)

    takes_then = True      # forward accepts ``then``

    def _cap_singles_on_decode(self, ctx) -> bool:
        return (self.cap_fast and hasattr(ctx, "attention_work") and kernels.attention_tma_pages(ctx.page_size)
                and kernels.attention_rows_tile_tokens(self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, False) > 0)

    def _cap_tiles_on_tcgen05(self, ctx) -> bool:
        return (self.cap_only and hasattr(ctx, "attention_work") and self.prefill_on_tcgen05(ctx.page_size)
                and kernels.attention_rows_tile_tokens(self.num_heads, self.num_kv_heads, self.head_dim, self.value_dim, False) > 0)

    def _fast_now(self, ctx) -> bool:
        """Whether this step's attention runs on the tensor-core kernels: bfloat16 with a head size they are built for;
        with a sink, a gate or an output factor also pages that their TMA-fed forms can tile."""
        return self.fast and (not self.extended or kernels.attention_tma_pages(ctx.page_size))

    def _attend(self, ctx, q, k_cache, v_cache, att, tables, **epilogue) -> None:
        """Attention of the step's rows: single decoded tokens split their context over many CTAs, portions of
        prompts run tile by tile (tensor cores); else the general kernel. ``epilogue``: sink, gate, gate_offset, out_scale."""
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        if not self._fast_now(ctx):
            kernels.attention_generic(q, k_cache, v_cache, att, ctx.row_req, ctx.positions, tables, H, Hkv, hd,
                                      ctx.page_size, self.scale, self.window, **epilogue)
            return
        rows, work, longest = ctx.attention_work(self.prefill_rows(ctx.page_size) // (H // Hkv))
        if rows.numel():
            n = rows.numel()
            part_o = ctx.scratch("att_part_o", (n, H * self.max_chunks * hd), torch.float32, capacity=ctx.max_requests)
            part_ml = ctx.scratch("att_part_ml", (n, H * self.max_chunks * 2), torch.float32, capacity=ctx.max_requests)
            n_chunks = (longest + self.chunk_keys - 1) // self.chunk_keys
            kernels.attention_decode(q, k_cache, v_cache, att, rows, ctx.row_req, ctx.positions, tables, H, Hkv, hd,
                                     ctx.page_size, self.scale, self.window, part_o, part_ml, self.max_chunks, n_chunks,
                                     **epilogue)
        if work.shape[0]:
            prefill = kernels.attention_prefill_tc if self.prefill_on_tcgen05(ctx.page_size) else kernels.attention_prefill
            prefill(q, k_cache, v_cache, att, work, ctx.positions, tables, H, Hkv, hd, ctx.page_size, self.scale,
                    self.window, **epilogue)

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        """``xn``: normalised input [T, hidden] in the compute dtype; ``x``: the 32-bit residual
        stream, to which the mixer's output is added. ``run`` names whose cache to use. ``then``: the Linear
        of the large product that follows this mixer (the feed-forward's first), for the last product here to
        ask the start of its weights into L2."""
        T = xn.shape[0]
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        k_cache, v_cache = ctx.pages(run.cache_layer)
        tables = ctx.block_tables(run.cache_layer)
        q = ctx.scratch("q", (T, H * hd), self.dtype)
        if self.extended:
            self._forward_extended(ctx, run, xn, x, q, k_cache, v_cache, tables, then)
            return
        if self.dtype is torch.bfloat16 and kernels.gemm_rope_store_supported(
                T, self.hidden_size, H, Hkv, hd, self.position.cos, self.position.interleaved):
            # rotation and page store in the epilogue of the product
            kernels.gemm_rope_store(xn, self.w_qkv.weight, ctx.positions, ctx.row_req, tables, self.position.cos,
                                    self.position.sin, self.position.interleaved, q, k_cache, v_cache, H, Hkv, hd,
                                    ctx.page_size, write_kv=run.writes_cache, w_tiles=self.w_qkv.weight_tiles)
        else:
            qkv = ctx.scratch("qkv", (T, (H + 2 * Hkv) * hd), torch.float32)
            self.w_qkv.forward(xn, qkv)
            kernels.rope_store(qkv, ctx.positions, ctx.row_req, tables, self.position.cos, self.position.sin,
                               self.position.interleaved, q, k_cache, v_cache, H, Hkv, hd, ctx.page_size,
                               write_kv=run.writes_cache)
        att = ctx.scratch("att", (T, H * hd), self.dtype)
        self._attend(ctx, q, k_cache, v_cache, att, tables)
        self.w_o.forward(att, x, accumulate=True, then=then)

    def _forward_extended(self, ctx, run, xn, x, q, k_cache, v_cache, tables, then) -> None:
        """The mixer with options: projections to 32-bit, then per head norm, rotation and page store, attention
        with sink and gate in its epilogue, and the output projection."""
        T = xn.shape[0]
        H, Hkv, hd = self.num_heads, self.num_kv_heads, self.head_dim
        proj = ctx.scratch("att_proj", (T, self.w_qkv.out_features), torch.float32)
        self.w_qkv.forward(xn, proj)
        if self.conv is not None:
            mixed = ctx.scratch("att_proj_conv", (T, self.conv_channels), torch.float32)
            state = ctx.state(run.cache_layer) if self.conv_taps > 1 else mixed      # one tap reaches no earlier token: no state is touched
            kernels.causal_conv(proj, 0, self.conv, None, state, self.state_offset if self.conv_taps > 1 else 0, ctx.row_req,
                                ctx.seg_start, ctx.seg_len, ctx.state_slots, mixed, activate=False)
            proj = mixed
        k_off = H * hd
        v_off = k_off if self.values_are_keys else k_off + Hkv * hd
        gate_off = v_off + Hkv * hd
        kernels.norm_rope_store(proj, 0, k_off, v_off, self.q_norm, self.k_norm, self.qk_norm_eps or 0.0,
                                getattr(self.position, "freq", None), self.position.interleaved, ctx.positions,
                                ctx.row_req, tables, q, k_cache, v_cache, H, Hkv, hd, ctx.page_size,
                                write_kv=run.writes_cache, value_dim=self.value_dim, wide_norm=self.wide_norm)
        if self.row_form:
            att = ctx.scratch("att", (T, H * self.value_dim), self.dtype)
            tiles_on = None
            if self._cap_tiles_on_tcgen05(ctx):
                tiles_on = (128 // (H // Hkv), lambda work: kernels.attention_prefill_tc(
                    q, k_cache, v_cache, att, work, ctx.positions, tables, H, Hkv, hd, ctx.page_size, self.scale, self.window,
                    softcap=self.softcap))
            singles_on = None
            if self._cap_singles_on_decode(ctx):
                def singles_on(rows, longest):
                    n = rows.numel()
                    part_o = ctx.scratch("att_part_o", (n, H * self.max_chunks * hd), torch.float32, capacity=ctx.max_requests)
                    part_ml = ctx.scratch("att_part_ml", (n, H * self.max_chunks * 2), torch.float32, capacity=ctx.max_requests)
                    kernels.attention_decode(q, k_cache, v_cache, att, rows, ctx.row_req, ctx.positions, tables, H, Hkv, hd,
                                             ctx.page_size, self.scale, self.window, part_o, part_ml, self.max_chunks,
                                             (longest + self.chunk_keys - 1) // self.chunk_keys, softcap=self.softcap)
            kernels.attention_rows_of_step(ctx, q, k_cache, v_cache, att, tables, H, Hkv, hd, self.value_dim, self.scale,
                                           self.window, self.chunk, self.slopes, self.sink_weight, softcap=self.softcap,
                                           tiles_on=tiles_on, singles_on=singles_on)
            self.w_o.forward(att, x, accumulate=True, then=then)
            return
        att = ctx.scratch("att", (T, H * hd), self.dtype)
        self._attend(ctx, q, k_cache, v_cache, att, tables, sink=self.sink, gate=proj if self.head_gate else None,
                     gate_offset=gate_off, out_scale=self.out_scale)
        self.w_o.forward(att, x, accumulate=True, then=then)
