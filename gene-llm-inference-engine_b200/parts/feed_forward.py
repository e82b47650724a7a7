"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..ops import kernels
from ..ops.linear import Linear
from .registry import register_feed_forward, sub_weights


@register_feed_forward("swiglu")
@register_feed_forward("gated_mlp")
class SwiGLUFeedForward:
    """x += W_down (act(W_gate xn) * (W_up xn)) (src/model/transformer.cpp:437-450).

    Params: ``hidden_size``, ``intermediate_size`` and optionally ``activation`` (one of ``kernels.ACTIVATIONS``: "silu", the
    default; "relu"; "gelu_tanh"; "capped_swish", which is not of the form act(gate) * up, with its bound
    ``activation_limit``) and ``bias`` (every projection has one: z = W u + b). Weights: ``w_gate_up`` [2I, hidden] (gate
    rows first, then up rows) and ``w_down`` [hidden, I]; with ``bias`` also ``b_gate_up`` [2I] and ``b_down`` [hidden]."""

    graph_safe = True      # launches depend only on the step's shape: decode steps may be captured in a CUDA graph


    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.intermediate_size = int(params["intermediate_size"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"gated feed-forward: unknown activation '{self.activation}'")
        self.limit = float(params.get("activation_limit") or 0.0)
        if self.activation == "capped_swish" and not self.limit > 0:
            raise ValueError("gated feed-forward: 'capped_swish' needs a positive activation_limit")
        I, D = self.intermediate_size, self.hidden_size
        if tuple(weights["w_gate_up"].shape) != (2 * I, D):
            raise ValueError(f"swiglu: w_gate_up has shape {tuple(weights['w_gate_up'].shape)}, expected ({2 * I}, {D})")
        if tuple(weights["w_down"].shape) != (D, I):
            raise ValueError(f"swiglu: w_down has shape {tuple(weights['w_down'].shape)}, expected ({D}, {I})")
        self.w_gate_up = Linear(weights["w_gate_up"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_down = Linear(weights["w_down"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.b_gate_up = self.b_down = None
        if params.get("bias"):
            for name, n in (("b_gate_up", 2 * I), ("b_down", D)):
                if weights[name].numel() != n:
                    raise ValueError(f"gated feed-forward: {name} has {weights[name].numel()} values, expected {n}")
            self.b_gate_up = weights["b_gate_up"].reshape(-1).to(device=build.device, dtype=torch.float32).contiguous()
            self.b_down = weights["b_down"].reshape(-1).to(device=build.device, dtype=torch.float32).contiguous()
        self.dtype = build.compute_dtype
        # a block that ends with a kernel of its own over the sublayers' sum may add ``b_down`` there (``leave_output_bias``)
        self.output_bias_left = False

    def leave_output_bias(self):
        """The caller adds the last product's bias itself from now on; returns it (None without one)."""
        self.output_bias_left = self.b_down is not None
        return self.b_down

    @property
    def first_product(self):
        """The Linear of the first product (a block hands it to the mixer that runs before, see AttentionMixer.forward)."""
        return self.w_gate_up

    def launch_key(self, ctx):
        """Its launches depend on the token count only (which the caller's key holds)."""
        return ()

    def forward(self, ctx, xn: torch.Tensor, x: torch.Tensor) -> None:
        T = xn.shape[0]
        h = ctx.scratch("ffn_hidden", (T, self.intermediate_size), self.dtype)
        if self.dtype is torch.bfloat16 and kernels.gemm_swiglu_supported(T, self.intermediate_size, self.hidden_size):
            # activation (and bias) in the product's epilogue
            kernels.gemm_swiglu(xn, self.w_gate_up.weight, h, self.activation, self.limit, self.b_gate_up)
        else:
            gu = ctx.scratch("gate_up", (T, 2 * self.intermediate_size), torch.float32)
            self.w_gate_up.forward(xn, gu)
            if self.activation == "silu" and self.b_gate_up is None:
                kernels.swiglu(gu, h)
            else:
                kernels.gated_act(gu, h, self.activation, self.limit, self.b_gate_up)
        self.w_down.forward(h, x, accumulate=True)
        if self.b_down is not None and not self.output_bias_left:
            kernels.add_bias(x, self.b_down)


@register_feed_forward("routed_experts")
class RoutedExpertsFeedForward:
    """A mixture of small gated feed-forwards of which every token uses ``top``: with z = W_r u in 32-bit and
    s = sigmoid(z), the experts with the largest s_e + ``correction``_e are chosen (the correction steers the choice
    only), and x += sum over the chosen e of s_e * W_down,e (act(W_gate,e u) * (W_up,e u)); the weights s_e are used
    as they are, not renormalised. With ``router`` = "table" nothing is scored: row ``token id`` of ``table`` [vocab, top]
    names the token's experts (different ones), each with weight 1 / top. ``shared``: the params of a gated feed-forward
    that every token runs besides, added to the sum.

    Params: ``hidden_size``, ``intermediate_size`` (of one expert), ``experts``, ``top`` and optionally ``activation``
    ("silu") with ``activation_limit``, ``router`` ("scored", the default, or "table", then with ``vocab_size``), ``shared``.
    Weights: ``router`` [E, hidden] and ``correction`` [E] (scored) or ``table`` [vocab, top] integers, ``w_gate_up``
    [E, 2I, hidden] (an expert's gate rows, then its up rows), ``w_down`` [E, hidden, I], the shared expert's under ``shared.``.

    The step's (token, choice) pairs are bucketed by expert on the device into tiles of rows; each tile runs its
    expert's matrices. Few pairs (decoding) and the 32-bit path: tiles of a few rows on the CUDA cores, the expert
    weights streamed once. Many pairs in bfloat16: the rows are gathered into tiles of 128 in the experts' order and
    the two products run on the tensor cores (the many-token product with a matrix per token tile, the activation in
    the first one's epilogue). The launches depend on the token count only (tiles beyond the step's number are not
    run), so the part is recorded into launch programs and CUDA graphs like the dense one."""

    TC_FROM_PAIRS = 256        # from this many (token, choice) pairs on the tensor-core form runs

    graph_safe = True

    def __init__(self, params, weights, build):
        self.hidden_size, self.intermediate_size = int(params["hidden_size"]), int(params["intermediate_size"])
        self.experts, self.top = int(params["experts"]), int(params["top"])
        self.activation = params.get("activation", "silu")
        if self.activation not in kernels.ACTIVATIONS:
            raise ValueError(f"routed experts: unknown activation '{self.activation}'")
        if not (1 <= self.top <= self.experts):
            raise ValueError(f"routed experts: top {self.top} must lie between 1 and the {self.experts} experts")
        self.limit = float(params.get("activation_limit") or 0.0)
        if self.activation == "capped_swish" and not self.limit > 0:
            raise ValueError("routed experts: 'capped_swish' needs a positive activation_limit")
        self.routing = params.get("router", "scored")
        if self.routing not in ("scored", "table"):
            raise ValueError(f"routed experts: unknown router '{self.routing}' (known: scored, table)")
        E, I, D = self.experts, self.intermediate_size, self.hidden_size
        chooser = (("router", (E, D)), ("correction", (E,))) if self.routing == "scored" else \
            (("table", (int(params["vocab_size"]), self.top)),)
        for name, shape in chooser + (("w_gate_up", (E, 2 * I, D)), ("w_down", (E, D, I))):
            if tuple(weights[name].shape) != shape:
                raise ValueError(f"routed experts: {name} has shape {tuple(weights[name].shape)}, expected {shape}")
        dev, dt = build.device, build.compute_dtype
        self.router = self.correction = self.table = None
        if self.routing == "scored":
            self.router = weights["router"].to(device=dev, dtype=torch.float32).contiguous()
            self.correction = weights["correction"].to(device=dev, dtype=torch.float32).contiguous()
        else:
            table = weights["table"]
            if table.is_floating_point():
                raise ValueError("routed experts: the table of experts must hold integers")
            table = table.to(torch.int64)
            if int(table.min()) < 0 or int(table.max()) >= E:
                raise ValueError(f"routed experts: the table names experts outside 0..{E - 1}")
            ordered = table.sort(dim=1).values
            if self.top > 1 and bool((ordered[:, 1:] == ordered[:, :-1]).any()):
                raise ValueError("routed experts: a row of the table names an expert twice")
            self.table = table.to(device=dev, dtype=torch.int32).contiguous()
        self.shared = None
        if params.get("shared"):
            self.shared = SwiGLUFeedForward(params["shared"], sub_weights(weights, "shared."), build)
        self.w_gate_up = weights["w_gate_up"].to(device=dev, dtype=dt).contiguous()
        self.w_down = weights["w_down"].to(device=dev, dtype=dt).contiguous()
        self.dtype = dt

    def launch_key(self, ctx):
        return ()

    def forward(self, ctx, xn: torch.Tensor, x: torch.Tensor) -> None:
        T = xn.shape[0]
        E, I, D, top = self.experts, self.intermediate_size, self.hidden_size, self.top
        most = getattr(ctx, "max_step_tokens", T)
        if self.dtype is torch.bfloat16 and T * top >= self.TC_FROM_PAIRS and \
                kernels.expert_product_tc_supported(I, D, True) and kernels.expert_product_tc_supported(D, I, False):
            self._forward_tensor_cores(ctx, xn, x, max(most, T))
            return
        tm = kernels.grouped_tile_rows()
        tiles, most_tiles = kernels.route_tiles(T, top, E), kernels.route_tiles(max(most, T), top, E)
        ids = ctx.scratch("route_ids", (T, top), torch.int32)
        weights = ctx.scratch("route_weights", (T, top), torch.float32)
        sorted_rows = ctx.scratch("route_sorted_rows", (tiles * tm,), torch.int32, capacity=most_tiles * tm)
        tile_group = ctx.scratch("route_tile_group", (tiles,), torch.int32, capacity=most_tiles)
        n_tiles = ctx.scratch("route_n_tiles", (1,), torch.int32, capacity=1)
        self._route(ctx, xn, ids, weights, sorted_rows, tile_group, n_tiles)
        hidden = ctx.scratch("expert_hidden", (T * top, I), torch.float32, capacity=max(most, T) * top)
        kernels.expert_product(xn, top, self.w_gate_up, hidden, sorted_rows, tile_group, n_tiles, gated=self.activation,
                               limit=self.limit)
        part = ctx.scratch("expert_out", (T * top, D), torch.float32, capacity=max(most, T) * top)
        kernels.expert_product(hidden, 1, self.w_down, part, sorted_rows, tile_group, n_tiles)
        kernels.route_combine(part, weights, x)
        if self.shared is not None:
            self.shared.forward(ctx, xn, x)

    def _route(self, ctx, xn, ids, weights, sorted_rows, tile_group, n_tiles, **tiles) -> None:
        """The step's (token, choice) pairs and their weights, bucketed by expert."""
        if self.routing == "table":
            kernels.route_table(ctx.tokens, ctx.feedback, self.table, self.experts, ids, weights, sorted_rows, tile_group, n_tiles,
                                **tiles)
        else:
            kernels.route(xn, self.router, self.correction, self.top, ids, weights, sorted_rows, tile_group, n_tiles, **tiles)

    def _forward_tensor_cores(self, ctx, xn: torch.Tensor, x: torch.Tensor, most: int) -> None:
        T = xn.shape[0]
        E, I, D, top = self.experts, self.intermediate_size, self.hidden_size, self.top
        tm = kernels.TC_TILE_ROWS
        tiles, most_tiles = kernels.route_tiles(T, top, E, tm), kernels.route_tiles(most, top, E, tm)
        ids = ctx.scratch("route_ids", (T, top), torch.int32)
        weights = ctx.scratch("route_weights", (T, top), torch.float32)
        sorted_rows = ctx.scratch("route_sorted_rows_tc", (tiles * tm,), torch.int32, capacity=most_tiles * tm)
        tile_group = ctx.scratch("route_tile_group_tc", (tiles,), torch.int32, capacity=most_tiles)
        pair_row = ctx.scratch("route_pair_row", (T * top,), torch.int32, capacity=most * top)
        n_tiles = ctx.scratch("route_n_tiles", (1,), torch.int32, capacity=1)
        self._route(ctx, xn, ids, weights, sorted_rows, tile_group, n_tiles, tile_rows=tm, pair_row=pair_row)
        rows = ctx.scratch("expert_rows", (tiles * tm, D), self.dtype, capacity=most_tiles * tm)
        kernels.gather_rows(xn, top, sorted_rows, n_tiles, tm, rows)
        hidden = ctx.scratch("expert_hidden_tc", (tiles * tm, I), self.dtype, capacity=most_tiles * tm)
        kernels.expert_product_tc(rows, self.w_gate_up, hidden, tile_group, n_tiles, gated=self.activation, limit=self.limit)
        part = ctx.scratch("expert_out_tc", (tiles * tm, D), torch.float32, capacity=most_tiles * tm)
        kernels.expert_product_tc(hidden, self.w_down, part, tile_group, n_tiles)
        kernels.route_combine(part, weights, x, pair_row=pair_row)
        if self.shared is not None:
            self.shared.forward(ctx, xn, x)
