"""Mixers that keep a state of fixed size per request instead of keys and values.

All run the same recurrence kernel, M_t = a_t M_(t-1) + b_t k_t (x) v_t and y_t = M_t^T q_t (+ skip v_t), per
head over each request's rows in order, with the 32-bit state [H, dk, dv] in the request's state slot
(``ctx.state(layer)[slot]``; the engine hands a new request a zeroed slot). They differ in where q, k, v, a and
b come from (a may be a number per head, per head and token, or per row of M and token) and in the gated norm
that follows. A mixer's state begins at ``state_offset`` floats into the slot (0 unless a mixer that holds several
state-keeping mixers moves it).
"""
from __future__ import annotations

import torch

from ..cache import StateNeed
from ..ops import kernels
from ..ops.linear import Linear
from .registry import register_mixer


def _scan_workspaces(ctx, T: int, H: int, dk: int, dv: int, row_decays: bool = False):
    """(part_len, ws_state, ws_decay) for a step's recurrence: segments that fit one part run in one launch on the
    state slot itself; longer ones are cut into parts that run side by side (kernels.linear_scan). ``row_decays``:
    the running products of the decays are kept per row of the state."""
    if T <= kernels.SCAN_PART:
        return {}
    R = ctx.n_requests
    parts = kernels.scan_parts(T, R)
    most = getattr(ctx, "max_step_tokens", T) // kernels.SCAN_PART + ctx.max_requests
    ws_state = ctx.scratch("scan_part_states", (parts, H * dk * dv), torch.float32, capacity=max(parts, most))
    ws_decay = ctx.scratch("scan_row_decays" if row_decays else "scan_decays", (T, H * dk if row_decays else H), torch.float32)
    return {"part_len": kernels.SCAN_PART, "ws_state": ws_state, "ws_decay": ws_decay}


def _vector(weights, name: str, n: int, build, what: str) -> torch.Tensor:
    w = weights[name]
    if w.numel() != n or w.dim() != 1:
        raise ValueError(f"{what}: {name} has shape {tuple(w.shape)}, expected ({n},)")
    return w.to(device=build.device, dtype=torch.float32).contiguous()


@register_mixer("linear_attention")
class LinearAttentionMixer:
    """Linear attention whose memory fades by a fixed factor per head. With u the input row, phi the activation and
    lambda_h the head's factor:  q = phi(Wq u), k = phi(Wk u) (H heads of dk), v = phi(Wv u) (H heads of dv);
    M_t = lambda_h M_(t-1) + k_t (x) v_t  (a dk x dv matrix per head, (x) the outer product);  y_t = M_t^T q_t, unscaled.
    All heads' y side by side are brought to unit RMS as one vector, weighted by ``norm`` [H dv], gated elementwise
    by sigmoid(Wg u) and sent through ``w_o``.

    Params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``decay`` (lambda, one per head), ``norm_eps``,
    ``activation`` ("silu" or "none") and optionally ``out_scale``. Weights: ``w_in`` [(2 H dk + 2 H dv), hidden]
    (rows of Wq, Wk, Wv, Wg in this order), ``w_o`` [hidden, H dv], ``norm`` [H dv]."""

    graph_safe = True

    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads, self.dk, self.dv = int(params["num_heads"]), int(params["key_dim"]), int(params["value_dim"])
        self.eps = float(params["norm_eps"])
        self.activate = params.get("activation", "silu") == "silu"
        if params.get("activation", "silu") not in ("silu", "none"):
            raise ValueError(f"linear attention: unknown activation '{params.get('activation')}'")
        self.out_scale = float(params.get("out_scale", 1.0))
        decay = [float(d) for d in params["decay"]]
        if len(decay) != self.num_heads:
            raise ValueError("linear attention: one decay per head is needed")
        if self.dk > 256:
            raise ValueError(f"linear attention: key size {self.dk} exceeds what the recurrence kernel holds (256)")
        H, dk, dv, D = self.num_heads, self.dk, self.dv, self.hidden_size
        self.decay = torch.tensor(decay, dtype=torch.float32, device=build.device)
        rows = 2 * H * dk + 2 * H * dv
        if tuple(weights["w_in"].shape) != (rows, D):
            raise ValueError(f"linear attention: w_in has shape {tuple(weights['w_in'].shape)}, expected ({rows}, {D})")
        if tuple(weights["w_o"].shape) != (D, H * dv):
            raise ValueError(f"linear attention: w_o has shape {tuple(weights['w_o'].shape)}, expected ({D}, {H * dv})")
        self.w_in = Linear(weights["w_in"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_o = Linear(weights["w_o"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.norm = _vector(weights, "norm", H * dv, build, "linear attention")
        self.dtype = build.compute_dtype
        self.state_offset = 0

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.num_heads * self.dk * self.dv,), "float32")

    def launch_key(self, ctx, run):
        return (run.cache_layer, ctx.n_requests)

    takes_then = True

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        T = xn.shape[0]
        H, dk, dv = self.num_heads, self.dk, self.dv
        proj = ctx.scratch("lin_att_proj", (T, self.w_in.out_features), torch.float32)
        self.w_in.forward(xn, proj)
        o = ctx.scratch("lin_att_out", (T, H * dv), torch.float32)
        kernels.linear_scan(proj, 0, proj, H * dk, proj, 2 * H * dk, H, 1, dk, dv, self.activate,
                            ctx.state(run.cache_layer), self.state_offset, ctx.seg_start, ctx.seg_len, ctx.state_slots, o, decay=self.decay,
                            **_scan_workspaces(ctx, T, H, dk, dv))
        y = ctx.scratch("lin_att_normed", (T, H * dv), self.dtype)
        kernels.gated_group_norm(o, proj, 2 * H * dk + H * dv, self.norm, y, 1, self.eps, gate_first=False,
                                 out_scale=self.out_scale)
        self.w_o.forward(y, x, accumulate=True, then=then)


@register_mixer("state_space")
class StateSpaceMixer:
    """A selective state-space mixer whose decay is one number per head and token. ``w_in`` gives, per token, five
    blocks in this order: a gate z (H P values), the signal u (H P), an input map B (G N), a read-out map C (G N) and a
    raw step r (H). u, B and C go through a depthwise convolution over the last ``conv_taps`` tokens of the request
    (``conv`` [channels, taps], column taps-1 weighs the newest token; ``conv_bias``; nothing before the first token)
    followed by SiLU. With delta = softplus(r + ``dt_bias``) (no upper bound) and rho_h = exp(``a_log``_h), head h
    (which shares B and C with the heads of its group, G groups of H / G heads) keeps an N x P matrix:
    M_t = exp(-rho_h delta_t) M_(t-1) + delta_t B_t (x) u_t;  y_t = M_t^T C_t + ``skip``_h u_t.
    y is gated by SiLU(z) first and only then brought to unit RMS, separately in each of ``norm_groups`` equal
    slices, weighted by ``norm`` and sent through ``w_o``. A request's state slot holds M and, behind it, the
    convolution's last taps-1 inputs [taps-1, channels].

    Params: ``hidden_size``, ``num_heads`` (H), ``head_dim`` (P), ``state_size`` (N), ``groups`` (G), ``conv_taps``,
    ``norm_groups``, ``norm_eps`` and optionally ``out_scale``."""

    graph_safe = True

    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads, self.head_dim = int(params["num_heads"]), int(params["head_dim"])
        self.state_size, self.groups = int(params["state_size"]), int(params["groups"])
        self.taps, self.norm_groups = int(params["conv_taps"]), int(params["norm_groups"])
        self.eps = float(params["norm_eps"])
        self.out_scale = float(params.get("out_scale", 1.0))
        H, P, N, G, D = self.num_heads, self.head_dim, self.state_size, self.groups, self.hidden_size
        if H % G:
            raise ValueError("state space: heads must be a multiple of groups")
        if N > 256:
            raise ValueError(f"state space: state size {N} exceeds what the recurrence kernel holds (256)")
        if not (1 <= self.taps <= 17):
            raise ValueError(f"state space: {self.taps} convolution taps are not supported (1 to 17)")
        self.inner = H * P
        self.channels = self.inner + 2 * G * N
        if self.inner % self.norm_groups:
            raise ValueError("state space: heads * head_dim must split into norm_groups equal parts")
        rows = 2 * self.inner + 2 * G * N + H
        if tuple(weights["w_in"].shape) != (rows, D):
            raise ValueError(f"state space: w_in has shape {tuple(weights['w_in'].shape)}, expected ({rows}, {D})")
        if tuple(weights["w_o"].shape) != (D, self.inner):
            raise ValueError(f"state space: w_o has shape {tuple(weights['w_o'].shape)}, expected ({D}, {self.inner})")
        if tuple(weights["conv"].shape) != (self.channels, self.taps):
            raise ValueError(f"state space: conv has shape {tuple(weights['conv'].shape)}, expected ({self.channels}, {self.taps})")
        self.w_in = Linear(weights["w_in"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_o = Linear(weights["w_o"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.conv = weights["conv"].to(device=build.device, dtype=torch.float32).contiguous()
        self.conv_bias = _vector(weights, "conv_bias", self.channels, build, "state space")
        self.dt_bias = _vector(weights, "dt_bias", H, build, "state space")
        self.a_log = _vector(weights, "a_log", H, build, "state space")
        self.skip = _vector(weights, "skip", H, build, "state space")
        self.norm = _vector(weights, "norm", self.inner, build, "state space")
        self.dtype = build.compute_dtype
        self.state_offset = 0

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.num_heads * self.state_size * self.head_dim + (self.taps - 1) * self.channels,), "float32")

    def launch_key(self, ctx, run):
        return (run.cache_layer, ctx.n_requests)

    takes_then = True

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        T = xn.shape[0]
        H, P, N, G = self.num_heads, self.head_dim, self.state_size, self.groups
        inner, C = self.inner, self.channels
        state = ctx.state(run.cache_layer)
        proj = ctx.scratch("ssm_proj", (T, self.w_in.out_features), torch.float32)
        self.w_in.forward(xn, proj)
        xbc = ctx.scratch("ssm_conv", (T, C), torch.float32)
        kernels.causal_conv(proj, inner, self.conv, self.conv_bias, state, self.state_offset + H * N * P, ctx.row_req, ctx.seg_start,
                            ctx.seg_len, ctx.state_slots, xbc)
        y = ctx.scratch("ssm_out", (T, inner), torch.float32)
        # q = C, k = B, v = x; a and b from the step size
        kernels.linear_scan(xbc, inner + G * N, xbc, inner, xbc, 0, H, H // G, N, P, False, state, self.state_offset, ctx.seg_start,
                            ctx.seg_len, ctx.state_slots, y, dt=proj, dt_offset=inner + C, dt_bias=self.dt_bias,
                            a_log=self.a_log, skip=self.skip, **_scan_workspaces(ctx, T, H, N, P))
        yn = ctx.scratch("ssm_normed", (T, inner), self.dtype)
        kernels.gated_group_norm(y, proj, 0, self.norm, yn, self.norm_groups, self.eps, gate_first=True,
                                 out_scale=self.out_scale)
        self.w_o.forward(yn, x, accumulate=True, then=then)


@register_mixer("gated_linear_attention")
class GatedLinearAttentionMixer:
    """Linear attention whose memory fades by a factor of its own per key channel and token. With u the input row:
    q = c Wq u (c = ``query_scale``), k = Wk u (H heads of dk), v = Wv u (H heads of dv); z = W2 (W1 u) + b (a product
    through ``decay_rank`` values) gives alpha = sigmoid(z)^(1 / ``tau``) per head and key channel;
    M_t = diag(alpha_t) M_(t-1) + k_t (x) v_t  (a dk x dv matrix per head);  y_t = M_t^T q_t.
    Each head's y is brought to unit RMS over its dv values, weighted by ``norm`` [dv] (one weight for all heads), all
    heads side by side are multiplied by SiLU(Wg u) and sent through ``w_o``. alpha, the recurrence and its state are
    32-bit; W1 u is handed to the second product in the compute dtype.

    Params: ``hidden_size``, ``num_heads``, ``key_dim``, ``value_dim``, ``tau``, ``norm_eps`` and optionally ``decay_rank``
    (as ``w_a1`` has rows when absent), ``query_scale`` (key_dim^-0.5) and ``out_scale``. Weights: ``w_in`` [(2 H dk + 2 H dv), hidden] (rows of Wq, Wk, Wv, Wg
    in this order), ``w_a1`` [rank, hidden], ``w_a2`` [H dk, rank], ``a2_bias`` [H dk], ``norm`` [dv], ``w_o`` [hidden, H dv]."""

    graph_safe = True

    def __init__(self, params, weights, build):
        self.hidden_size = int(params["hidden_size"])
        self.num_heads, self.dk, self.dv = int(params["num_heads"]), int(params["key_dim"]), int(params["value_dim"])
        # the rank of the decay's projection: given, or as the weights' shapes say
        self.tau, self.rank = float(params["tau"]), int(params.get("decay_rank") or weights["w_a1"].shape[0])
        self.eps = float(params["norm_eps"])
        self.q_scale = float(params.get("query_scale", self.dk ** -0.5))
        self.out_scale = float(params.get("out_scale", 1.0))
        if not self.tau > 0:
            raise ValueError("gated linear attention: tau must be positive")
        if self.dk > 256:
            raise ValueError(f"gated linear attention: key size {self.dk} exceeds what the recurrence kernel holds (256)")
        H, dk, dv, D = self.num_heads, self.dk, self.dv, self.hidden_size
        for name, shape in (("w_in", (2 * H * dk + 2 * H * dv, D)), ("w_a1", (self.rank, D)), ("w_a2", (H * dk, self.rank)),
                            ("w_o", (D, H * dv))):
            if tuple(weights[name].shape) != shape:
                raise ValueError(f"gated linear attention: {name} has shape {tuple(weights[name].shape)}, expected {shape}")
        self.w_in = Linear(weights["w_in"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_a1 = Linear(weights["w_a1"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_a2 = Linear(weights["w_a2"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.w_o = Linear(weights["w_o"], build.compute_dtype, build.device, tiles=build.weight_tiles)
        self.a2_bias = _vector(weights, "a2_bias", H * dk, build, "gated linear attention")
        self.norm = _vector(weights, "norm", dv, build, "gated linear attention").repeat(H).contiguous()
        self.dtype = build.compute_dtype
        self.state_offset = 0

    def cache_need(self):
        return None

    def state_need(self):
        return StateNeed((self.num_heads * self.dk * self.dv,), "float32")

    def launch_key(self, ctx, run):
        return (run.cache_layer, ctx.n_requests)

    takes_then = True

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        T = xn.shape[0]
        H, dk, dv = self.num_heads, self.dk, self.dv
        proj = ctx.scratch("gla_proj", (T, self.w_in.out_features), torch.float32)
        self.w_in.forward(xn, proj)
        low = ctx.scratch("gla_decay_low", (T, self.rank), self.dtype)
        self.w_a1.forward(xn, low)
        z = ctx.scratch("gla_decay_z", (T, H * dk), torch.float32)
        self.w_a2.forward(low, z)
        o = ctx.scratch("gla_out", (T, H * dv), torch.float32)
        kernels.linear_scan(proj, 0, proj, H * dk, proj, 2 * H * dk, H, 1, dk, dv, False, ctx.state(run.cache_layer),
                            self.state_offset, ctx.seg_start, ctx.seg_len, ctx.state_slots, o, row_gate=z,
                            row_gate_bias=self.a2_bias, tau=self.tau, q_scale=self.q_scale,
                            **_scan_workspaces(ctx, T, H, dk, dv, row_decays=True))
        y = ctx.scratch("gla_normed", (T, H * dv), self.dtype)
        kernels.gated_group_norm(o, proj, 2 * H * dk + H * dv, self.norm, y, H, self.eps, gate_first=False, gate_act="silu",
                                 out_scale=self.out_scale)
        self.w_o.forward(y, x, accumulate=True, then=then)


@register_mixer("parallel")
class ParallelMixer:
    """Several mixers side by side on the same input. ``combine`` "sum" (the default): x += sum_i scale_i * mixer_i(xn).
    ``combine`` "mean_normed": every branch's output is first brought to unit RMS over the model width and weighted by
    its own ``<name>_out`` [hidden] (eps ``combine_eps``), and x += (1 / n) sum_i of these. Params: ``branches``, a list of
    (name, PartSpec, scale); branch ``name`` is built from the weights under ``<name>.`` with its scale as ``out_scale``.
    At most one branch may keep pages; the states of branches that keep one lie behind one another in the layer's slot."""

    def __init__(self, params, weights, build):
        from ..config import PartSpec
        from .registry import MIXERS, build_part, sub_weights
        self.branches = []
        self.combine = params.get("combine", "sum")
        if self.combine not in ("sum", "mean_normed"):
            raise ValueError(f"parallel mixer: unknown way to combine the branches '{self.combine}'")
        for name, spec, scale in params["branches"]:
            spec = PartSpec(spec.kind, dict(spec.params, out_scale=float(scale)))
            self.branches.append((name, build_part(MIXERS, "mixer", spec, sub_weights(weights, name + "."), build)))
        if sum(m.cache_need() is not None for _, m in self.branches) > 1:
            raise ValueError("parallel mixer: at most one branch may keep pages")
        self._state_size = 0
        for name, m in self.branches:
            need = m.state_need()
            if need is None:
                continue
            if need.dtype != "float32" or len(need.shape) != 1 or not hasattr(m, "state_offset"):
                raise ValueError(f"parallel mixer: the state of branch '{name}' cannot be laid behind another's")
            m.state_offset = self._state_size
            self._state_size += (need.shape[0] + 3) // 4 * 4          # every branch's state starts on 16 bytes
        for name, m in self.branches:
            setattr(self, name, m)
        self.graph_safe = all(getattr(m, "graph_safe", False) for _, m in self.branches)
        self.out_norms = None
        if self.combine == "mean_normed":
            self.eps = float(params["combine_eps"])
            self.hidden_size = int(params["hidden_size"])
            self.out_norms = []
            for name, _ in self.branches:
                w = weights[name + "_out"]
                if tuple(w.shape) != (self.hidden_size,):
                    raise ValueError(f"parallel mixer: {name}_out has shape {tuple(w.shape)}, expected ({self.hidden_size},)")
                # the mean's factor goes into the weight once, in 32-bit
                self.out_norms.append((w.to(device=build.device, dtype=torch.float32) / len(self.branches)).contiguous())

    def cache_need(self):
        return next((m.cache_need() for _, m in self.branches if m.cache_need() is not None), None)

    def state_need(self):
        return StateNeed((self._state_size,), "float32") if self._state_size else None

    def launch_key(self, ctx, run):
        key = ()
        for _, m in self.branches:
            fn = getattr(m, "launch_key", None)
            k = fn(ctx, run) if fn is not None else None
            if k is None:
                return None
            key += tuple(k)
        if self.combine == "mean_normed":
            # decided here, once per run and before it: a run that is repeated from its launch program does not pass through
            # ``forward``, and the next mixer of this kind must still learn that the sums are zero after this one
            sums = self._sums(ctx, ctx.n_tokens)
            clear = self._sums_clear(ctx, sums)
            if getattr(ctx, "carry", None) is not None:
                ctx.carry["parallel_branch_decided"] = (id(self), run.cache_layer, clear)
                ctx.carry["parallel_branch_sums"] = tuple(t.data_ptr() for t in sums)
            key += (clear,)
        return key

    takes_then = True

    def _sums(self, ctx, T: int):
        return [ctx.scratch(f"parallel_branch_{i}", (T, self.hidden_size), torch.float32) for i in range(len(self.branches))]

    def _sums_clear(self, ctx, sums) -> bool:
        """Whether the branches' own sums are known to be zero (the mixer of this kind that ran before in this step left these
        very buffers so)."""
        carry = getattr(ctx, "carry", None)
        return bool(carry is not None and carry.get("parallel_branch_sums") == tuple(t.data_ptr() for t in sums))

    def forward(self, ctx, run, xn: torch.Tensor, x: torch.Tensor, then=None) -> None:
        if self.combine == "mean_normed":
            # every branch adds into a sum of its own, which the combining kernel norms, adds to x and clears again
            sums = self._sums(ctx, xn.shape[0])
            carry = getattr(ctx, "carry", None)
            decided = carry.get("parallel_branch_decided") if carry is not None else None
            if decided is not None and decided[:2] == (id(self), run.cache_layer):
                clear = decided[2]                       # ``launch_key`` looked before it marked the sums as zero
            else:
                clear = self._sums_clear(ctx, sums)
            for (_, m), own in zip(self.branches, sums):
                if not clear:
                    kernels.scale_cast(x, own, None, 0.0)
                m.forward(ctx, run, xn, own)
            for own, w in zip(sums, self.out_norms):
                kernels.add_normed(own, w, x, self.eps, clear_y=True)
            if carry is not None:
                carry["parallel_branch_sums"] = tuple(t.data_ptr() for t in sums)
            return
        for i, (_, m) in enumerate(self.branches):
            last = i == len(self.branches) - 1
            if last and then is not None and getattr(m, "takes_then", False):
                m.forward(ctx, run, xn, x, then=then)
            else:
                m.forward(ctx, run, xn, x)
