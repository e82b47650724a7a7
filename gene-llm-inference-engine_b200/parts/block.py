"""Arrangements of the parts of one layer."""
from __future__ import annotations

import torch

from .registry import FEED_FORWARDS, MIXERS, NORMS, build_part, register_block, sub_weights


@register_block("pre_norm")
class PreNormBlock:
    """x += mixer(norm(x)); x += feed_forward(norm(x)), the residual stream x kept in 32-bit
    (src/model/transformer.cpp:379-451)."""

    def __init__(self, layer_spec, weights, build):
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm,
                                            sub_weights(weights, "feed_forward_norm."), build)
        self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                       sub_weights(weights, "feed_forward."), build)
        self.dtype = build.compute_dtype

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        xn = ctx.scratch("normed", tuple(x.shape), self.dtype)
        T = x.shape[0]
        # each half of the layer is one launch program when its parts say what their launches depend on
        # (``launch_key``); a part without that method (one that computes with other libraries) runs as it is
        key = _launch_key(ctx, (self.mixer_norm, None), (self.mixer, run))
        if key is not None:
            ctx.recorded(self, ("mixer", run, T) + key, lambda: self._mixer_half(ctx, run, xn, x))
        else:
            self._mixer_half(ctx, run, xn, x)
        ctx.tap("attn_out", run.layer, x)
        key = _launch_key(ctx, (self.feed_forward_norm, None), (self.feed_forward, None))
        if key is not None:
            ctx.recorded(self, ("feed_forward", T) + key, lambda: self._feed_forward_half(ctx, xn, x))
        else:
            self._feed_forward_half(ctx, xn, x)
        ctx.tap("ffn_out", run.layer, x)

    def _mixer_half(self, ctx, run, xn, x) -> None:
        self.mixer_norm.forward(x, xn)
        then = getattr(self.feed_forward, "first_product", None)
        if then is not None and getattr(self.mixer, "takes_then", False):
            self.mixer.forward(ctx, run, xn, x, then=then)      # the mixer's last product asks for the weights that follow
        else:
            self.mixer.forward(ctx, run, xn, x)

    def _feed_forward_half(self, ctx, xn, x) -> None:
        self.feed_forward_norm.forward(x, xn)
        self.feed_forward.forward(ctx, xn, x)


@register_block("post_norm")
class PostNormBlock:
    """x <- N1(alpha x + mixer(x)) and, when the layer has a feed-forward, x <- N2(alpha x + ff(x)): the norm
    comes after the residual sum and the sublayers read the stream x itself. ``block_params``: ``alpha`` (1).

    The stream stays 32-bit. A sublayer reads ``xn`` (x in the compute dtype; x itself on the 32-bit path)
    and adds its output to ``acc``, which holds alpha x. One kernel takes the norm of acc into x and, in the
    same pass, prepares xn and acc of the sublayer that follows; the next layer of this arrangement finds them
    ready (``ctx.carry``), so that a layer costs one memory-bound kernel per sublayer besides the sublayers."""

    def __init__(self, layer_spec, weights, build):
        self.alpha = float(layer_spec.block_params.get("alpha", 1.0))
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm,
                                                sub_weights(weights, "feed_forward_norm."), build)
            self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                           sub_weights(weights, "feed_forward."), build)
        self.dtype = build.compute_dtype

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        from ..ops import kernels
        T = x.shape[0]
        acc = ctx.scratch("post_norm_acc", tuple(x.shape), torch.float32)
        xn = x if self.dtype is torch.float32 else ctx.scratch("normed", tuple(x.shape), self.dtype)
        carry = getattr(ctx, "carry", None)
        ready = carry is not None and carry.get("post_norm") == (x.data_ptr(), self.alpha)
        key = _launch_key(ctx, (self.mixer_norm, None), (self.mixer, run))
        second = self.feed_forward is not None

        def mixer_half():
            if not ready:
                kernels.scale_cast(x, acc, None if xn is x else xn, self.alpha)
            self.mixer.forward(ctx, run, xn, acc)
            # with a feed-forward to come, the same pass prepares what it reads and adds to
            kernels.residual_norm(acc, self.mixer_norm.weight, x, self.mixer_norm.eps, self.alpha,
                                  acc_out=acc, xn_out=None if xn is x else xn)

        if key is not None:
            ctx.recorded(self, ("mixer", run, T, ready) + key, mixer_half)
        else:
            mixer_half()
        ctx.tap("attn_out", run.layer, x)
        if second:
            def feed_forward_half():
                self.feed_forward.forward(ctx, xn, acc)
                kernels.residual_norm(acc, self.feed_forward_norm.weight, x, self.feed_forward_norm.eps, self.alpha,
                                      acc_out=acc, xn_out=None if xn is x else xn)
            key = _launch_key(ctx, (self.feed_forward_norm, None), (self.feed_forward, None))
            if key is not None:
                ctx.recorded(self, ("feed_forward", T) + key, feed_forward_half)
            else:
                feed_forward_half()
        ctx.tap("ffn_out", run.layer, x)
        if carry is not None:
            carry["post_norm"] = (x.data_ptr(), self.alpha)      # acc = alpha x and xn = x hold for whoever runs next


@register_block("output_norm")
class OutputNormBlock:
    """x <- x + N1(mixer(x)) and, when the layer has a feed-forward, x <- x + N2(ff(x)): the norm stands on the
    sublayer's output only, and the sublayers read the stream x itself.

    The stream stays 32-bit. A sublayer reads ``xn`` (x in the compute dtype; x itself on the 32-bit path) and adds
    its output to ``y``, which is zero when it starts. One kernel adds the normed y to x and, in the same pass,
    writes the next sublayer's xn and clears y; the next layer of this arrangement finds both ready (``ctx.carry``)."""

    def __init__(self, layer_spec, weights, build):
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm,
                                                sub_weights(weights, "feed_forward_norm."), build)
            self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                           sub_weights(weights, "feed_forward."), build)
        self.dtype = build.compute_dtype

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        from ..ops import kernels
        T = x.shape[0]
        y = ctx.scratch("output_norm_y", tuple(x.shape), torch.float32)
        xn = x if self.dtype is torch.float32 else ctx.scratch("normed", tuple(x.shape), self.dtype)
        carry = getattr(ctx, "carry", None)
        ready = carry is not None and carry.get("output_norm") == x.data_ptr()
        cast = None if xn is x else xn

        def mixer_half():
            if not ready:
                kernels.scale_cast(x, y, cast, 0.0)          # y = 0, xn = x
            self.mixer.forward(ctx, run, xn, y)
            kernels.add_normed(y, self.mixer_norm.weight, x, self.mixer_norm.eps, xn_out=cast, clear_y=True)

        key = _launch_key(ctx, (self.mixer_norm, None), (self.mixer, run))
        if key is not None:
            ctx.recorded(self, ("mixer", run, T, ready) + key, mixer_half)
        else:
            mixer_half()
        ctx.tap("attn_out", run.layer, x)
        if self.feed_forward is not None:
            def feed_forward_half():
                self.feed_forward.forward(ctx, xn, y)
                kernels.add_normed(y, self.feed_forward_norm.weight, x, self.feed_forward_norm.eps, xn_out=cast, clear_y=True)
            key = _launch_key(ctx, (self.feed_forward_norm, None), (self.feed_forward, None))
            if key is not None:
                ctx.recorded(self, ("feed_forward", T) + key, feed_forward_half)
            else:
                feed_forward_half()
        ctx.tap("ffn_out", run.layer, x)
        if carry is not None:
            carry["output_norm"] = x.data_ptr()      # y = 0 and xn = x hold for whoever runs next


@register_block("parallel")
class ParallelBlock:
    """One norm, whose output h both sublayers read, and one residual sum: fresh = x + m (mixer(h) + ff(h)) (``block_params``:
    ``residual_mult`` m, 1 by default; the layer may lack a feed-forward). With ``depth_slot`` s >= 1 and ``depth_slots`` the
    stream that goes on is a learned mix of everything so far: with R_0 the stream the first layer read and R_j the fresh
    result of the layer with slot j, x <- sum over j <= s of ``depth_weights``[j] R_j (weights: ``depth_weights`` [s + 1]);
    without a slot x <- fresh.

    The stream stays 32-bit. Both sublayers add into ``y``, which is zero when they start; one kernel then forms fresh
    (adding the bias of the feed-forward's last product, if it has one),
    keeps it in the step's history [tokens, slots, width], mixes, clears y and, when the next block is of this kind with a
    norm of a single weight, writes that block's normed input in the same pass (``ctx.carry``)."""

    def __init__(self, layer_spec, weights, build):
        bp = layer_spec.block_params
        self.mult = float(bp.get("residual_mult", 1.0))
        self.slot = int(bp.get("depth_slot", 0))
        self.slots = int(bp.get("depth_slots", 0))
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                           sub_weights(weights, "feed_forward."), build)
        # the bias of the feed-forward's last product is added by the kernel that ends the layer
        leave = getattr(self.feed_forward, "leave_output_bias", None)
        self.y_bias = leave() if leave is not None else None
        self.depth_weights = None
        if self.slot:
            if not (1 <= self.slot < self.slots):
                raise ValueError(f"parallel block: slot {self.slot} lies outside the {self.slots} kept results")
            w = weights["depth_weights"]
            if w.numel() != self.slot + 1:
                raise ValueError(f"parallel block: {w.numel()} depth weights, expected {self.slot + 1}")
            self.depth_weights = w.reshape(-1).to(device=build.device, dtype=torch.float32).contiguous()
        self.dtype = build.compute_dtype
        self._next = None           # the block of the next run, when this kernel can write its normed input

    def followed_by(self, block) -> None:
        ok = isinstance(block, ParallelBlock) and hasattr(block.mixer_norm, "scalar")
        if self._next is None and ok:
            self._next = block
        elif self._next is not block:
            self._next = False      # several successors (a layer that runs more than once): nothing is prepared

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        from ..ops import kernels
        T, D = x.shape
        y = ctx.scratch("parallel_y", (T, D), torch.float32)
        xn = ctx.scratch("normed", (T, D), self.dtype)
        hist = ctx.scratch("depth_history", (T, self.slots, D), torch.float32) if self.slot else None
        carry = getattr(ctx, "carry", None)
        state = carry.get("parallel") if carry is not None else None
        # what the block before left: y = 0 everywhere, xn = this block's normed input, the history filled up to its slot
        ready = state is not None and state[0] == x.data_ptr() and state[1] is self
        first = self.slot and not (state is not None and state[0] == x.data_ptr() and state[2])
        nxt = self._next if self._next else None

        def layer():
            if not ready:
                if state is None or state[0] != x.data_ptr():
                    kernels.scale_cast(x, y, None, 0.0)                          # y = 0
                self.mixer_norm.forward(x, xn)
            self.mixer.forward(ctx, run, xn, y)
            if self.feed_forward is not None:
                self.feed_forward.forward(ctx, xn, y)
            kernels.depth_mix(x, y, self.mult, hist, self.slot, self.depth_weights, first=bool(first),
                              next_weight=nxt.mixer_norm.scalar if nxt else None, eps=nxt.mixer_norm.eps if nxt else 0.0,
                              xn_out=xn if nxt else None, y_bias=self.y_bias)

        parts = [(self.mixer_norm, None), (self.mixer, run)] + ([(self.feed_forward, None)] if self.feed_forward is not None else [])
        key = _launch_key(ctx, *parts)
        if key is not None:
            ctx.recorded(self, ("layer", run, T, ready, bool(first), state is None or state[0] != x.data_ptr()) + key, layer)
        else:
            layer()
        ctx.tap("attn_out", run.layer, x)
        ctx.tap("ffn_out", run.layer, x)
        if carry is not None:
            carry["parallel"] = (x.data_ptr(), nxt, bool(self.slot))


@register_block("hyper_connections")
class HyperConnectionBlock:
    """A pre-norm layer over several copies X[0..S-1] of the residual stream instead of one. Sublayer q (1: the mixer, 2: the
    feed-forward, which a layer may lack) reads u = sum_s a_q[s] X[s], computes y = sublayer(N_q(u)), and every copy is then
    rewritten at once from the old ones: X'[t] = sum_s M_q[s, t] X[s] + b_q[t] y. The first block of this kind in a row
    starts from copies that all equal the stream it is handed; the last one leaves the sum of the copies there.
    ``block_params``: ``streams`` (S). Weights: ``hc1.in`` [S], ``hc1.out`` [S], ``hc1.mix`` [S, S] (indexed [from, to]) and the
    same under ``hc2.``.

    The copies are 32-bit, [tokens, S, width], scratch of the step. A sublayer adds into ``y``, which is zero when it starts.
    One kernel per sublayer rewrites the copies, clears y and writes the normed input of the sublayer that runs next (the
    feed-forward's, or the next block's mixer's when that block is of this kind with as many copies) in the same pass, so a
    layer costs one memory-bound kernel per sublayer beside the sublayers (``ctx.carry`` tells the next block what it finds)."""

    def __init__(self, layer_spec, weights, build):
        self.streams = int(layer_spec.block_params["streams"])
        if not (1 <= self.streams <= 8):
            raise ValueError(f"hyper-connection block: {self.streams} copies of the stream are not supported (1 to 8)")
        self.mixer_norm = build_part(NORMS, "norm", layer_spec.mixer_norm, sub_weights(weights, "mixer_norm."), build)
        self.mixer = build_part(MIXERS, "mixer", layer_spec.mixer, sub_weights(weights, "mixer."), build)
        self.feed_forward = self.feed_forward_norm = None
        if layer_spec.feed_forward is not None:
            self.feed_forward_norm = build_part(NORMS, "norm", layer_spec.feed_forward_norm,
                                                sub_weights(weights, "feed_forward_norm."), build)
            self.feed_forward = build_part(FEED_FORWARDS, "feed-forward", layer_spec.feed_forward,
                                           sub_weights(weights, "feed_forward."), build)
        S = self.streams
        self.connections = []
        for q in (1, 2) if self.feed_forward is not None else (1,):
            got = {}
            for name, shape in (("in", (S,)), ("out", (S,)), ("mix", (S, S))):
                w = weights[f"hc{q}.{name}"]
                if tuple(w.shape) != shape:
                    raise ValueError(f"hyper-connection block: hc{q}.{name} has shape {tuple(w.shape)}, expected {shape}")
                got[name] = w.to(device=build.device, dtype=torch.float32).contiguous()
            self.connections.append(got)
        self.dtype = build.compute_dtype
        self._next = {}             # run (by the layer whose cache it uses) -> the block that runs after it, when of this kind

    def followed_in_run(self, run, block) -> None:
        ok = isinstance(block, HyperConnectionBlock) and block.streams == self.streams
        self._next[run.cache_layer] = block if ok else None

    def forward(self, ctx, run, x: torch.Tensor) -> None:
        from ..ops import kernels
        T, D = x.shape
        S = self.streams
        X = ctx.scratch("stream_copies", (T, S, D), torch.float32)
        y = ctx.scratch("stream_y", (T, D), torch.float32)
        xn = ctx.scratch("normed", (T, D), self.dtype)
        carry = getattr(ctx, "carry", None)
        state = carry.get("stream_copies") if carry is not None else None
        # what the block before left: the copies, y = 0 and xn = this block's normed input
        ready = state is not None and state == (x.data_ptr(), id(self))
        nxt = self._next.get(run.cache_layer)
        show = bool(getattr(ctx, "tapping", False))
        first, second = self.connections[0], (self.connections[1] if self.feed_forward is not None else None)

        def rewrite(con, to_norm, to_in, sum_out):
            kernels.streams(X, y=y, clear_y=True, mix=con["mix"], out_w=con["out"], in_w=to_in,
                            norm_weight=None if to_norm is None else to_norm.weight,
                            eps=0.0 if to_norm is None else to_norm.eps, xn_out=None if to_norm is None else xn, sum_out=sum_out)

        def after(sum_now):
            """What the kernel that ends this block's last sublayer prepares: the next block's read, or the sum of the copies."""
            if nxt is not None:
                return nxt.mixer_norm, nxt.connections[0]["in"], (x if sum_now else None)
            return None, None, x

        def mixer_half():
            if not ready:
                kernels.scale_cast(x, y, None, 0.0)                                   # y = 0
                kernels.streams(X, single=x, in_w=first["in"], norm_weight=self.mixer_norm.weight, eps=self.mixer_norm.eps, xn_out=xn)
            self.mixer.forward(ctx, run, xn, y)
            if second is not None:
                rewrite(first, self.feed_forward_norm, second["in"], x if show else None)
            else:
                rewrite(first, *after(show))

        key = _launch_key(ctx, (self.mixer_norm, None), (self.mixer, run))
        if key is not None:
            ctx.recorded(self, ("mixer", run, T, ready) + key, mixer_half)
        else:
            mixer_half()
        ctx.tap("attn_out", run.layer, x)
        if second is not None:
            def feed_forward_half():
                self.feed_forward.forward(ctx, xn, y)
                rewrite(second, *after(show))
            key = _launch_key(ctx, (self.feed_forward_norm, None), (self.feed_forward, None))
            if key is not None:
                ctx.recorded(self, ("feed_forward", run, T) + key, feed_forward_half)
            else:
                feed_forward_half()
        ctx.tap("ffn_out", run.layer, x)
        if carry is not None:
            if nxt is not None:
                carry["stream_copies"] = (x.data_ptr(), id(nxt))
            else:
                carry.pop("stream_copies", None)


def build_extra(layer_spec, key: str, table, what: str, weights, build):
    """Builds the part that a layer's ``extra`` names ``key`` (for arrangements with more parts than
    the usual four), with the weights under ``<key>.``."""
    if key not in layer_spec.extra:
        raise KeyError(f"block arrangement '{layer_spec.block}' needs a part '{key}' that the layer's specification lacks")
    return build_part(table, what, layer_spec.extra[key], sub_weights(weights, key + "."), build)


def _launch_key(ctx, *parts):
    """The joint key of some parts' launches for this step, or None when one of them has none (or the
    context records nothing)."""
    if not hasattr(ctx, "recorded"):
        return None
    key = ()
    for part, run in parts:
        fn = getattr(part, "launch_key", None)
        if fn is None:
            return None
        k = fn(ctx) if run is None else fn(ctx, run)
        if k is None:
            return None
        key += tuple(k)
    return key
