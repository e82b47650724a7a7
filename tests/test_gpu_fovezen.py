"""Fovezen on the GPU against the plain implementation in plain_fovezen.py: each kernel and each mechanism alone, then
whole models through the step engine under different cuts of the same requests (whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches on reused pages and state slots), keys made to stand out far back,
at page borders and on either side of a window's edge, the first tokens of a sequence, and greedy generation through
the engine's own entry point and scheduler."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import fovezen_configs as fc
import plain_fovezen as pf
import tiny_configs as tc
import trace_tools as tt
from test_gpu_nipadra import _run_mixer
from test_gpu_gekupel import PagesCtx

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
F = torch.float64
EPS = 1e-5


def _build(dtype, max_position=4096):
    from geneinfer_b200.parts import BuildContext
    return BuildContext(DEV, dtype, max_position)


def _bf(t):
    return t.to(torch.bfloat16).float()


def _close(got, want, dtype, what, f32=2e-5, b16=2e-2):
    err = float((got.double() - want.double()).abs().max() / max(1.0, float(want.abs().max())))
    assert err < (f32 if dtype is torch.float32 else b16), f"{what}: {err}"


class StateCtx(PagesCtx):
    """A mixer's view of a step with pages of its own widths and a state slot per request."""

    def __init__(self, dtype, n_requests, Hkv=1, hd=16, vd=16, state_floats=1, page_size=8, max_len=256):
        super().__init__(dtype, n_requests, Hkv, hd, vd, page_size=page_size, max_len=max_len)
        self._state = torch.zeros(n_requests + 1, max(state_floats, 1), dtype=torch.float32, device=DEV)
        self.max_position = max_len

    def begin(self, lengths):
        self.carry.clear()          # as the engine does when a forward pass starts
        return super().begin(lengths)

    def tap(self, tag, layer, tensor):
        pass


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("S", [1, 2, 3, 8])
@pytest.mark.parametrize("D", [200, 7, 4500])
def test_stream_copies_kernel(dtype, S, D):
    """The start from one stream, a rewrite with the next read in the same pass, a rewrite alone, a read alone, the sum."""
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(S * 10 + D)
    T = 6
    x = torch.randn(T, D, generator=g) * 2
    a1, a2 = torch.randn(S, generator=g), torch.randn(S, generator=g)
    M, b = torch.randn(S, S, generator=g), torch.randn(S, generator=g)
    w = 1 + 0.3 * torch.randn(D, generator=g)
    X = torch.full((T, S, D), float("nan"), device=DEV)
    xn = torch.full((T, D), float("nan"), dtype=dtype, device=DEV)
    kernels.streams(X, single=x.to(DEV), in_w=a1.to(DEV), norm_weight=w.to(DEV), eps=EPS, xn_out=xn)
    copies = x.double()[None].repeat(S, 1, 1)
    _close(X.cpu().transpose(0, 1), copies, torch.float32, "copies of the single stream", f32=1e-7)
    u = torch.einsum("s,std->td", a1.double(), copies)
    _close(xn.cpu().float(), pf.unit_rms(u, EPS) * w.double(), dtype, "first read", f32=3e-6, b16=1e-2)
    y = torch.randn(T, D, generator=g)
    yd = y.to(DEV).clone()
    total = torch.full((T, D), float("nan"), device=DEV)
    kernels.streams(X, y=yd, clear_y=True, mix=M.to(DEV), out_w=b.to(DEV), in_w=a2.to(DEV), norm_weight=w.to(DEV), eps=EPS,
                    xn_out=xn, sum_out=total)
    copies = torch.einsum("sr,std->rtd", M.double(), copies) + b.double()[:, None, None] * y.double()[None]
    assert not yd.any()
    _close(X.cpu().transpose(0, 1), copies, torch.float32, "rewritten copies", f32=2e-6)
    _close(total.cpu(), copies.sum(0), torch.float32, "sum of the copies", f32=2e-6)
    u = torch.einsum("s,std->td", a2.double(), copies)
    _close(xn.cpu().float(), pf.unit_rms(u, EPS) * w.double(), dtype, "read after the rewrite", f32=3e-6, b16=1e-2)
    # a rewrite alone (y kept), then a read alone
    yd = y.to(DEV).clone()
    kernels.streams(X, y=yd, mix=M.to(DEV), out_w=b.to(DEV))
    assert torch.equal(yd.cpu(), y)
    copies = torch.einsum("sr,std->rtd", M.double(), copies) + b.double()[:, None, None] * y.double()[None]
    before = X.clone()
    kernels.streams(X, in_w=a1.to(DEV), norm_weight=w.to(DEV), eps=EPS, xn_out=xn)
    assert torch.equal(X, before)
    u = torch.einsum("s,std->td", a1.double(), copies)
    _close(xn.cpu().float(), pf.unit_rms(u, EPS) * w.double(), dtype, "read alone", f32=5e-6, b16=1e-2)


@pytest.mark.parametrize("taps", [1, 2, 3, 5])
def test_convolution_without_bias_or_activation_and_its_state(taps):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(taps)
    C, off, ld = 37, 5, 50
    w = torch.randn(C, taps, generator=g)
    seqs = [torch.randn(n, ld, generator=g) for n in (9, 1, 14)]
    want = [pf.short_conv(s[:, off:off + C].double(), w.double()) for s in seqs]
    state = torch.zeros(4, 3 + (taps - 1) * C, device=DEV)
    slots = [2, 0, 3]
    got = [[] for _ in seqs]
    at = [0, 0, 0]
    for lengths in ([1, 1, 2], [2, 0, 1], [1, 0, 3], [5, 0, 8]):
        live = [r for r, n in enumerate(lengths) if n]
        rows = torch.cat([seqs[r][at[r]:at[r] + lengths[r]] for r in live]).to(DEV)
        starts = np.cumsum([0] + [lengths[r] for r in live])
        row_req = torch.cat([torch.full((lengths[r],), i) for i, r in enumerate(live)]).int().to(DEV)
        out = torch.full((rows.shape[0], C), float("nan"), device=DEV)
        kernels.causal_conv(rows, off, w.to(DEV), None, state, 3, row_req, torch.tensor(starts[:-1], dtype=torch.int32, device=DEV),
                            torch.tensor([lengths[r] for r in live], dtype=torch.int32, device=DEV),
                            torch.tensor([slots[r] for r in live], dtype=torch.int32, device=DEV), out, activate=False)
        for i, r in enumerate(live):
            got[r].append(out[starts[i]:starts[i + 1]].cpu())
            at[r] += lengths[r]
    for r in range(3):
        _close(torch.cat(got[r]), want[r], torch.float32, f"convolution, request {r}", f32=2e-6)
    assert not state[:, :3].any() and not state[1].any()


def _plain_row_decay_scan(q, k, v, z, tau, S0=None):
    T, H, dk = q.shape
    dv = v.shape[2]
    alpha = torch.exp(-pf.softplus(-z) / tau)
    S = torch.zeros(H, dk, dv, dtype=F) if S0 is None else S0.clone()
    o = torch.zeros(T, H, dv, dtype=F)
    for t in range(T):
        S = alpha[t][:, :, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return o, S


@pytest.mark.parametrize("H, dk, dv", [(3, 16, 24), (2, 48, 40), (1, 100, 33), (2, 200, 8), (5, 8, 64)])
def test_recurrence_with_a_decay_per_row(H, dk, dv):
    """One walk from a state that an earlier step left; a step of more than 128 tokens cut into parts that run side by
    side; single tokens; the bias on z and the constant on the queries."""
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(H * 100 + dk)
    tau, qs = 4.0, 0.37
    lens = [300, 2, 150]
    ld = 2 * H * dk + H * dv + 3
    rows = [torch.randn(n, ld, generator=g) * 0.5 for n in lens]
    gate = [torch.randn(n, H * dk + 2, generator=g) * 2 + 2 for n in lens]
    bias = torch.randn(H * dk, generator=g)
    want = []
    for r, z in zip(rows, gate):
        n = r.shape[0]
        q, k = r[:, 3:3 + H * dk].double().view(n, H, dk) * qs, r[:, 3 + H * dk:3 + 2 * H * dk].double().view(n, H, dk)
        v = r[:, 3 + 2 * H * dk:].double().view(n, H, dv)
        want.append(_plain_row_decay_scan(q, k, v, (z[:, 2:].double() + bias.double()).view(n, H, dk), tau))
    for cuts in ([[300, 2, 150]], [[1, 1, 1], [129, 1, 20], [1, 0, 1], [169, 0, 128]]):
        state = torch.zeros(4, 5 + H * dk * dv, device=DEV)
        slots, at, got = [3, 1, 0], [0, 0, 0], [[], [], []]
        for lengths in cuts:
            live = [r for r, n in enumerate(lengths) if n]
            T = sum(lengths)
            x = torch.cat([rows[r][at[r]:at[r] + lengths[r]] for r in live]).to(DEV)
            z = torch.cat([gate[r][at[r]:at[r] + lengths[r]] for r in live]).to(DEV)
            starts = np.cumsum([0] + [lengths[r] for r in live])
            out = torch.full((T, H * dv), float("nan"), device=DEV)
            extra = {}
            if T > kernels.SCAN_PART:
                extra = {"part_len": kernels.SCAN_PART, "ws_state": torch.full((kernels.scan_parts(T, len(live)), H * dk * dv), float("nan"), device=DEV),
                         "ws_decay": torch.full((T, H * dk), float("nan"), device=DEV)}
            kernels.linear_scan(x, 3, x, 3 + H * dk, x, 3 + 2 * H * dk, H, 1, dk, dv, False, state, 5,
                                torch.tensor(starts[:-1], dtype=torch.int32, device=DEV),
                                torch.tensor([lengths[r] for r in live], dtype=torch.int32, device=DEV),
                                torch.tensor([slots[r] for r in live], dtype=torch.int32, device=DEV), out,
                                row_gate=z, row_gate_offset=2, row_gate_bias=bias.to(DEV), tau=tau, q_scale=qs, **extra)
            for i, r in enumerate(live):
                got[r].append(out[starts[i]:starts[i + 1]].cpu())
                at[r] += lengths[r]
        for r in range(3):
            _close(torch.cat(got[r]), want[r][0].reshape(lens[r], H * dv), torch.float32, f"outputs of request {r}, {len(cuts)} steps", f32=1e-5)
            _close(state[slots[r], 5:].cpu(), want[r][1].reshape(-1), torch.float32, f"state of request {r}", f32=1e-5)
        assert not state[:, :5].any() and not state[2].any()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("W, groups", [(96, 3), (70, 5), (256, 1)])
def test_group_norm_with_a_silu_gate_after_it(dtype, W, groups):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(W)
    y, gate, w = torch.randn(9, W, generator=g) * 3, torch.randn(9, W + 8, generator=g) * 2, torch.randn(W, generator=g)
    out = torch.empty(9, W, dtype=dtype, device=DEV)
    kernels.gated_group_norm(y.to(DEV), gate.to(DEV), 8, w.to(DEV), out, groups, 1e-3, gate_first=False, gate_act="silu")
    want = pf.unit_rms(y.double().view(9, groups, W // groups), 1e-3).reshape(9, W) * w.double() * pf.silu(gate[:, 8:].double())
    _close(out.cpu().float(), want, dtype, "norm, then SiLU gate", f32=2e-6, b16=1e-2)


@pytest.mark.parametrize("H, Hkv, hd, vd, rot_dims", [(3, 1, 32, 32, 16), (4, 2, 16, 24, 16), (2, 2, 64, 8, 0), (5, 5, 8, 8, 4)])
def test_norm_over_the_whole_projection_then_partial_rotation_in_halves(H, Hkv, hd, vd, rot_dims):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(H * 7 + hd)
    T, page = 11, 4
    ld = (H + Hkv) * hd + Hkv * vd
    proj = torch.randn(T, ld, generator=g) * 2
    qw, kw = torch.randn(H * hd, generator=g), torch.randn(Hkv * hd, generator=g)
    freq = torch.tensor([50.0 ** (-2.0 * i / max(rot_dims, 1)) for i in range(rot_dims // 2)])
    positions = torch.tensor([0, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10], dtype=torch.int32)
    tables = torch.tensor([[2, 0, 1]], dtype=torch.int32)
    q = torch.full((T, H * hd), float("nan"), device=DEV)
    kc, vc = torch.full((3, Hkv, page, hd), float("nan"), device=DEV), torch.full((3, Hkv, page, vd), float("nan"), device=DEV)
    kernels.norm_rope_store(proj.to(DEV), 0, H * hd, (H + Hkv) * hd, qw.to(DEV), kw.to(DEV), EPS, freq.to(DEV) if rot_dims else None, False,
                            positions.to(DEV), torch.zeros(T, dtype=torch.int32, device=DEV), tables.to(DEV), q, kc, vc, H, Hkv, hd, page,
                            value_dim=vd, wide_norm=True)
    pq = pf.norm_plain(proj[:, :H * hd].double(), qw, EPS).view(T, H, hd)
    pk = pf.norm_plain(proj[:, H * hd:(H + Hkv) * hd].double(), kw, EPS).view(T, Hkv, hd)
    if rot_dims:
        pq, pk = pf.rotate_half_layout(pq, freq.double(), rot_dims), pf.rotate_half_layout(pk, freq.double(), rot_dims)
    _close(q.cpu().view(T, H, hd), pq, torch.float32, "queries", f32=5e-6)
    order = [2, 0, 1]
    keys = torch.stack([kc[order[t // page], :, t % page].cpu() for t in range(T)])
    vals = torch.stack([vc[order[t // page], :, t % page].cpu() for t in range(T)])
    _close(keys, pk, torch.float32, "keys in their pages", f32=5e-6)
    _close(vals, proj[:, (H + Hkv) * hd:].view(T, Hkv, vd), torch.float32, "values in their pages", f32=1e-7)


def test_wavelength_scaling_of_the_rotation_frequencies():
    from geneinfer_b200.parts import POSITION_ENCODINGS
    rot = {"base": 250.0, "dims": 32, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}
    part = POSITION_ENCODINGS["rope_on_device"]({"head_dim": 48, "rotary_dim": 32, "theta": 250.0, "pairing": "half_split",
                                                 "wavelength_scaling": {"factor": 4.0, "low": 1.0, "high": 4.0, "original": 64}}, {}, _build(torch.float32))
    want = pf.scaled_frequencies(rot, F)
    plain = pf.scaled_frequencies({"base": 250.0, "dims": 32}, F)
    ratio = (want / plain).tolist()
    assert ratio[0] == 1.0 and abs(ratio[-1] - 0.25) < 1e-12 and any(0.26 < r < 0.99 for r in ratio)      # all three ranges occur
    assert float((part.freq.cpu().double() - want).abs().max() / want.max()) < 1e-7 and not part.interleaved


# ------------------------------------------------------------------------------------------ mixers alone
def _mat(rows, cols, g, std=0.3):
    return _bf(torch.randn(rows, cols, generator=g) * std)


GLA = {"heads": 3, "dim": 16, "vdim": 40, "tau": 6.0, "rank": 8}


def _gla_weights(D, m, g, p="p."):
    H, d, dv, r = m["heads"], m["dim"], m["vdim"], m["rank"]
    return {p + "q": _mat(H * d, D, g), p + "k": _mat(H * d, D, g), p + "v": _mat(H * dv, D, g), p + "g": _mat(H * dv, D, g),
            p + "a1": _mat(r, D, g), p + "a2": _mat(H * d, r, g, 0.8), p + "a2.b": torch.rand(H * d, generator=g) * 4,
            p + "norm": 1 + 0.2 * torch.randn(dv, generator=g), p + "o": _mat(D, H * dv, g)}


def _gla_part(D, m, w, dtype, p="p."):
    from geneinfer_b200.parts import MIXERS
    return MIXERS["gated_linear_attention"](
        {"hidden_size": D, "num_heads": m["heads"], "key_dim": m["dim"], "value_dim": m["vdim"], "tau": m["tau"], "norm_eps": EPS},
        {"w_in": torch.cat([w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"]]), "w_a1": w[p + "a1"], "w_a2": w[p + "a2"],
         "a2_bias": w[p + "a2.b"], "norm": w[p + "norm"], "w_o": w[p + "o"]}, _build(dtype))


CUTS = {"whole": [[40, 2, 19]], "token by token": [[1, 1, 1]] * 2 + [[1, 0, 1]] * 17 + [[1, 0, 0]] * 21,
        "portions": [[2, 1, 3], [5, 1, 2], [2, 0, 14], [31, 0, 0]], "tail decoded": [[30, 2, 10]] + [[1, 0, 1]] * 9 + [[1, 0, 0]]}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [GLA, dict(GLA, heads=1, dim=64, vdim=16, rank=16, tau=1.0), dict(GLA, heads=2, dim=40, vdim=40, rank=12)])
def test_gated_linear_attention_with_its_state_carried_across_steps(dtype, m):
    D = 48
    g = torch.Generator().manual_seed(4)
    w = _gla_weights(D, m, g)
    part = _gla_part(D, m, w, dtype)
    assert part.rank == m["rank"] and part.state_need().shape == (m["heads"] * m["dim"] * m["vdim"],)
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (40, 2, 19)]
    rnd = pf.ident if dtype is torch.float32 else pf.bf16
    want = [pf.gated_linear_attention(w, "p.", m, x.double(), EPS, F, rnd) for x in inputs]
    for name, cuts in CUTS.items():
        ctx = StateCtx(dtype, 3, state_floats=part.state_need().shape[0])
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"gated linear attention, request {r}, {name}", b16=3e-2)


def test_a_slowly_fading_row_remembers_a_far_token_and_a_fast_one_forgets_it():
    """Head 0's decays are set near 1 and head 1's near 0 through the bias of z; the value written at token 3 is read at the end."""
    D, m = 32, {"heads": 2, "dim": 16, "vdim": 16, "tau": 1.0, "rank": 8}
    g = torch.Generator().manual_seed(12)
    w = _gla_weights(D, m, g)
    w["p.a2"] = w["p.a2"] * 0.0
    w["p.a2.b"] = torch.cat([torch.full((16,), 12.0), torch.full((16,), -3.0)])
    n = 300
    x = _bf(torch.randn(n, D, generator=g) * 0.05)
    x[3] = _bf(torch.randn(D, generator=g) * 3)
    want = pf.gated_linear_attention(w, "p.", m, x.double(), EPS, F, pf.ident)
    without = pf.gated_linear_attention(w, "p.", m, torch.cat([x[:3], x[4:]]).double(), EPS, F, pf.ident)
    assert float((want[-1] - without[-1]).abs().max()) > 0.05 * float(want[-1].abs().max())       # the far token matters at the end
    part = _gla_part(D, m, w, torch.float32)
    for cuts in ([[n]], [[200]] + [[1]] * 100, [[2], [129], [128], [41]]):
        got = _run_mixer(part, StateCtx(torch.float32, 1, state_floats=part.state_need().shape[0], max_len=320), [x], cuts, torch.float32, D)
        _close(got[0], want, torch.float32, f"far memory, {len(cuts)} steps", f32=3e-5)


LEFT = {"heads": 6, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3, "mask": {"size": 11}, "conv": 3, "softcap": 4.0}


def _left_weights(D, m, g, p="p."):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    w = {p + "q": _mat(H * d, D, g), p + "k": _mat(G * d, D, g), p + "v": _mat(G * dv, D, g), p + "o": _mat(D, H * dv, g),
         p + "q.norm": 1 + 0.3 * torch.randn(d, generator=g), p + "k.norm": 1 + 0.3 * torch.randn(d, generator=g)}
    if m.get("conv"):
        for n, rows in (("q", H * d), ("k", G * d), ("v", G * dv)):
            w[p + n + ".conv"] = torch.randn(rows, m["conv"], generator=g) * 0.6
    return w


def _left_part(D, m, w, dtype, p="p."):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    weights = {"w_qkv": torch.cat([w[p + "q"], w[p + "k"], w[p + "v"]]), "w_o": w[p + "o"], "q_norm": w[p + "q.norm"], "k_norm": w[p + "k.norm"]}
    if m.get("conv"):
        weights["conv"] = torch.cat([w[p + "q.conv"], w[p + "k.conv"], w[p + "v.conv"]])
    return MIXERS["attention"]({"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                                "value_dim": m["vdim"], "scale": m["scale"], "window": (m.get("mask") or {}).get("size"), "position": PartSpec("none", {}),
                                "qk_norm_eps": EPS, "conv_taps": m.get("conv"), "softcap": m.get("softcap")}, weights, _build(dtype))


def _left_ctx(part, m, dtype, n, max_len=256, page_size=8):
    need = part.state_need()
    return StateCtx(dtype, n, Hkv=m["kv_heads"], hd=m["dim"], vd=m["vdim"], state_floats=need.shape[0] if need else 1,
                    page_size=page_size, max_len=max_len)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [LEFT, dict(LEFT, heads=2, kv_heads=2, dim=64, vdim=64, conv=2, softcap=None, mask={"size": 5}),
                               dict(LEFT, heads=4, kv_heads=1, dim=32, vdim=16, conv=None, mask={"size": 300}),
                               dict(LEFT, heads=3, kv_heads=3, dim=16, vdim=32, conv=1, mask=None),
                               # soft-capped scores at the head sizes whose prompt portions the tcgen05 kernel runs
                               dict(LEFT, heads=4, kv_heads=2, dim=64, vdim=64, conv=2, softcap=2.5, scale=0.5, mask={"size": 23}),
                               dict(LEFT, heads=2, kv_heads=1, dim=128, vdim=128, conv=None, softcap=1.5, scale=0.3, mask={"size": 300})])
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_window_attention_with_a_convolution_of_its_projections(dtype, m, cut):
    D = 40
    g = torch.Generator().manual_seed(9)
    w = _left_weights(D, m, g)
    part = _left_part(D, m, w, dtype)
    if (m.get("conv") or 1) > 1:
        assert part.state_need().shape == ((m["conv"] - 1) * ((m["heads"] + m["kv_heads"]) * m["dim"] + m["kv_heads"] * m["vdim"]),)
    else:
        assert part.state_need() is None
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (40, 2, 19)]
    rnd = pf.ident if dtype is torch.float32 else pf.bf16
    want = [pf.window_conv_attention(w, "p.", m, x.double(), EPS, F, rnd) for x in inputs]
    ctx = _left_ctx(part, m, dtype, 3)
    # capped scores alone, at head sizes 64 and 128 in bfloat16: the tensor-core kernels of plain attention take the cap
    fast = dtype is torch.bfloat16 and m.get("softcap") is not None and m["dim"] == m["vdim"] and m["dim"] in (64, 128)
    assert part._cap_singles_on_decode(ctx) == fast and part._cap_tiles_on_tcgen05(ctx) == fast
    got = _run_mixer(part, ctx, inputs, CUTS[cut], dtype, D)
    for r in range(3):
        _close(got[r], want[r], dtype, f"window attention, request {r}, {cut}", b16=3e-2)


def test_the_soft_cap_is_part_of_the_scores():
    D, m = 40, dict(LEFT, scale=3.0, softcap=2.0, mask={"size": 30})
    g = torch.Generator().manual_seed(10)
    w = _left_weights(D, m, g)
    x = _bf(torch.randn(25, D, generator=g))
    capped = pf.window_conv_attention(w, "p.", m, x.double(), EPS, F, pf.ident)
    free = pf.window_conv_attention(w, "p.", dict(m, softcap=None), x.double(), EPS, F, pf.ident)
    assert float((capped - free).abs().max()) > 0.05 * float(free.abs().max())
    part = _left_part(D, m, w, torch.float32)
    got = _run_mixer(part, _left_ctx(part, m, torch.float32, 1), [x], [[20]] + [[1]] * 5, torch.float32, D)
    _close(got[0], capped, torch.float32, "soft-capped scores")


def _sharp_left(D, m, g, key_at, n):
    """Weights and inputs such that the query of the last token answers the key written at ``key_at`` and nothing else:
    one input direction drives one query/key channel hard; without a convolution the key is the token's own."""
    w = _left_weights(D, m, g)
    for name in ("p.q", "p.k"):
        w[name] = w[name] * 0.05
    x = _bf(torch.randn(n, D, generator=g) * 0.3)
    x[:, 0] = 0.0
    x[:, 1] = 0.0
    w["p.q"][:, 1] = 0.0
    w["p.k"][:, 0] = 0.0
    for h in range(m["heads"]):
        w["p.q"][h * m["dim"] + 2, 1] = 6.0            # input direction 1 asks
    for h in range(m["kv_heads"]):
        w["p.k"][h * m["dim"] + 2, 0] = 6.0            # input direction 0 answers
    x[key_at, 0] = 3.0
    x[n - 1, 1] = 3.0
    return w, x


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("distance", [0, 1, 7, 8, 9, 36, 37, 38])
def test_a_key_that_stands_out_on_either_side_of_the_windows_edge(decoded, distance):
    """Window 37: the key ``distance`` back is seen up to 36 and not from 37 on; also at a page border (8) and beside it."""
    D, n = 24, 60
    m = dict(LEFT, heads=2, kv_heads=1, dim=16, vdim=16, scale=1.0, softcap=None, conv=None, mask={"size": 37})
    g = torch.Generator().manual_seed(11)
    w, x = _sharp_left(D, m, g, n - 1 - distance, n)
    want = pf.window_conv_attention(w, "p.", m, x.double(), EPS, F, pf.ident)
    # the weights make the one key count when it is visible: moving the window's edge by one changes the last row
    other = pf.window_conv_attention(w, "p.", dict(m, mask={"size": 38 if distance == 37 else 36 if distance == 36 else 37}), x.double(), EPS, F, pf.ident)
    if distance in (36, 37):
        assert float((want[-1] - other[-1]).abs().max()) > 0.2 * float(want[-1].abs().max())
    for dtype in DTYPES:
        part = _left_part(D, m, w, dtype)
        cuts = [[n - 20]] + [[1]] * 20 if decoded else [[13], [n - 13]]
        rnd = pf.ident if dtype is torch.float32 else pf.bf16
        ref = want if dtype is torch.float32 else pf.window_conv_attention(w, "p.", m, x.double(), EPS, F, rnd)
        got = _run_mixer(part, _left_ctx(part, m, dtype, 1), [x], cuts, dtype, D)
        _close(got[0][-1], ref[-1], dtype, f"key {distance} back, {'decoded' if decoded else 'in a portion'}, {dtype}", b16=3e-2)


@pytest.mark.parametrize("cuts", [[[1], [1], [1], [1], [5]], [[2], [2], [5]], [[9]], [[3], [1], [5]]])
def test_the_first_tokens_see_zeros_before_the_sequence_through_the_convolution(cuts):
    """Five taps: tokens 0..3 reach back before the start; portions shorter than the reach follow one another."""
    D, m = 24, dict(LEFT, conv=5, mask={"size": 4})
    g = torch.Generator().manual_seed(13)
    w = _left_weights(D, m, g)
    x = _bf(torch.randn(9, D, generator=g))
    want = pf.window_conv_attention(w, "p.", m, x.double(), EPS, F, pf.ident)
    part = _left_part(D, m, w, torch.float32)
    ctx = _left_ctx(part, m, torch.float32, 1)
    ctx._state.fill_(0.0)
    got = _run_mixer(part, ctx, [x], cuts, torch.float32, D)
    _close(got[0], want, torch.float32, f"first tokens, cuts {cuts}")


ROT = {"heads": 6, "kv_heads": 3, "dim": 16, "vdim": 32, "scale": 0.25,
       "rot": {"base": 10000.0, "dims": 8, "scaling": {"factor": 8.0, "low": 1.0, "high": 4.0, "original": 64}}}


def _rot_weights(D, m, g, p="p."):
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    return {p + "q": _mat(H * d, D, g), p + "k": _mat(G * d, D, g), p + "v": _mat(G * dv, D, g), p + "o": _mat(D, H * dv, g),
            p + "q.norm": 1 + 0.3 * torch.randn(H * d, generator=g), p + "k.norm": 1 + 0.3 * torch.randn(G * d, generator=g)}


def _rot_part(D, m, w, dtype, p="p.", max_position=4096):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    position = PartSpec("none", {})
    if m.get("rot"):
        pp = {"head_dim": m["dim"], "rotary_dim": m["rot"]["dims"], "theta": m["rot"]["base"], "pairing": "half_split"}
        if m["rot"].get("scaling"):
            pp["wavelength_scaling"] = m["rot"]["scaling"]
        position = PartSpec("rope_on_device", pp)
    return MIXERS["attention"]({"hidden_size": D, "num_heads": m["heads"], "num_kv_heads": m["kv_heads"], "head_dim": m["dim"],
                                "value_dim": m["vdim"], "scale": m["scale"], "window": None, "position": position, "qk_norm_eps": EPS,
                                "qk_norm_wide": True},
                               {"w_qkv": torch.cat([w[p + "q"], w[p + "k"], w[p + "v"]]), "w_o": w[p + "o"], "q_norm": w[p + "q.norm"],
                                "k_norm": w[p + "k.norm"]}, _build(dtype, max_position))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", [ROT, dict(ROT, heads=4, kv_heads=2, dim=64, vdim=64, rot={"base": 500.0, "dims": 64}),
                               dict(ROT, heads=2, kv_heads=1, dim=128, vdim=128, rot={"base": 250000.0, "dims": 64}),
                               dict(ROT, heads=3, kv_heads=3, dim=32, vdim=32, rot=None)])
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_attention_with_a_norm_over_the_whole_projection(dtype, m, cut):
    D = 48
    g = torch.Generator().manual_seed(14)
    w = _rot_weights(D, m, g)
    part = _rot_part(D, m, w, dtype)
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (40, 2, 19)]
    rnd = pf.ident if dtype is torch.float32 else pf.bf16
    want = [pf.rotary_attention(w, "p.", m, x.double(), EPS, F, rnd) for x in inputs]
    ctx = StateCtx(dtype, 3, Hkv=m["kv_heads"], hd=m["dim"], vd=m["vdim"], page_size=16)
    got = _run_mixer(part, ctx, inputs, CUTS[cut], dtype, D)
    for r in range(3):
        _close(got[r], want[r], dtype, f"attention, request {r}, {cut}", b16=3e-2)


@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("back", [0, 1, 15, 16, 17, 650])
def test_one_key_among_hundreds(decoded, back):
    """The last query answers one key only, far back, at a page border or its own; no rotation, so that the score does not
    depend on the distance."""
    D, n = 24, 700
    m = dict(ROT, heads=2, kv_heads=1, dim=16, vdim=16, scale=1.0, rot=None)
    g = torch.Generator().manual_seed(15)
    w = _rot_weights(D, m, g)
    x = _bf(torch.randn(n, D, generator=g) * 0.3)
    x[:, 0] = x[:, 1] = 0.0
    w["p.q"], w["p.k"] = w["p.q"] * 0.02, w["p.k"] * 0.02
    w["p.q"][:, 1] = 0.0
    w["p.k"][:, 0] = 0.0
    w["p.q"][2, 1] = w["p.q"][18, 1] = 8.0
    w["p.k"][2, 0] = 8.0
    w["p.q.norm"], w["p.k.norm"] = torch.full((32,), 2.0), torch.full((16,), 2.0)
    x[n - 1 - back, 0] = 3.0
    x[n - 1, 1] = 3.0
    want = pf.rotary_attention(w, "p.", m, x.double(), EPS, F, pf.ident)
    moved = x.clone()
    moved[n - 1 - back, 0] = 0.0
    assert float((pf.rotary_attention(w, "p.", m, moved.double(), EPS, F, pf.ident)[-1] - want[-1]).abs().max()) > 0.2 * float(want[-1].abs().max())
    part = _rot_part(D, m, w, torch.float32)
    ctx = StateCtx(torch.float32, 1, Hkv=1, hd=16, vd=16, page_size=16, max_len=704)
    cuts = [[n - 40]] + [[1]] * 40 if decoded else [[300], [398], [2]]
    got = _run_mixer(part, ctx, [x], cuts, torch.float32, D)
    _close(got[0][-1], want[-1], torch.float32, f"key {back} back among {n}")


@pytest.mark.parametrize("dtype", DTYPES)
def test_parallel_mixer_takes_the_mean_of_its_normed_branches(dtype):
    from geneinfer_b200.config import PartSpec
    from geneinfer_b200.parts import MIXERS
    D = 48
    g = torch.Generator().manual_seed(16)
    ml, mr = LEFT, GLA
    w = {**_left_weights(D, ml, g, "p.left."), **_gla_weights(D, mr, g, "p.right."),
         "p.left.out": 1 + 0.3 * torch.randn(D, generator=g), "p.right.out": 1 + 0.3 * torch.randn(D, generator=g)}
    weights = {"left_out": w["p.left.out"], "right_out": w["p.right.out"]}
    spec_l = PartSpec("attention", {"hidden_size": D, "num_heads": 6, "num_kv_heads": 2, "head_dim": 16, "value_dim": 24, "scale": 0.3,
                                    "window": 11, "position": PartSpec("none", {}), "qk_norm_eps": EPS, "conv_taps": 3, "softcap": 4.0})
    spec_r = PartSpec("gated_linear_attention", {"hidden_size": D, "num_heads": 3, "key_dim": 16, "value_dim": 40, "tau": 6.0, "norm_eps": EPS})
    weights.update({"left.w_qkv": torch.cat([w["p.left.q"], w["p.left.k"], w["p.left.v"]]), "left.w_o": w["p.left.o"],
                    "left.q_norm": w["p.left.q.norm"], "left.k_norm": w["p.left.k.norm"],
                    "left.conv": torch.cat([w["p.left.q.conv"], w["p.left.k.conv"], w["p.left.v.conv"]]),
                    "right.w_in": torch.cat([w["p.right.q"], w["p.right.k"], w["p.right.v"], w["p.right.g"]]), "right.w_a1": w["p.right.a1"],
                    "right.w_a2": w["p.right.a2"], "right.a2_bias": w["p.right.a2.b"], "right.norm": w["p.right.norm"], "right.w_o": w["p.right.o"]})
    part = MIXERS["parallel"]({"branches": [("left", spec_l, 1.0), ("right", spec_r, 1.0)], "combine": "mean_normed", "combine_eps": EPS,
                               "hidden_size": D}, weights, _build(dtype))
    conv_floats, rec_floats = 2 * (8 * 16 + 2 * 24), 3 * 16 * 40
    assert part.state_need().shape == (conv_floats + rec_floats,) and part.right.state_offset == conv_floats and part.left.state_offset == 0
    assert part.cache_need().value_dim == 24
    inputs = [_bf(torch.randn(n, D, generator=g)) for n in (40, 2, 19)]
    rnd = pf.ident if dtype is torch.float32 else pf.bf16
    want = [pf.parallel_mixer(w, "p.", {"left": ml, "right": mr}, x.double(), EPS, F, rnd) for x in inputs]
    for name, cuts in CUTS.items():
        ctx = StateCtx(dtype, 3, Hkv=2, hd=16, vd=24, state_floats=conv_floats + rec_floats)
        got = _run_mixer(part, ctx, inputs, cuts, dtype, D)
        for r in range(3):
            _close(got[r], want[r], dtype, f"parallel mixer, request {r}, {name}", b16=3e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_requests_in_one_batch_equal_each_alone(dtype):
    """Three unequal requests batched against each alone, on scattered pages and other state slots: the same bits in 32-bit."""
    D = 40
    g = torch.Generator().manual_seed(17)
    for kind in ("left", "gla"):
        if kind == "left":
            w = _left_weights(D, LEFT, g)
            make = lambda: _left_part(D, LEFT, w, dtype)
            ctx_of = lambda part, n: _left_ctx(part, LEFT, dtype, n)
        else:
            w = _gla_weights(D, GLA, g)
            make = lambda: _gla_part(D, GLA, w, dtype)
            ctx_of = lambda part, n: StateCtx(dtype, n, state_floats=part.state_need().shape[0])
        part = make()
        inputs = [_bf(torch.randn(n, D, generator=g)) for n in (33, 5, 12)]
        together = _run_mixer(part, ctx_of(part, 3), inputs, [[20, 1, 3], [1, 1, 2], [12, 3, 7]], dtype, D)
        for r in range(3):
            alone = _run_mixer(part, ctx_of(part, 1), [inputs[r]], [[[20, 1, 3][r]], [[1, 1, 2][r]], [[12, 3, 7][r]]], dtype, D)
            assert torch.equal(alone[0], together[r]), f"{kind}: request {r} depends on its batch"


def test_hyper_connection_block_against_the_plain_layer():
    """A layer of three copies around a feed-forward only mixer stand-in: the block with the plain model's sublayer rule."""
    from geneinfer_b200.config import LayerSpec, PartSpec
    from geneinfer_b200.parts import BLOCKS, LayerRun
    D, S, T = 40, 3, 7
    g = torch.Generator().manual_seed(18)
    m = GLA
    w = _gla_weights(D, m, g, "l0.mix.")
    w.update({"l0.norm1": 0.2 * torch.randn(D, generator=g), "l0.norm2": 0.2 * torch.randn(D, generator=g),
              "l0.mlp.gate": _mat(56, D, g), "l0.mlp.up": _mat(56, D, g), "l0.mlp.down": _mat(D, 56, g)})
    for c in ("hc1", "hc2"):
        w[f"l0.{c}.in"], w[f"l0.{c}.out"], w[f"l0.{c}.mix"] = torch.randn(S, generator=g), torch.randn(S, generator=g), torch.randn(S, S, generator=g)
    norm = PartSpec("rmsnorm", {"size": D, "eps": EPS, "weight_offset": 1.0})
    spec = LayerSpec(mixer=PartSpec("gated_linear_attention", {"hidden_size": D, "num_heads": 3, "key_dim": 16, "value_dim": 40, "tau": 6.0, "norm_eps": EPS}),
                     feed_forward=PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": 56, "activation": "capped_swish", "activation_limit": 0.7}),
                     mixer_norm=norm, feed_forward_norm=norm, block="hyper_connections", block_params={"streams": S})
    p = "l0.mix."
    weights = {"mixer_norm.weight": w["l0.norm1"], "feed_forward_norm.weight": w["l0.norm2"],
               "mixer.w_in": torch.cat([w[p + "q"], w[p + "k"], w[p + "v"], w[p + "g"]]), "mixer.w_a1": w[p + "a1"], "mixer.w_a2": w[p + "a2"],
               "mixer.a2_bias": w[p + "a2.b"], "mixer.norm": w[p + "norm"], "mixer.w_o": w[p + "o"],
               "feed_forward.w_gate_up": torch.cat([w["l0.mlp.gate"], w["l0.mlp.up"]]), "feed_forward.w_down": w["l0.mlp.down"]}
    for c in ("hc1", "hc2"):
        for n in ("in", "out", "mix"):
            weights[f"{c}.{n}"] = w[f"l0.{c}.{n}"]
    block = BLOCKS["hyper_connections"](spec, weights, _build(torch.float32))
    x = torch.randn(T, D, generator=g)
    cfg = {"norm": {"eps": EPS}, "streams": S, "layers": [{"type": "parallel", "mixer": None, "mlp": {"limit": 0.7}}]}
    X = x.double()[None].repeat(S, 1, 1)
    X = pf.sublayer_streams(X, lambda h: pf.gated_linear_attention(w, p, m, h, EPS, F, pf.ident), w, "l0.hc1.", EPS, w["l0.norm1"])
    X = pf.sublayer_streams(X, lambda h: pf.feed_forward(w, "l0.mlp.", {"limit": 0.7}, h, F, pf.ident), w, "l0.hc2.", EPS, w["l0.norm2"])
    ctx = StateCtx(torch.float32, 1, state_floats=3 * 16 * 40)
    ctx.begin([T])
    xd = x.to(DEV).clone()
    block.forward(ctx, LayerRun(0, 0, True), xd)
    _close(xd.cpu(), X.sum(0), torch.float32, "the sum of the copies after the layer")
    assert cfg["streams"] == block.streams


# ------------------------------------------------------------------------------------------ whole models
_TMP = {}
LENGTHS = {"a": [1, 2, 3, 75, 20, 120, 47, 30], "b": [150, 4, 64, 1, 180], "c": [90, 2, 33, 1, 140, 17], "d": [1, 2, 100, 30, 7]}
CONFIGS = {"a": fc.FOV_A, "b": fc.FOV_B, "c": fc.FOV_C, "d": fc.FOV_D}
SEEDS = {"a": 23, "b": 31, "c": 37, "d": 41}


def _model_dir(case, tmp_path_factory):
    if case not in _TMP:
        _TMP[case] = fc.make_model_dir(CONFIGS[case], SEEDS[case], str(tmp_path_factory.mktemp("fovezen_" + case)), std=0.15)
    return _TMP[case]


def _requests(case):
    return {f"r{i}": tc.random_tokens(n, CONFIGS[case]["vocab"], 400 + i) for i, n in enumerate(LENGTHS[case])}


_PLAIN = {}


def _plain(case, folder, rounded=False, single=False):
    key = (case, rounded, single)
    if key not in _PLAIN:
        w, cfg = pf.load(folder)
        _PLAIN[key] = {rid: pf.forward(w, cfg, toks, torch.float32 if single else F, pf.bf16 if rounded else pf.ident).double().numpy()
                       for rid, toks in _requests(case).items()}
    return _PLAIN[key]


def _bound(exact, other, floor, times=3.0):
    """``times`` the distance between the plain model in two precisions, and at least ``floor``."""
    return max(floor, times * max(tt.rel_err(other[r], exact[r]) for r in exact))


def _tolerance(case, folder, dtype):
    """bfloat16: three times the distance between the exact plain model and the plain model with bfloat16 operands of the
    matrix products: the engine rounds at the same places, its sums run in other orders. 32-bit: 3e-5, or eight times the
    distance between the plain model in float64 and in float32 where that is more: a norm that follows a nearly cancelling sum
    (a query and a key at right angles at a sequence's first tokens, whose product is all that a head's memory holds yet)
    raises a position's 32-bit rounding far above 1e-5 in any 32-bit implementation, the plain one included, by a factor that
    depends on the order of its sums. (A wrong key, window, state or copy moves these models' logits by a tenth of their size.)"""
    if dtype == "float32":
        return _bound(_plain(case, folder), _plain(case, folder, single=True), 3e-5, 8.0)
    return _bound(_plain(case, folder), _plain(case, folder, True), 0.0)


def _engine(folder, dtype, n_pages, max_requests=4, page_size=16, max_step_tokens=512):
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    model = load_model(folder, dtype=dtype, max_position=512)
    return StepEngine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests, max_step_tokens=max_step_tokens,
                      debug_checks=True)


def _all_free(engine):
    return engine.cache.slots.free_count == engine.max_requests and all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_whole_prompts_decoding_portions_and_mixed_batches_agree_with_the_plain_model(case, dtype, tmp_path_factory):
    folder = _model_dir(case, tmp_path_factory)
    reqs, plain, tol = _requests(case), _plain(case, folder), _tolerance(case, folder, dtype)
    traces = {"whole": tt.trace_whole(reqs), "decode": tt.trace_tail_decode(reqs, tail=40), "portions": tt.trace_portions(reqs),
              "mixed": tt.trace_mixed(reqs, seed=3, tail=12), "mixed2": tt.trace_mixed(reqs, seed=8, max_live=3, tail=30)}
    results = {}
    for name, steps in traces.items():
        # the pool holds what the trace's live requests need, no more: pages and state slots are used again
        n_pages = tt.max_tokens_of(steps, reqs, 16) // 16 + (8 if name.startswith("mixed") else 0)
        engine = _engine(folder, dtype, n_pages)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"Fovezen {case} {dtype} {name}")
        engine.cache.check_invariants()
        assert _all_free(engine)
        results[name] = got
    if dtype == "float32":       # the same position under different cuts: equal but for rounding
        for name in ("decode", "portions", "mixed"):
            for key, row in results[name].items():
                ref = results["whole"][key]
                assert float(np.abs(row - ref).max()) < tol * max(1.0, float(np.abs(ref).max())), (name, key)


def test_the_stream_after_every_layer_run(tmp_path_factory):
    """The sum of the copies after each run of a layer (a looped layer counts every time), for a prompt fed whole and in portions."""
    folder = _model_dir("a", tmp_path_factory)
    w, cfg = pf.load(folder)
    toks = tc.random_tokens(45, 211, 6)
    after = []
    pf.forward(w, cfg, toks, layers_out=after)
    for sizes in ((45,), (7, 30, 2, 6)):
        engine = _engine(folder, "float32", n_pages=8)
        seen = []

        def tap(tag, layer, tensor, ctx):
            if tag == "ffn_out":
                seen.append((layer, tensor.detach().float().cpu()))
        engine.tap = tap
        tt.run_in_process(engine, tt.trace_portions({"r": toks}, sizes=sizes))
        runs = len(after)
        assert [l for l, _ in seen[:runs]] == pf.layer_order(cfg)
        for i in range(runs):
            got = torch.cat([t for _, t in seen[i::runs]])
            assert float((got.double() - after[i]).abs().max()) < 3e-5 * float(after[i].abs().max()), f"run {i}, portions {sizes}"


def test_passes_of_a_looped_layer_keep_caches_and_states_of_their_own(tmp_path_factory):
    folder = _model_dir("a", tmp_path_factory)
    engine = _engine(folder, "float32", n_pages=8)
    runs = engine.model.runs
    assert [r.layer for r in runs] == [0, 1, 0, 1, 0, 1, 2, 3] and len({r.cache_layer for r in runs}) == 8
    assert engine.model.layers[4] is engine.model.layers[0] and engine.model.layers[7] is engine.model.layers[1]
    assert sorted(engine.layer_state) == [0, 1, 3, 4, 5, 6, 7] and sorted(engine.layer_pages) == [1, 2, 3, 5, 7]
    assert len({t.data_ptr() for t in engine.layer_state.values()}) == 7


def test_long_decoding_under_graphs(tmp_path_factory):
    """170 tokens decoded one by one after a 12-token prompt, over page borders and past every window; CUDA graphs replay the steps."""
    folder = _model_dir("a", tmp_path_factory)
    toks = tc.random_tokens(182, 211, 77)
    w, cfg = pf.load(folder)
    want = {"r": pf.forward(w, cfg, toks).numpy()}
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folder, dtype, n_pages=12)
        got = tt.run_in_process(engine, tt.trace_tail_decode({"r": toks}, tail=170))
        tt.compare(got, want, _tolerance("a", folder, dtype), f"long decoding {dtype}")
        assert engine.graph_replays > 100 and _all_free(engine)


def test_state_slots_start_from_zero_when_they_are_used_again(tmp_path_factory):
    folder = _model_dir("c", tmp_path_factory)
    reqs = _requests("c")
    engine = _engine(folder, "float32", n_pages=20, max_requests=1)
    plain = _plain("c", folder)
    for rid in ("r0", "r4", "r2", "r0"):
        got = tt.run_in_process(engine, tt.trace_portions({rid: reqs[rid]}, sizes=(9, 2, 40)))
        tt.compare(got, plain, _tolerance("c", folder, "float32"), f"request {rid} on the one slot")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype, tmp_path_factory):
    from geneinfer_b200 import Engine
    folder = _model_dir("b", tmp_path_factory)
    w, cfg = pf.load(folder)
    prompts = [tc.random_tokens(n, 300, 900 + n) for n in (5, 40, 1, 18, 9)]
    engine = Engine(folder, dtype=dtype, max_seq_len=256, max_running=3, kv_pages=60, step_tokens=32, prefill_chunk=16)
    got = engine.generate(prompts, max_new_tokens=10, temperature=0.0)
    for prompt, gen in zip(prompts, got):
        assert len(gen) == 10
        tokens = list(prompt)
        for k, t in enumerate(gen):
            logits = pf.forward(w, cfg, tokens)[-1].numpy()
            best = int(np.argmax(logits))
            if t != best:                 # only a near-tie may differ
                assert float(logits[best] - logits[t]) < (1e-4 if dtype == "float32" else 8e-2), (k, t, best)
            tokens.append(t)
    assert engine.stats.max_running_seen == 3 and engine.steps.cache.slots.free_count == 3


@pytest.mark.parametrize("page_size", [8, 12, 64])
def test_other_page_sizes(page_size, tmp_path_factory):
    folder = _model_dir("b", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("b").items())[:3]}
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    for dtype in ("float32", "bfloat16"):
        steps = tt.trace_mixed(reqs, seed=2, tail=20)
        model = load_model(folder, dtype=dtype, max_position=384)
        engine = StepEngine(model, page_size=page_size, n_pages=tt.max_tokens_of(steps, reqs, 64) // page_size + 8, max_requests=4,
                            max_step_tokens=512, debug_checks=True)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, _plain("b", folder), _tolerance("b", folder, dtype), f"page size {page_size} {dtype}")


def test_trace_replay_tool_and_command_line(tmp_path, tmp_path_factory):
    folder = _model_dir("d", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("d").items())[1:5]}
    steps = tt.trace_mixed(reqs, seed=5, max_live=2, tail=6)
    got = tt.run_trace_tool(folder, "float32", steps, tt.max_tokens_of(steps, reqs), str(tmp_path / "out"), 77)
    tt.compare(got, _plain("d", folder), _tolerance("d", folder, "float32"), "trace replay")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", folder, "--prompt-ids", "5 9 2 70",
                        "--steps", "12", "--temperature", "0", "--no-echo", "--dtype", "fp32", "--max-seq-len", "64"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    out = [int(t) for t in p.stdout.split()]
    w, cfg = pf.load(folder)
    tokens = [5, 9, 2, 70]
    for t in out[:4]:
        logits = pf.forward(w, cfg, tokens)[-1].numpy()
        assert t == int(np.argmax(logits)) or float(logits.max() - logits[t]) < 1e-4
        tokens.append(t)
    assert len(out) == 9


def _random_config(seed):
    """A configuration drawn from a seed: sizes, layer order, copies, loop and constants all differ from case to case."""
    import random
    r = random.Random(seed)
    width = r.choice([64, 72, 96, 160, 176, 256, 320])
    layers = []

    def ff():
        return (r.choice([40, 64, 136, 320, 100]), r.choice([0.5, 1.0, 2.0, 7.0])) if r.random() < 0.75 else (None, 1.0)
    for _ in range(r.randint(1, 5)):
        kind = r.choice(["attention", "mamba2", "parallel"])
        f, limit = ff()
        if kind == "attention":
            kv = r.choice([1, 2, 3])
            dim = r.choice([16, 32, 48, 64, 96, 128])
            dims = r.choice([None, dim, dim // 2, 8])
            scaling = (r.choice([2.0, 8.0]), 1.0, r.choice([2.0, 4.0]), r.choice([16, 64, 2048])) if dims and r.random() < 0.6 else None
            layers.append(fc.attention(kv * r.choice([1, 2, 4]), kv, dim, r.choice([dim, 16, 48, 80]), r.choice([0.08, 0.125, 0.2]),
                                       rot=None if dims is None else fc.rot(r.choice([100.0, 10000.0, 250000.0]), dims, scaling), ff=f, limit=limit))
        elif kind == "mamba2":
            groups = r.choice([1, 2, 3])
            heads = groups * r.choice([1, 2, 4])
            vdim = r.choice([8, 16, 24, 48, 64])
            ng = r.choice([n for n in (1, 2, heads) if (heads * vdim) % n == 0])
            layers.append(fc.mamba2(heads, vdim, r.choice([8, 16, 48, 100]), groups, r.choice([1, 2, 3, 4]), ng, ff=f, limit=limit))
        else:
            kv = r.choice([1, 2, 4])
            dim = r.choice([16, 24, 32, 64, 80, 128])
            layers.append(fc.parallel(fc.left(kv * r.choice([1, 2, 3]), kv, dim, r.choice([dim, 16, 48, 96]), r.choice([0.1, 0.125, 0.3]),
                                              r.choice([None, 1, 3, 16, 17, 50, 96, 1000]), conv=r.choice([None, 1, 2, 3, 4]), softcap=r.choice([None, 5.0, 30.0])),
                                      fc.right(r.randint(1, 6), r.choice([8, 16, 32, 48, 72, 128]), r.choice([8, 16, 32, 40, 96]), r.choice([1.0, 4.0, 16.0]),
                                               r.choice([4, 8, 16, 20, 32])), ff=f, limit=limit))
    n = len(layers)
    loop = None
    if r.random() < 0.6:
        start = r.randint(0, n - 1)
        loop = (start, r.randint(start + 1, n), r.randint(1, 3))
    return fc.model(width, r.randint(50, 600), r.choice([1e-6, 1e-5, 1e-3]), layers, streams=r.choice([None, 1, 2, 3, 4]),
                    logit_scale=r.choice([None, 0.5, 1.7]), loop=loop)


@pytest.mark.parametrize("seed", range(int(os.environ.get("GENEINFER_TEST_SEEDS", "12"))))
def test_random_configurations_under_a_mixed_trace(seed, tmp_path):
    config = _random_config(seed)
    folder = fc.make_model_dir(config, 100 + seed, str(tmp_path / "m"), std=0.15)
    w, cfg = pf.load(folder)
    reqs = {f"r{i}": tc.random_tokens(n, config["vocab"], 700 + 10 * seed + i) for i, n in enumerate([130, 3, 61, 1, 200, 18])}
    exact = {rid: pf.forward(w, cfg, toks).numpy() for rid, toks in reqs.items()}
    rounded = {rid: pf.forward(w, cfg, toks, F, pf.bf16).numpy() for rid, toks in reqs.items()}
    single = {rid: pf.forward(w, cfg, toks, torch.float32).double().numpy() for rid, toks in reqs.items()}
    steps = tt.trace_mixed(reqs, seed=seed, tail=10)
    for dtype in ("float32", "bfloat16"):
        tol = _bound(exact, single, 3e-5, 8.0) if dtype == "float32" else _bound(exact, rounded, 0.0)
        engine = _engine(folder, dtype, tt.max_tokens_of(steps, reqs, 16) // 16 + 4)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, exact, tol, f"random configuration {seed} {dtype}: {config}")
        assert _all_free(engine)
