"""Pinorax on the GPU against the plain implementation in plain_pinorax.py: each kernel and each mechanism alone, then
whole models through the step engine under different cuts of the same requests (whole prompts, token-by-token
decoding, portions down to two tokens, mixed batches on reused pages), keys made to stand out far back, at page
borders and at the first position, and greedy generation through the engine's own entry point and scheduler."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import pinorax_configs as pc
import plain_pinorax as pp
import tiny_configs as tc
import trace_tools as tt
from test_gpu_nipadra import _run_mixer
from test_gpu_gekupel import PagesCtx

pytestmark = pytest.mark.gpu
DEV = torch.device("cuda:0")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = [torch.float32, torch.bfloat16]
F = torch.float64


def _build(dtype, max_position=4096):
    from geneinfer_b200.parts import BuildContext
    return BuildContext(DEV, dtype, max_position)


def _bf(t):
    return t.to(torch.bfloat16).float()


def _dbl(w):
    return {k: (v if v.dtype in (torch.int32, torch.int64) else v.double()) for k, v in w.items()}


def _close(got, want, dtype, what, f32=2e-5, b16=2e-2):
    err = float((got.double() - want.double()).abs().max() / max(1.0, float(want.abs().max())))
    assert err < (f32 if dtype is torch.float32 else b16), f"{what}: {err}"


# ------------------------------------------------------------------------------------------ kernels alone
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [200, 7, 4500])
def test_depth_mix_kernel(dtype, D):
    """Three layers' ends after one another: the history fills slot by slot, the stream becomes the weighted sum, y is
    cleared and the next layer's normed input comes out of the same pass."""
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(1)
    T, slots, m = 9, 4, 0.37
    x0 = torch.randn(T, D, generator=g) * 2
    ys = [torch.randn(T, D, generator=g) for _ in range(3)]
    ws = [torch.randn(s + 1, generator=g) for s in (1, 2, 3)]
    x = x0.to(DEV).clone()
    hist = torch.full((T, slots, D), float("nan"), device=DEV)
    results, stream = [x0.double()], x0.double()
    for s in (1, 2, 3):
        y = ys[s - 1].to(DEV).clone()
        xn = torch.full((T, D), float("nan"), dtype=dtype, device=DEV) if s != 2 else None
        gain = torch.tensor([1.3], device=DEV)
        bias = torch.randn(D, generator=g) if s == 2 else None          # a sublayer's bias left to this kernel
        kernels.depth_mix(x, y, m, hist, s, ws[s - 1].to(DEV), first=s == 1, next_weight=gain if xn is not None else None,
                          eps=1e-3, xn_out=xn, y_bias=None if bias is None else bias.to(DEV))
        results.append(stream + m * (ys[s - 1].double() + (bias.double() if bias is not None else 0.0)))
        stream = pp.depth_average(results, ws[s - 1].double())
        assert not y.any()
        _close(x.cpu(), stream, torch.float32, f"stream after slot {s}", f32=2e-6)
        _close(hist[:, s].cpu(), results[s], torch.float32, f"kept result {s}", f32=1e-6)
        if xn is not None:
            _close(xn.cpu().float(), pp.scalar_norm(stream, torch.tensor(1.3, dtype=F), 1e-3), dtype, f"normed input after slot {s}", f32=3e-6, b16=1e-2)
    _close(hist[:, 0].cpu(), x0, torch.float32, "slot 0 keeps what the first layer read", f32=1e-7)
    # without a history: x += m y
    x, y = x0.to(DEV).clone(), ys[0].to(DEV).clone()
    kernels.depth_mix(x, y, m)
    _close(x.cpu(), x0.double() + m * ys[0].double(), torch.float32, "no history", f32=1e-6)
    assert not y.any()


@pytest.mark.parametrize("dtype", DTYPES)
def test_small_elementwise_kernels(dtype):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(2)
    T, D, rows = 11, 52, 30
    x, table = torch.randn(T, D, generator=g), _bf(torch.randn(rows, D, generator=g))
    index = torch.tensor([0, 29, 3, 3, 17, 1, 2, 28, 5, 9, 0], dtype=torch.int32)
    xd = x.to(DEV).clone()
    kernels.add_rows_at(xd, table.to(DEV).to(dtype), index.to(DEV))
    _close(xd.cpu(), x + table[index.long()], torch.float32, "add_rows_at", f32=1e-7)
    b = torch.randn(D, generator=g)
    kernels.add_bias(xd, b.to(DEV))
    _close(xd.cpu(), x + table[index.long()] + b, torch.float32, "add_bias", f32=1e-7)
    a, gate = torch.randn(T, 20, generator=g), torch.randn(T, 47, generator=g) * 3
    out = torch.empty(T, 20, dtype=dtype, device=DEV)
    kernels.sigmoid_gate(a.to(DEV), gate.to(DEV), 27, out)
    _close(out.cpu().float(), a.double() * torch.sigmoid(gate[:, 27:].double()), dtype, "sigmoid_gate", f32=1e-6, b16=1e-2)
    z = torch.randn(T, 33, generator=g) * 40
    zd = z.to(DEV).clone()
    kernels.softcap(zd, 12.5)
    _close(zd.cpu(), pp.softcap(z.double(), 12.5), torch.float32, "softcap", f32=1e-6)
    assert float(zd.abs().max()) <= 12.5


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T", [3, 40, 200])
@pytest.mark.parametrize("H, N, K", [(3, 40, 48), (5, 7, 30), (2, 72, 64)])
def test_head_product_with_an_output_gate(dtype, T, H, N, K):
    """A matrix per head and, in the same kernel, the sigmoid of a gate value per output (few rows, tiles of 16, tiles of 64)."""
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(6)
    a = torch.randn(T, H * K, generator=g)
    w = _bf(torch.randn(H, N, K, generator=g) * 0.3)
    gate = torch.randn(T, 11 + H * N + 3, generator=g) * 2
    want = torch.einsum("thk,hnk->thn", a.view(T, H, K).double(), w.double()).reshape(T, H * N) * torch.sigmoid(gate[:, 11:11 + H * N].double())
    for out_dtype in (torch.float32, dtype):
        out = torch.full((T, H * N), float("nan"), dtype=out_dtype, device=DEV)
        kernels.head_product(a.to(DEV), 0, K, w.to(DEV).to(dtype), out, 0, N, gate=gate.to(DEV), gate_offset=11)
        _close(out.cpu().float(), want, out_dtype, "gated head product", f32=1e-5, b16=1e-2)
    with pytest.raises(Exception, match="gate"):
        kernels.head_product(a.to(DEV), 0, K, w.to(DEV).to(dtype), out, 0, N, gate=gate.to(DEV), gate_offset=15)


@pytest.mark.parametrize("I", [24, 7])
@pytest.mark.parametrize("biased", [False, True])
def test_capped_activation(I, biased):
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(3)
    gu = torch.randn(13, 2 * I, generator=g) * 3
    bias = torch.randn(2 * I, generator=g) if biased else None
    z = gu.double() + (bias.double() if biased else 0.0)
    gate, up = torch.clamp(z[:, :I], max=1.5), torch.clamp(z[:, I:], -1.5, 1.5)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1.0)
    assert float((z[:, :I] > 1.5).float().mean()) > 0.1 and float((z[:, I:].abs() > 1.5).float().mean()) > 0.2
    for dtype in DTYPES:
        out = torch.empty(13, I, dtype=dtype, device=DEV)
        kernels.gated_act(gu.to(DEV), out, "capped_swish", 1.5, None if bias is None else bias.to(DEV))
        _close(out.cpu().float(), want, dtype, "capped swish", f32=1e-6, b16=1e-2)
    silu = z[:, :I] * torch.sigmoid(z[:, :I]) * z[:, I:]
    out = torch.empty(13, I, device=DEV)
    kernels.gated_act(gu.to(DEV), out, "silu", 0.0, None if bias is None else bias.to(DEV))
    _close(out.cpu(), silu, torch.float32, "silu with a bias", f32=1e-6)


@pytest.mark.parametrize("T, E, top, tile_rows", [(19, 5, 2, None), (300, 7, 3, 128), (4, 3, 1, None), (33, 4, 4, None)])
def test_route_table_kernel(T, E, top, tile_rows):
    """The experts of a row are the table's row of its token id; a token named by its place in the feedback buffer is
    looked up there. Every pair lands in one tile of its expert."""
    from geneinfer_b200.ops import kernels
    g = torch.Generator().manual_seed(4)
    vocab = 41
    table = torch.rand(vocab, E, generator=g).argsort(1)[:, :top].int()
    tokens = torch.randint(0, vocab, (T,), generator=g).int()
    feedback = torch.randint(0, vocab, (8,), generator=g).int()
    real = tokens.clone()
    tokens[1], real[1] = -4, feedback[3]
    tm = tile_rows or kernels.grouped_tile_rows()
    tiles = kernels.route_tiles(T, top, E, tm)
    ids = torch.full((T, top), -1, dtype=torch.int32, device=DEV)
    wts = torch.full((T, top), float("nan"), device=DEV)
    srt = torch.full((tiles * tm,), -9, dtype=torch.int32, device=DEV)
    grp = torch.full((tiles,), -9, dtype=torch.int32, device=DEV)
    cnt = torch.zeros(1, dtype=torch.int32, device=DEV)
    pair_row = torch.full((T * top,), -9, dtype=torch.int32, device=DEV) if tile_rows else None
    kernels.route_table(tokens.to(DEV), feedback.to(DEV), table.to(DEV), E, ids, wts, srt, grp, cnt, tile_rows=tile_rows, pair_row=pair_row)
    assert torch.equal(ids.cpu(), table[real.long()])
    assert torch.equal(wts.cpu(), torch.full((T, top), 1.0 / top))
    n = int(cnt.item())
    pairs = srt.cpu()[:n * tm]
    assert sorted(pairs[pairs >= 0].tolist()) == list(range(T * top))
    for i in range(n):
        mine = pairs[i * tm:(i + 1) * tm]
        assert all(int(ids.view(-1)[p]) == int(grp[i]) for p in mine[mine >= 0].tolist())
    if pair_row is not None:
        where = pair_row.cpu()
        assert all(int(pairs[where[p]]) == p for p in range(T * top))


# ------------------------------------------------------------------------------------------ mechanisms alone
def test_scalar_norm_and_learned_positions():
    from geneinfer_b200.parts import NORMS, POSITION_ENCODINGS
    g = torch.Generator().manual_seed(5)
    for dtype in DTYPES:
        x = torch.randn(6, 70, generator=g) * 3
        norm = NORMS["rmsnorm_scalar"]({"size": 70, "eps": 1e-4}, {"weight": torch.tensor(0.8)}, _build(dtype))
        out = torch.empty(6, 70, dtype=dtype, device=DEV)
        norm.forward(x.to(DEV), out)
        _close(out.cpu().float(), pp.scalar_norm(x.double(), torch.tensor(0.8, dtype=F), 1e-4), dtype, "scalar norm", f32=2e-6, b16=1e-2)
        with pytest.raises(ValueError, match="expected one"):
            NORMS["rmsnorm_scalar"]({"size": 70, "eps": 1e-4}, {"weight": torch.ones(70)}, _build(dtype))
        table = _bf(torch.randn(40, 70, generator=g))
        part = POSITION_ENCODINGS["learned"]({"size": 70, "positions": 40}, {"table": table}, _build(dtype, 40))

        class Ctx:
            positions = torch.tensor([0, 39, 7, 8, 9, 0], dtype=torch.int32, device=DEV)
        xd = x.to(DEV).clone()
        part.add_to(Ctx, xd)
        _close(xd.cpu(), x + table[Ctx.positions.cpu().long()], torch.float32, "learned positions", f32=1e-7)
        with pytest.raises(ValueError, match="context length"):      # no vector for a position beyond the table
            POSITION_ENCODINGS["learned"]({"size": 70, "positions": 40}, {"table": table}, _build(dtype, 41))


CUTS = {"whole": [[40]], "decode": [[1]] * 40, "portions": [[2], [3], [11], [2], [1], [9], [2], [10]], "tail": [[23]] + [[1]] * 17}
# one form that the CUDA-core attention runs in both precisions, one that the tensor cores run in bfloat16
LAT = {"small": {"heads": 3, "dim": 24, "vdim": 40, "kv_rank": 48, "scale": 0.3},
       "wide": {"heads": 8, "dim": 16, "vdim": 24, "kv_rank": 64, "scale": 0.22},
       "one": {"heads": 1, "dim": 20, "vdim": 12, "kv_rank": 36, "scale": 0.4}}


def _lat_weights(D, m, g, std=0.25):
    H, d, dv, kr = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    rn = lambda *s: _bf(torch.randn(*s, generator=g) * std)      # noqa: E731
    return {"q": rn(H * d, D), "dkv": rn(kr, D), "dkv.norm": 1 + 0.2 * torch.randn(kr, generator=g), "uk": rn(H * d, kr),
            "uv": rn(H * dv, kr), "g": rn(H * dv, D), "o": rn(D, H * dv), "sink": torch.randn(H, generator=g)}


def _lat_part(D, m, w, dtype, gate=True):
    from geneinfer_b200.parts import MIXERS
    params = {"hidden_size": D, "num_heads": m["heads"], "head_dim": m["dim"], "rotary_dim": 0, "value_dim": m["vdim"], "q_rank": None,
              "kv_rank": m["kv_rank"], "scale": m["scale"], "window": None, "norm_eps": 1e-5, "position": None, "sink": "learned",
              "output_gate": gate}
    weights = {"w_down": torch.cat([w["q"], w["dkv"]] + ([w["g"]] if gate else [])), "kv_latent_norm": w["dkv.norm"], "w_uk": w["uk"],
               "w_uv": w["uv"], "w_o": w["o"], "sink": w["sink"]}
    return MIXERS["latent_attention"](params, weights, _build(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("form", sorted(LAT))
@pytest.mark.parametrize("cut", sorted(CUTS))
def test_latent_mixer_under_every_cut(dtype, form, cut):
    D, m = 56, LAT[form]
    g = torch.Generator().manual_seed(8)
    w = _lat_weights(D, m, g)
    part = _lat_part(D, m, w, dtype)
    need = part.cache_need()
    assert (need.num_kv_heads, need.head_dim, need.value_width, need.window) == (1, m["kv_rank"], 0, None)
    x = _bf(torch.randn(40, D, generator=g))
    want = pp.latent_attention(x.double(), m, _dbl(w), 1e-5, pp.ident if dtype is torch.float32 else pp.bf16)
    got = _run_mixer(part, PagesCtx(dtype, 1, 1, m["kv_rank"], 0), [x], CUTS[cut], dtype, D)[0]
    _close(got, want, dtype, f"latent mixer {form}, {cut}", b16=3e-2)


def test_the_output_gate_and_the_sink_are_part_of_the_result():
    """Leaving either out moves the output: the engine's result equals the plain mixer only with both."""
    D, m = 56, LAT["small"]
    g = torch.Generator().manual_seed(9)
    w = _lat_weights(D, m, g)
    x = _bf(torch.randn(30, D, generator=g))
    want = pp.latent_attention(x.double(), m, _dbl(w), 1e-5)
    got = _run_mixer(_lat_part(D, m, w, torch.float32), PagesCtx(torch.float32, 1, 1, 48, 0), [x], [[30]], torch.float32, D)[0]
    _close(got, want, torch.float32, "gated mixer")
    no_gate = _run_mixer(_lat_part(D, m, w, torch.float32, gate=False), PagesCtx(torch.float32, 1, 1, 48, 0), [x], [[30]], torch.float32, D)[0]
    assert float((no_gate - want).abs().max()) > 0.05
    no_sink = dict(_dbl(w), sink=torch.full((3,), -40.0, dtype=F))
    assert float((pp.latent_attention(x.double(), m, no_sink, 1e-5) - want).abs().max()) > 0.02


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("form", ["small", "wide"])
def test_requests_in_one_batch_equal_each_alone(dtype, form):
    """Unequal requests side by side, one sitting steps out, on scattered pages: each equals its run alone."""
    D, m = 56, LAT[form]
    g = torch.Generator().manual_seed(10)
    w = _lat_weights(D, m, g)
    part = _lat_part(D, m, w, dtype)
    xs = [_bf(torch.randn(n, D, generator=g)) for n in (37, 9, 22)]
    cuts = [[5, 0, 1], [1, 2, 1], [20, 0, 1], [1, 7, 0], [10, 0, 19]]
    got = _run_mixer(part, PagesCtx(dtype, 3, 1, m["kv_rank"], 0), xs, cuts, dtype, D)
    for r, x in enumerate(xs):
        alone = _run_mixer(part, PagesCtx(dtype, 1, 1, m["kv_rank"], 0), [x], [[len(x)]], dtype, D)[0]
        _close(got[r], alone, dtype, f"request {r} in a batch", f32=2e-6, b16=1.5e-2)
        _close(got[r], pp.latent_attention(x.double(), m, _dbl(w), 1e-5), dtype, f"request {r} against the plain mixer", b16=4e-2)


def _sharp(D, m, g):
    """Weights in which input feature 0 makes a strong key and feature 1 a query that asks for it, in every head."""
    w = _lat_weights(D, m, g, std=0.1)
    for name in ("q", "dkv"):
        w[name][:, :2] = 0
    w["dkv"][0, 0] = 3.0
    w["uk"][:] = 0
    for h in range(m["heads"]):
        w["q"][h * m["dim"], 1] = 1.0            # the head's first query dimension reads feature 1
        w["uk"][h * m["dim"], 0] = 1.0           # its first key dimension the latent's first value
    return w


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("form", ["small", "wide"])
@pytest.mark.parametrize("decoded", [False, True])
@pytest.mark.parametrize("qi, ki", [(700, 0), (700, 1), (650, 7), (650, 8), (703, 15), (703, 16), (640, 639), (640, 640), (641, 642)])
def test_one_key_among_hundreds(qi, ki, decoded, form, dtype):
    """No window: a key hundreds of positions back (the first token, either side of a page border) decides the output,
    as a prompt portion and token by token; a key that comes after the query does not count."""
    D, T, m = 56, 720, LAT[form]
    g = torch.Generator().manual_seed(14)
    w = _sharp(D, m, g)
    part = _lat_part(D, m, w, dtype)
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[ki, 0] = 6.0
    x[qi, 1] = 6.0
    x = _bf(x)
    cuts = [[T]] if not decoded else [[qi - 2]] + [[1]] * (T - qi + 2)
    got = _run_mixer(part, PagesCtx(dtype, 1, 1, m["kv_rank"], 0, max_len=768), [x], cuts, dtype, D)[0]
    want = pp.latent_attention(x.double(), m, _dbl(w), 1e-5)
    _close(got[qi - 3:], want[qi - 3:], dtype, f"query {qi}, key {ki}", b16=3e-2)
    x2 = x.clone()
    x2[ki, 0] = 0
    moved = float((pp.latent_attention(x2.double(), m, _dbl(w), 1e-5)[qi] - want[qi]).abs().max())
    assert (moved > 0.05) == (ki <= qi), f"the key {ki} moves the query {qi} by {moved}"


def test_with_no_key_worth_seeing_the_sink_takes_the_weight():
    D, T, m, dtype = 56, 50, LAT["small"], torch.float32
    g = torch.Generator().manual_seed(15)
    w = _sharp(D, m, g)
    w["sink"][:] = torch.tensor([4.0, 0.0, -4.0])
    x = 0.3 * torch.randn(T, D, generator=g)
    x[:, :2] = 0
    x[45, 1] = -6.0                  # a query that scores every key low: what is left over goes to the sink
    x[10:20, 0] = 6.0
    x = _bf(x)
    want = pp.latent_attention(x.double(), m, _dbl(w), 1e-5)
    for cuts in ([[T]], [[40]] + [[1]] * 10):
        got = _run_mixer(_lat_part(D, m, w, dtype), PagesCtx(dtype, 1, 1, 48, 0), [x], cuts, dtype, D)[0]
        _close(got, want, dtype, "sink")
    flat = dict(_dbl(w), sink=torch.zeros(3, dtype=F))
    assert float((pp.latent_attention(x.double(), m, flat, 1e-5)[45] - want[45]).abs().max()) > 0.01


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows", [5, 200])
def test_dense_feed_forward_with_biases(dtype, rows):
    from geneinfer_b200.parts import FEED_FORWARDS
    g = torch.Generator().manual_seed(11)
    D, I = 64, 88
    w = {"gate": _bf(torch.randn(I, D, generator=g) * 0.2), "up": _bf(torch.randn(I, D, generator=g) * 0.2),
         "down": _bf(torch.randn(D, I, generator=g) * 0.2), "gate.b": torch.randn(I, generator=g), "up.b": torch.randn(I, generator=g),
         "down.b": torch.randn(D, generator=g)}
    part = FEED_FORWARDS["gated_mlp"]({"hidden_size": D, "intermediate_size": I, "activation": "silu", "bias": True},
                                      {"w_gate_up": torch.cat([w["gate"], w["up"]]), "b_gate_up": torch.cat([w["gate.b"], w["up.b"]]),
                                       "w_down": w["down"], "b_down": w["down.b"]}, _build(dtype))
    x = _bf(torch.randn(rows, D, generator=g))
    y = torch.ones(rows, D, device=DEV)
    part.forward(PagesCtx(dtype, 1, 1, 8, 8), x.to(DEV).to(dtype), y)
    want = 1.0 + pp.dense_ff(x.double(), _dbl(w), pp.ident if dtype is torch.float32 else pp.bf16)
    _close(y.cpu(), want, dtype, "dense feed-forward with biases", b16=1.5e-2)
    no_bias = dict(_dbl(w), **{k: torch.zeros_like(w[k]).double() for k in ("gate.b", "up.b", "down.b")})
    assert float((1.0 + pp.dense_ff(x.double(), no_bias) - want).abs().max()) > 0.3


def _experts(D, I, E, top, vocab, shared, g):
    w = {"table": torch.rand(vocab, E, generator=g).argsort(1)[:, :top].int()}
    for e in range(E):
        w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"] = (_bf(torch.randn(*s, generator=g) * 0.3) for s in ((I, D), (I, D), (D, I)))
    if shared:
        w["shared.gate"], w["shared.up"], w["shared.down"] = (_bf(torch.randn(*s, generator=g) * 0.3) for s in ((shared, D), (shared, D), (D, shared)))
    return w


def _experts_part(D, I, E, top, vocab, shared, limits, w, dtype):
    from geneinfer_b200.parts import FEED_FORWARDS
    weights = {"table": w["table"], "w_gate_up": torch.stack([torch.cat([w[f"e{e}.gate"], w[f"e{e}.up"]]) for e in range(E)]),
               "w_down": torch.stack([w[f"e{e}.down"] for e in range(E)])}
    sh = None
    if shared:
        sh = {"hidden_size": D, "intermediate_size": shared, "activation": "capped_swish", "activation_limit": limits[1]}
        weights["shared.w_gate_up"], weights["shared.w_down"] = torch.cat([w["shared.gate"], w["shared.up"]]), w["shared.down"]
    return FEED_FORWARDS["routed_experts"]({"hidden_size": D, "intermediate_size": I, "experts": E, "top": top, "activation": "capped_swish",
                                            "activation_limit": limits[0], "router": "table", "vocab_size": vocab, "shared": sh},
                                           weights, _build(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("T, E, top, D, I, shared", [(30, 5, 2, 48, 40, 24), (300, 6, 2, 64, 40, 72), (9, 3, 1, 56, 20, 0), (400, 4, 3, 72, 8, 16),
                                                      (17, 2, 2, 50, 14, 6)])
def test_experts_by_token_id_with_a_shared_expert(dtype, T, E, top, D, I, shared):
    """Few pairs run on the CUDA cores, many (bfloat16) on the tensor cores; a token's experts depend on its id alone."""
    g = torch.Generator().manual_seed(12)
    vocab, limits = 37, (0.7, 1.9)
    w = _experts(D, I, E, top, vocab, shared, g)
    part = _experts_part(D, I, E, top, vocab, shared, limits, w, dtype)
    x = _bf(torch.randn(T, D, generator=g))
    tokens = torch.randint(0, vocab, (T,), generator=g)
    ctx = PagesCtx(dtype, 1, 1, 8, 8)
    ctx.max_step_tokens = 1024
    ctx.tokens, ctx.feedback = tokens.int().to(DEV), None
    y = torch.zeros(T, D, device=DEV)
    part.forward(ctx, x.to(DEV).to(dtype), y)
    mlp = {"router": {"top": top}, "expert": {"limit": limits[0]}, "shared": {"limit": limits[1]} if shared else None}
    want = pp.table_experts(x.double(), tokens.tolist(), mlp, _dbl(w), pp.ident if dtype is torch.float32 else pp.bf16)
    _close(y.cpu(), want, dtype, "experts by token id", b16=1.5e-2)
    # the same rows under other ids give other results; the same id gives the same
    ctx.tokens = ((tokens + 1) % vocab).int().to(DEV)
    y2 = torch.zeros(T, D, device=DEV)
    part.forward(ctx, x.to(DEV).to(dtype), y2)
    assert top == E or float((y2 - y).abs().max()) > 0.05
    with pytest.raises(ValueError, match="twice|outside"):
        bad = dict(w, table=torch.zeros(vocab, top, dtype=torch.int32) + (E if top == 1 else 0))
        _experts_part(D, I, E, top, vocab, shared, limits, bad, dtype)


# ------------------------------------------------------------------------------------------ whole models
_TMP = {}
LENGTHS = {"a": [1, 2, 3, 75, 20, 120, 47, 30], "b": [150, 4, 64, 1, 99], "c": [90, 2, 33, 1, 140, 17], "d": [1, 2, 100, 30, 7]}
CONFIGS = {"a": pc.PIN_A, "b": pc.PIN_B, "c": pc.PIN_C, "d": pc.PIN_D}
SEEDS = {"a": 23, "b": 31, "c": 37, "d": 41}


def _model_dir(case, tmp_path_factory):
    if case not in _TMP:
        _TMP[case] = pc.make_model_dir(CONFIGS[case], SEEDS[case], str(tmp_path_factory.mktemp("pinorax_" + case)), std=0.2)
    return _TMP[case]


def _requests(case):
    return {f"r{i}": tc.random_tokens(n, CONFIGS[case]["vocab"], 400 + i) for i, n in enumerate(LENGTHS[case])}


_PLAIN = {}


def _plain(case, folder, rounded=False):
    key = (case, rounded)
    if key not in _PLAIN:
        cfg, w = pp.load(folder)
        _PLAIN[key] = {rid: pp.forward(cfg, w, toks, pp.bf16 if rounded else pp.ident)[0].numpy() for rid, toks in _requests(case).items()}
    return _PLAIN[key]


def _tolerance(case, folder, dtype):
    """32-bit: rounding of the logits' size. bfloat16: the engine rounds at other places than the plain model's ``bf16``
    (it applies the heads' key matrices to the queries), so it is compared with the exact plain model and allowed three
    times the distance between the plain model's two precisions."""
    if dtype == "float32":
        return 3e-5
    exact, rounded = _plain(case, folder), _plain(case, folder, True)
    return 3.0 * max(tt.rel_err(rounded[r], exact[r]) for r in exact)


def _engine(folder, dtype, n_pages, max_requests=4, page_size=16, max_step_tokens=512):
    from geneinfer_b200.engine.loading import load_model
    from geneinfer_b200.engine.step import StepEngine
    model = load_model(folder, dtype=dtype, max_position=512)
    return StepEngine(model, page_size=page_size, n_pages=n_pages, max_requests=max_requests, max_step_tokens=max_step_tokens,
                      debug_checks=True)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("case", ["a", "b", "c", "d"])
def test_whole_prompts_decoding_portions_and_mixed_batches_agree_with_the_plain_model(case, dtype, tmp_path_factory):
    folder = _model_dir(case, tmp_path_factory)
    reqs, plain, tol = _requests(case), _plain(case, folder), _tolerance(case, folder, dtype)
    traces = {"whole": tt.trace_whole(reqs), "decode": tt.trace_tail_decode(reqs, tail=40), "portions": tt.trace_portions(reqs),
              "mixed": tt.trace_mixed(reqs, seed=3, tail=12), "mixed2": tt.trace_mixed(reqs, seed=8, max_live=3, tail=30)}
    results = {}
    for name, steps in traces.items():
        # the pool holds what the trace's live requests need, no more: pages are used again
        n_pages = tt.max_tokens_of(steps, reqs, 16) // 16 + (8 if name.startswith("mixed") else 0)
        engine = _engine(folder, dtype, n_pages)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, plain, tol, f"Pinorax {case} {dtype} {name}")
        engine.cache.check_invariants()
        assert engine.cache.slots.free_count == 4 and all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)
        results[name] = got
    if dtype == "float32":       # the same position under different cuts: equal but for rounding
        for name in ("decode", "portions", "mixed"):
            for key, row in results[name].items():
                ref = results["whole"][key]
                assert float(np.abs(row - ref).max()) < 2e-5 * max(1.0, float(np.abs(ref).max())), (name, key)


def test_the_stream_after_every_layer(tmp_path_factory):
    """What goes on after each layer (its result mixed with all earlier ones), against the plain model, for a prompt
    fed whole and in portions: the kept results of a step's rows are its own."""
    folder = _model_dir("a", tmp_path_factory)
    cfg, w = pp.load(folder)
    toks = tc.random_tokens(45, 190, 6)
    _, after = pp.forward(cfg, w, toks)
    for sizes in ((45,), (7, 30, 2, 6)):
        engine = _engine(folder, "float32", n_pages=8)
        seen = {}

        def tap(tag, layer, tensor, ctx):
            if tag == "ffn_out":
                seen.setdefault(layer, []).append(tensor.detach().float().cpu())
        engine.tap = tap
        tt.run_in_process(engine, tt.trace_portions({"r": toks}, sizes=sizes))
        for i in range(len(cfg["layers"])):
            got = torch.cat(seen[i])
            assert float((got.double() - after[i]).abs().max()) < 2e-5 * float(after[i].abs().max()), f"layer {i}, portions {sizes}"


def test_long_decoding_under_graphs(tmp_path_factory):
    """160 tokens decoded one by one after a 12-token prompt, over page borders; CUDA graphs replay the steps."""
    folder = _model_dir("a", tmp_path_factory)
    toks = tc.random_tokens(172, 190, 77)
    cfg, w = pp.load(folder)
    want = {"r": pp.forward(cfg, w, toks)[0].numpy()}
    for dtype in ("float32", "bfloat16"):
        engine = _engine(folder, dtype, n_pages=11)
        got = tt.run_in_process(engine, tt.trace_tail_decode({"r": toks}, tail=160))
        tt.compare(got, want, _tolerance("a", folder, dtype), f"long decoding {dtype}")
        assert engine.graph_replays > 100
        assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)


def test_no_position_beyond_the_table(tmp_path_factory):
    """The design has a vector for ``max_positions`` positions: the engine's context length is at most that."""
    folder = _model_dir("d", tmp_path_factory)
    engine = _engine(folder, "float32", n_pages=16)
    assert engine.model.max_position == 128
    toks = tc.random_tokens(128, 77, 3)
    cfg, w = pp.load(folder)
    got = tt.run_in_process(engine, tt.trace_portions({"r": toks}, sizes=(100, 27, 1)))
    tt.compare(got, {"r": pp.forward(cfg, w, toks)[0].numpy()}, 3e-5, "up to the last position")
    from geneinfer_b200.engine.step import StepEntry
    engine.open("long")
    with pytest.raises(Exception):
        engine.step([StepEntry("long", tc.random_tokens(129, 77, 4), [128])])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_greedy_generation_through_the_engine_and_its_scheduler(dtype, tmp_path_factory):
    from geneinfer_b200 import Engine
    folder = _model_dir("b", tmp_path_factory)
    cfg, w = pp.load(folder)
    prompts = [tc.random_tokens(n, 260, 900 + n) for n in (5, 40, 1, 18, 9)]
    engine = Engine(folder, dtype=dtype, max_seq_len=256, max_running=3, kv_pages=40, step_tokens=32, prefill_chunk=16)
    got = engine.generate(prompts, max_new_tokens=10, temperature=0.0)
    for prompt, gen in zip(prompts, got):
        assert len(gen) == 10
        tokens = list(prompt)
        for k, t in enumerate(gen):
            logits = pp.forward(cfg, w, tokens)[0][-1].numpy()
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
    folder = _model_dir("a", tmp_path_factory)
    reqs = {k: v for k, v in list(_requests("a").items())[3:6]}
    steps = tt.trace_mixed(reqs, seed=5, max_live=2, tail=6)
    got = tt.run_trace_tool(folder, "float32", steps, tt.max_tokens_of(steps, reqs), str(tmp_path / "out"), 190)
    tt.compare(got, _plain("a", folder), 3e-5, "trace replay")
    p = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "gi_generate"), "--model", folder, "--prompt-ids", "5 9 2 100",
                        "--steps", "12", "--temperature", "0", "--no-echo", "--dtype", "fp32", "--max-seq-len", "64"],
                       capture_output=True, text=True, timeout=600)
    assert p.returncode == 0, p.stderr
    out = [int(t) for t in p.stdout.split()]
    cfg, w = pp.load(folder)
    tokens = [5, 9, 2, 100]
    for t in out[:4]:
        logits = pp.forward(cfg, w, tokens)[0][-1].numpy()
        assert t == int(np.argmax(logits)) or float(logits.max() - logits[t]) < 1e-4
        tokens.append(t)
    assert len(out) == 9


def _random_config(seed):
    """A configuration drawn from a seed: sizes, layer order, feed-forward kinds and constants all differ from case to case."""
    import random
    r = random.Random(seed)
    width = r.choice([64, 72, 96, 160, 176, 256])
    layers = []
    for _ in range(r.randint(1, 7)):
        kind = r.choice(["none", "dense", "moe", "moe", "moe"])
        if kind == "none":
            mlp = None
        elif kind == "dense":
            mlp = pc.dense(r.choice([40, 64, 136, 320, 100]))
        else:
            experts = r.randint(2, 16)
            shared = (r.choice([8, 24, 64, 128]), r.choice([0.5, 1.5, 3.0])) if r.random() < 0.7 else None
            mlp = pc.moe(r.choice([8, 24, 48, 88, 44]), r.choice([0.5, 1.0, 2.0, 7.0]), experts, r.randint(1, min(4, experts)), shared=shared)
        layers.append(pc.layer(r.randint(1, 12), r.choice([8, 16, 32, 64, 96]), r.choice([8, 16, 40, 64, 72, 128]),
                               r.choice([16, 32, 64, 80, 128, 192, 256]), r.choice([0.08, 0.125, 0.2, 0.3]), mlp))
    return pc.model(width, r.randint(50, 600), 256, r.choice([1e-6, 1e-5, 1e-3]), r.choice([0.3, 0.5, 1.0, 1.4]),
                    r.choice([5.0, 15.0, 30.0, 100.0]), layers)


@pytest.mark.parametrize("seed", range(8))
def test_random_configurations_under_a_mixed_trace(seed, tmp_path):
    config = _random_config(seed)
    folder = pc.make_model_dir(config, 100 + seed, str(tmp_path / "m"), std=0.15)
    cfg, w = pp.load(folder)
    reqs = {f"r{i}": tc.random_tokens(n, config["vocab"], 700 + 10 * seed + i) for i, n in enumerate([130, 3, 61, 1, 200, 18])}
    exact = {rid: pp.forward(cfg, w, toks)[0].numpy() for rid, toks in reqs.items()}
    rounded = {rid: pp.forward(cfg, w, toks, pp.bf16)[0].numpy() for rid, toks in reqs.items()}
    steps = tt.trace_mixed(reqs, seed=seed, tail=10)
    for dtype in ("float32", "bfloat16"):
        tol = 3e-5 if dtype == "float32" else 3.0 * max(tt.rel_err(rounded[r], exact[r]) for r in exact)
        engine = _engine(folder, dtype, tt.max_tokens_of(steps, reqs, 16) // 16 + 4)
        got = tt.run_in_process(engine, steps)
        engine.check_status()
        tt.compare(got, exact, tol, f"random configuration {seed} {dtype}")
        assert all(g.pool.free_count == g.pool.n_pages for g in engine.cache.groups)
