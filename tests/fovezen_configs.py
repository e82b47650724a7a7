"""Small Fovezen configurations for the tests: sizes that differ from one another in every field, with values that a
particular model may happen to make equal (key and value sizes, heads and key/value heads, rotary and head size) or 1
(streams, groups, norm groups, loop passes) chosen apart."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def mlp(ff, limit):
    return None if ff is None else {"ff": ff, "kind": "dense", "limit": limit}


def attention(heads, kv_heads, dim, vdim, scale, rot=None, ff=None, limit=1.0):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if rot is not None:
        m["rot"] = rot
    return {"type": "attention", "mixer": m, "mlp": mlp(ff, limit)}


def rot(base, dims, scaling=None):
    r = {"base": base, "dims": dims}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    return r


def mamba2(heads, vdim, state, groups, conv, norm_groups, ff=None, limit=1.0):
    return {"type": "mamba2", "mixer": {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "conv": conv,
                                        "norm_groups": norm_groups}, "mlp": mlp(ff, limit)}


def left(heads, kv_heads, dim, vdim, scale, window, conv=None, softcap=None):
    m = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale}
    if window is not None:
        m["mask"] = {"size": window}
    if conv is not None:
        m["conv"] = conv
    if softcap is not None:
        m["softcap"] = softcap
    return m


def right(heads, dim, vdim, tau, rank):
    return {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau, "rank": rank}


def parallel(l, r, ff=None, limit=1.0):
    return {"type": "parallel", "mixer": {"left": l, "right": r}, "mlp": mlp(ff, limit)}


def model(width, vocab, eps, layers, streams=None, logit_scale=None, loop=None):
    cfg = {"architecture": "Fovezen", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers}
    if streams is not None:
        cfg["streams"] = streams
    if logit_scale is not None:
        cfg["logit_scale"] = logit_scale
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


# A: three copies of the stream, the first two layers run three times, every mixer kind, a layer without a feed-forward
FOV_A = model(96, 211, 1e-5, [
    mamba2(4, 24, 16, 2, 4, 2, ff=136, limit=0.8),
    parallel(left(6, 2, 16, 24, 0.3, 20, conv=2, softcap=5.0), right(3, 16, 40, 8.0, 8), ff=72, limit=2.0),
    attention(6, 3, 16, 32, 0.25, rot=rot(10000.0, 8, (8.0, 1.0, 4.0, 64)), ff=None),
    parallel(left(2, 1, 32, 32, 0.2, 7, conv=4), right(2, 48, 24, 3.0, 12)),
], streams=3, logit_scale=0.7, loop=(0, 2, 3))

# B: head sizes the tensor-core attention kernels serve (64), equal key and value sizes, one key/value head per head in one
# mixer and one for all in another, the whole head rotated without scaling, four copies, the loop over the last layers
FOV_B = model(128, 300, 1e-6, [
    attention(4, 2, 64, 64, 0.125, rot=rot(500000.0, 64), ff=200, limit=1.5),
    parallel(left(4, 4, 64, 64, 0.125, 150, softcap=20.0), right(4, 32, 16, 16.0, 16), ff=64, limit=0.5),
    mamba2(8, 16, 32, 4, 3, 4),
    attention(2, 1, 64, 64, 0.2, ff=96, limit=3.0),
], streams=4, loop=(1, 4, 2))

# C: one copy of the stream (with its own weights), no loop, a window shorter than a page and one longer than every prompt,
# a convolution of one tap (a factor per channel, no state)
FOV_C = model(80, 170, 1e-5, [
    parallel(left(5, 5, 16, 16, 0.25, 5, conv=3, softcap=50.0), right(5, 16, 16, 1.0, 24), ff=100, limit=1.0),
    attention(2, 1, 48, 16, 0.15, rot=rot(20.0, 48, (2.0, 1.0, 8.0, 16))),
    parallel(left(2, 2, 48, 80, 0.15, 400, conv=1), right(1, 64, 80, 30.0, 8), ff=40, limit=4.0),
    mamba2(1, 80, 64, 1, 1, 1, ff=60, limit=1.2),
], streams=1, logit_scale=2.0)

# D: no copies at all (a plain residual stream), a loop of one layer run four times, a width that is no multiple of 8,
# a parallel pair whose attention has no window
FOV_D = model(100, 77, 1e-3, [
    attention(3, 3, 32, 32, 0.18, rot=rot(300.0, 16)),
    mamba2(2, 40, 48, 2, 2, 1, ff=56, limit=0.9),
    parallel(left(3, 1, 32, 16, 0.3, None, conv=2), right(2, 32, 48, 4.0, 16), ff=88, limit=1.1),
], loop=(1, 2, 4))

SHARP = {"std": 0.12}


def make_model_dir(config, seed, out_dir, dtype="bfloat16", std=0.12):
    from geneinfer_b200.weights import write_random_model
    return write_random_model(config, seed, out_dir, dtype, std=std)
