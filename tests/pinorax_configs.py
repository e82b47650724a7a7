"""Small Pinorax configurations for the tests. Every layer of a configuration has sizes of its own, and values that a
particular model may happen to make equal (head and value sizes, the latent's rank and a head's size, the experts'
and the shared expert's widths and limits) or 1 (heads, the experts a token uses, the residual's factor) are chosen
apart."""
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def dense(ff):
    return {"ff": ff, "kind": "dense"}


def moe(ff, limit, experts, top, shared=None):
    out = {"expert": {"ff": ff, "limit": limit}, "kind": "moe", "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared[0], "limit": shared[1]}
    return out


def layer(heads, dim, vdim, kv_rank, scale, mlp=None):
    return {"mixer": {"dim": dim, "heads": heads, "kv_rank": kv_rank, "scale": scale, "vdim": vdim}, "mlp": mlp,
            "type": "latent_attention"}


def model(width, vocab, max_positions, eps, mult, cap, layers):
    return {"architecture": "Pinorax", "layers": layers, "logit_softcap": cap, "max_positions": max_positions,
            "norm": {"eps": eps}, "residual_mult": mult, "vocab": vocab, "width": width}


# A: both kinds of feed-forward and a layer without one; a mixture without a shared expert; one expert to a token;
# values wider and narrower than the keys; one head
PIN_A = model(96, 190, 512, 1e-5, 0.45, 9.0, [
    layer(3, 24, 40, 48, 0.2, moe(40, 0.8, 5, 2, shared=(56, 1.7))),
    layer(5, 8, 16, 40, 0.3, dense(136)),
    layer(1, 32, 8, 72, 0.15),
    layer(2, 16, 24, 56, 0.25, moe(72, 2.5, 3, 1)),
    layer(4, 24, 24, 24, 0.22, dense(64)),
    layer(3, 24, 40, 48, 0.2, moe(24, 1.2, 7, 3, shared=(24, 0.6))),
])

# B: heads and ranks that the tensor-core form of the attention serves in bfloat16 (eight and sixteen heads, latents of
# 64 and 128 values) beside a layer that it does not; a factor above one on the residual; a table as long as needed only
PIN_B = model(128, 260, 400, 1e-6, 1.25, 30.0, [
    layer(8, 16, 24, 64, 0.25, dense(200)),
    layer(16, 32, 8, 128, 0.17, moe(56, 1.0, 4, 3, shared=(72, 3.0))),
    layer(9, 12, 20, 136, 0.3, moe(48, 0.5, 9, 4)),
    layer(8, 40, 48, 64, 0.12),
])

# C: sizes that fit no tile: a width and ranks that are no multiples of 8 (nor of 4), three heads, odd value sizes, seven
# experts of 44 of which a token uses three, a single layer's depth mix of two terms at the end
PIN_C = model(100, 131, 300, 1e-4, 0.7, 4.0, [
    layer(3, 20, 28, 52, 0.35, moe(44, 1.5, 7, 3, shared=(30, 0.9))),
    layer(6, 10, 7, 34, 0.5, dense(60)),
    layer(7, 6, 10, 30, 0.4, moe(10, 2.0, 2, 2)),
])

# D: one layer only (the depth mix has two terms), a single expert table column
PIN_D = model(64, 77, 128, 1e-6, 1.0, 50.0, [layer(2, 8, 12, 16, 0.35, moe(16, 1.0, 3, 1, shared=(8, 2.0)))])


def make_model_dir(config, seed, out_dir, dtype="bfloat16", std=0.12):
    from geneinfer_b200.weights import write_random_model
    return write_random_model(config, seed, out_dir, dtype, std=std)
