"""What a checkpoint must hold for an architecture, and how it becomes parameters of parts.

A ``WeightPlan`` lists every tensor by its name in the checkpoint with the shape the configuration
implies, the name patterns that may be present but are not used, and a function that assembles the
read tensors into the parameter dictionary of the model (``layers.3.mixer.w_qkv`` and so on).
"""
from __future__ import annotations

import fnmatch
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Tuple

import torch


@dataclass(frozen=True)
class TensorRule:
    name: str
    shape: Tuple[int, ...]   # an extent of -1 is left open: whatever the checkpoint has there is taken
    kind: str = "matrix"     # "matrix", "vector" (norm weights and the like) or "table" (integers)
    # how random weights are drawn for this tensor, when not as its kind says: (mean, std) of a normal
    # distribution, or ("uniform", low, high)
    init: Optional[Tuple] = None


@dataclass
class WeightPlan:
    rules: List[TensorRule]
    ignorable: List[str] = field(default_factory=list)      # fnmatch patterns of unused tensors
    assemble: Callable[[Dict[str, torch.Tensor]], Dict[str, torch.Tensor]] = lambda t: dict(t)

    def is_ignorable(self, name: str) -> bool:
        return any(fnmatch.fnmatchcase(name, p) for p in self.ignorable)


def llama_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Llama checkpoint (src/loader/hf_checkpoint.cpp:214-235).

    q/k/v are concatenated into one ``w_qkv`` [A+2K, D] and gate/up into one ``w_gate_up`` [2I, D]
    (gate rows first) so that each pair of projections is a single matrix product. A tied model's
    head is the embedding table itself (one copy on the device)."""
    D, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    A, K = cfg.attn_dim, cfg.kv_dim
    rules = [TensorRule("model.embed_tokens.weight", (V, D))]
    for l in range(cfg.num_hidden_layers):
        p = f"model.layers.{l}."
        rules += [
            TensorRule(p + "input_layernorm.weight", (D,), "vector"),
            TensorRule(p + "self_attn.q_proj.weight", (A, D)),
            TensorRule(p + "self_attn.k_proj.weight", (K, D)),
            TensorRule(p + "self_attn.v_proj.weight", (K, D)),
            TensorRule(p + "self_attn.o_proj.weight", (D, A)),
            TensorRule(p + "post_attention_layernorm.weight", (D,), "vector"),
            TensorRule(p + "mlp.gate_proj.weight", (I, D)),
            TensorRule(p + "mlp.up_proj.weight", (I, D)),
            TensorRule(p + "mlp.down_proj.weight", (D, I)),
        ]
    rules.append(TensorRule("model.norm.weight", (D,), "vector"))
    ignorable = ["model.layers.*.self_attn.rotary_emb.inv_freq"]
    if cfg.tie_word_embeddings:
        ignorable.append("lm_head.weight")      # a redundant copy some exporters leave in tied models
    else:
        rules.append(TensorRule("lm_head.weight", (V, D)))

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["model.embed_tokens.weight"]}
        for l in range(cfg.num_hidden_layers):
            p, q = f"model.layers.{l}.", f"layers.{l}."
            out[q + "mixer_norm.weight"] = t[p + "input_layernorm.weight"]
            out[q + "mixer.w_qkv"] = _cat([t[p + "self_attn.q_proj.weight"], t[p + "self_attn.k_proj.weight"],
                                           t[p + "self_attn.v_proj.weight"]])
            out[q + "mixer.w_o"] = t[p + "self_attn.o_proj.weight"]
            out[q + "feed_forward_norm.weight"] = t[p + "post_attention_layernorm.weight"]
            out[q + "feed_forward.w_gate_up"] = _cat([t[p + "mlp.gate_proj.weight"], t[p + "mlp.up_proj.weight"]])
            out[q + "feed_forward.w_down"] = t[p + "mlp.down_proj.weight"]
        out["final_norm.weight"] = t["model.norm.weight"]
        out["head.weight"] = out["embedding.weight"] if cfg.tie_word_embeddings else t["lm_head.weight"]
        return out

    return WeightPlan(rules, ignorable, assemble)


def nipadra_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Nipadra checkpoint: ``embed``, ``final.norm`` and, for layer i,
    ``l<i>.norm1`` / ``l<i>.norm2``, the mixer's tensors under ``l<i>.mix.`` and the feed-forward's under
    ``l<i>.mlp.``. Projections that read the same input are concatenated row-wise into one matrix product
    each: [q; k; v; g] of a lightning mixer, [q; k; g] of the windowed attention, [gate; up] of the feed-forward."""
    D, V = cfg.width, cfg.vocab
    zero = (0.0, 0.05)                   # norm weights of this design are stored around zero
    rules = [TensorRule("embed", (V, D))]
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}."
        rules.append(TensorRule(p + "norm1", (D,), "vector", zero))
        if layer.ff is not None:
            rules.append(TensorRule(p + "norm2", (D,), "vector", zero))
        m = layer.mixer
        if layer.type == "lightning":
            rules += [TensorRule(p + "mix.q", (m.heads * m.dim, D)), TensorRule(p + "mix.k", (m.heads * m.dim, D)),
                      TensorRule(p + "mix.v", (m.heads * m.vdim, D)), TensorRule(p + "mix.g", (m.heads * m.vdim, D)),
                      TensorRule(p + "mix.o", (D, m.heads * m.vdim)), TensorRule(p + "mix.norm", (m.heads * m.vdim,), "vector")]
        else:
            a, s = m.left, m.right
            q = p + "mix.left."
            rules += [TensorRule(q + "q", (a.heads * a.dim, D)), TensorRule(q + "k", (a.kv_heads * a.dim, D)),
                      TensorRule(q + "q.norm", (a.dim,), "vector"), TensorRule(q + "k.norm", (a.dim,), "vector"),
                      TensorRule(q + "g", (a.heads, D)), TensorRule(q + "o", (D, a.heads * a.vdim))]
            q = p + "mix.right."
            rules += [TensorRule(q + "in", (2 * s.inner + 2 * s.groups * s.state + s.heads, D)),
                      TensorRule(q + "conv", (s.conv_channels, s.conv), "vector", (0.0, 0.4)),
                      TensorRule(q + "conv.b", (s.conv_channels,), "vector", (0.0, 0.1)),
                      TensorRule(q + "dt_bias", (s.heads,), "vector", ("uniform", -3.0, 0.5)),
                      TensorRule(q + "A_log", (s.heads,), "vector", ("uniform", -1.5, 1.0)),
                      TensorRule(q + "D", (s.heads,), "vector", (1.0, 0.2)),
                      TensorRule(q + "norm", (s.inner,), "vector"), TensorRule(q + "o", (D, s.inner))]
        if layer.ff is not None:
            rules += [TensorRule(p + "mlp.gate", (layer.ff, D)), TensorRule(p + "mlp.up", (layer.ff, D)),
                      TensorRule(p + "mlp.down", (D, layer.ff))]
    rules.append(TensorRule("final.norm", (D,), "vector", zero))

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["embed"], "head.weight": t["embed"],
                                        "final_norm.weight": t["final.norm"]}
        for i, layer in enumerate(cfg.layers):
            p, q = f"l{i}.", f"layers.{i}."
            out[q + "mixer_norm.weight"] = t[p + "norm1"]
            if layer.type == "lightning":
                out[q + "mixer.w_in"] = _cat([t[p + "mix.q"], t[p + "mix.k"], t[p + "mix.v"], t[p + "mix.g"]])
                out[q + "mixer.w_o"] = t[p + "mix.o"]
                out[q + "mixer.norm"] = t[p + "mix.norm"]
            else:
                a, b = p + "mix.left.", q + "mixer.left."
                out[b + "w_qkv"] = _cat([t[a + "q"], t[a + "k"], t[a + "g"]])
                out[b + "q_norm"], out[b + "k_norm"], out[b + "w_o"] = t[a + "q.norm"], t[a + "k.norm"], t[a + "o"]
                a, b = p + "mix.right.", q + "mixer.right."
                out[b + "w_in"], out[b + "w_o"], out[b + "norm"] = t[a + "in"], t[a + "o"], t[a + "norm"]
                out[b + "conv"], out[b + "conv_bias"] = t[a + "conv"], t[a + "conv.b"]
                out[b + "dt_bias"], out[b + "a_log"], out[b + "skip"] = t[a + "dt_bias"], t[a + "A_log"], t[a + "D"]
            if layer.ff is not None:
                out[q + "feed_forward_norm.weight"] = t[p + "norm2"]
                out[q + "feed_forward.w_gate_up"] = _cat([t[p + "mlp.gate"], t[p + "mlp.up"]])
                out[q + "feed_forward.w_down"] = t[p + "mlp.down"]
        return out

    return WeightPlan(rules, [], assemble)


def gekupel_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Gekupel checkpoint: ``embed``, ``head``, ``final.norm`` and, for a layer i that has
    weights of its own, ``l<i>.norm1`` / ``l<i>.norm2``, the mixer's tensors under ``l<i>.mix.`` and the feed-forward's
    under ``l<i>.mlp.`` (a mixture: ``e<k>.gate`` / ``.up`` / ``.down`` per expert, ``router``, ``correction``). A layer
    that names another under ``weights_of`` has none. Projections that read the same input become one product: [q; k; v]
    of the attention, [dq; dkv] of the latent attention, [gate; up] of a feed-forward; the experts' matrices are stacked."""
    D, V = cfg.width, cfg.vocab
    rules = [TensorRule("embed", (V, D)), TensorRule("head", (V, D)), TensorRule("final.norm", (D,), "vector")]
    for i, layer in enumerate(cfg.layers):
        if layer.weights_of is not None:
            continue
        p, m = f"l{i}.", layer.mixer
        rules.append(TensorRule(p + "norm1", (D,), "vector"))
        if layer.type == "attention":
            rules += [TensorRule(p + "mix.q", (m.heads * m.dim, D)), TensorRule(p + "mix.k", (m.kv_heads * m.dim, D)),
                      TensorRule(p + "mix.v", (m.kv_heads * m.vdim, D)), TensorRule(p + "mix.o", (D, m.heads * m.vdim)),
                      TensorRule(p + "mix.sink", (m.heads,), "vector", (0.0, 1.0))]
        else:
            rules += [TensorRule(p + "mix.dq", (m.q_rank, D)), TensorRule(p + "mix.dq.norm", (m.q_rank,), "vector"),
                      TensorRule(p + "mix.uq", (m.heads * (m.dim + m.rot_dim), m.q_rank)),
                      TensorRule(p + "mix.dkv", (m.kv_rank + m.rot_dim, D)), TensorRule(p + "mix.dkv.norm", (m.kv_rank,), "vector"),
                      TensorRule(p + "mix.uk", (m.heads * m.dim, m.kv_rank)), TensorRule(p + "mix.uv", (m.heads * m.vdim, m.kv_rank)),
                      TensorRule(p + "mix.o", (D, m.heads * m.vdim))]
            if m.sink:
                rules.append(TensorRule(p + "mix.sink", (m.heads,), "vector", (0.0, 1.0)))
        f = layer.mlp
        if f is None:
            continue
        rules.append(TensorRule(p + "norm2", (D,), "vector"))
        if f.kind == "dense":
            rules += [TensorRule(p + "mlp.gate", (f.ff, D)), TensorRule(p + "mlp.up", (f.ff, D)), TensorRule(p + "mlp.down", (D, f.ff))]
        else:
            for e in range(f.experts):
                q = f"{p}mlp.e{e}."
                rules += [TensorRule(q + "gate", (f.ff, D)), TensorRule(q + "up", (f.ff, D)), TensorRule(q + "down", (D, f.ff))]
            rules += [TensorRule(p + "mlp.router", (f.experts, D)), TensorRule(p + "mlp.correction", (f.experts,), "vector", (0.0, 0.1))]

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["embed"], "head.weight": t["head"], "final_norm.weight": t["final.norm"]}
        for i, layer in enumerate(cfg.layers):
            if layer.weights_of is not None:
                continue
            p, q = f"l{i}.", f"layers.{i}."
            out[q + "mixer_norm.weight"] = t[p + "norm1"]
            a, b = p + "mix.", q + "mixer."
            if layer.type == "attention":
                out[b + "w_qkv"] = _cat([t[a + "q"], t[a + "k"], t[a + "v"]])
            else:
                out[b + "w_down"] = _cat([t[a + "dq"], t[a + "dkv"]])
                out[b + "q_latent_norm"], out[b + "kv_latent_norm"] = t[a + "dq.norm"], t[a + "dkv.norm"]
                out[b + "w_uq"], out[b + "w_uk"], out[b + "w_uv"] = t[a + "uq"], t[a + "uk"], t[a + "uv"]
            out[b + "w_o"] = t[a + "o"]
            if a + "sink" in t:
                out[b + "sink"] = t[a + "sink"]
            f = layer.mlp
            if f is None:
                continue
            out[q + "feed_forward_norm.weight"] = t[p + "norm2"]
            a, b = p + "mlp.", q + "feed_forward."
            if f.kind == "dense":
                out[b + "w_gate_up"] = _cat([t[a + "gate"], t[a + "up"]])
                out[b + "w_down"] = t[a + "down"]
            else:
                out[b + "w_gate_up"] = torch.stack([_cat([t[f"{a}e{e}.gate"], t[f"{a}e{e}.up"]]) for e in range(f.experts)])
                out[b + "w_down"] = torch.stack([t[f"{a}e{e}.down"] for e in range(f.experts)])
                out[b + "router"], out[b + "correction"] = t[a + "router"], t[a + "correction"]
        return out

    return WeightPlan(rules, [], assemble)


def pinorax_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Pinorax checkpoint: ``embed``, ``pos`` (a vector per position), ``head``, ``final.norm``
    (a single number) and, for layer i, ``l<i>.norm1`` (a single number), ``l<i>.dwa`` (the i + 2 weights of its depth mix),
    the mixer's tensors under ``l<i>.mix.`` and the feed-forward's under ``l<i>.mlp.`` (dense: ``gate``, ``up``, ``down`` with a
    bias ``.b`` each; a mixture: ``e<k>.gate`` / ``.up`` / ``.down`` per expert, ``table`` [vocab, top] of expert indices and
    ``shared.gate`` / ``.up`` / ``.down``). Projections that read the same input become one product: [q; dkv; g] of the
    mixer, [gate; up] of a feed-forward; the experts' matrices are stacked."""
    D, V = cfg.width, cfg.vocab
    rules = [TensorRule("embed", (V, D)), TensorRule("pos", (cfg.max_positions, D)), TensorRule("head", (V, D)),
             TensorRule("final.norm", (), "vector")]
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        rules += [TensorRule(p + "norm1", (), "vector"),
                  TensorRule(p + "mix.q", (m.heads * m.dim, D)), TensorRule(p + "mix.dkv", (m.kv_rank, D)),
                  TensorRule(p + "mix.dkv.norm", (m.kv_rank,), "vector"), TensorRule(p + "mix.uk", (m.heads * m.dim, m.kv_rank)),
                  TensorRule(p + "mix.uv", (m.heads * m.vdim, m.kv_rank)), TensorRule(p + "mix.sink", (m.heads,), "vector", (0.0, 1.0)),
                  TensorRule(p + "mix.g", (m.heads * m.vdim, D)), TensorRule(p + "mix.o", (D, m.heads * m.vdim))]
        f = layer.mlp
        if f is not None and f.kind == "dense":
            for name, shape in (("gate", (f.ff, D)), ("up", (f.ff, D)), ("down", (D, f.ff))):
                rules += [TensorRule(p + "mlp." + name, shape), TensorRule(p + "mlp." + name + ".b", shape[:1], "vector", (0.0, 0.1))]
        elif f is not None:
            for e in range(f.experts):
                q = f"{p}mlp.e{e}."
                rules += [TensorRule(q + "gate", (f.ff, D)), TensorRule(q + "up", (f.ff, D)), TensorRule(q + "down", (D, f.ff))]
            rules.append(TensorRule(p + "mlp.table", (V, f.top), "table", ("distinct", f.experts)))
            if f.shared_ff:
                q = p + "mlp.shared."
                rules += [TensorRule(q + "gate", (f.shared_ff, D)), TensorRule(q + "up", (f.shared_ff, D)),
                          TensorRule(q + "down", (D, f.shared_ff))]
        rules.append(TensorRule(p + "dwa", (i + 2,), "vector", (1.0 / (i + 2), 0.2)))

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["embed"], "embedding_position.table": t["pos"], "head.weight": t["head"],
                                        "final_norm.weight": t["final.norm"]}
        for i, layer in enumerate(cfg.layers):
            p, q = f"l{i}.", f"layers.{i}."
            out[q + "mixer_norm.weight"] = t[p + "norm1"]
            out[q + "depth_weights"] = t[p + "dwa"]
            a, b = p + "mix.", q + "mixer."
            out[b + "w_down"] = _cat([t[a + "q"], t[a + "dkv"], t[a + "g"]])
            out[b + "kv_latent_norm"] = t[a + "dkv.norm"]
            out[b + "w_uk"], out[b + "w_uv"], out[b + "w_o"], out[b + "sink"] = t[a + "uk"], t[a + "uv"], t[a + "o"], t[a + "sink"]
            f = layer.mlp
            if f is None:
                continue
            a, b = p + "mlp.", q + "feed_forward."
            if f.kind == "dense":
                out[b + "w_gate_up"] = _cat([t[a + "gate"], t[a + "up"]])
                out[b + "b_gate_up"] = _cat([t[a + "gate.b"], t[a + "up.b"]])
                out[b + "w_down"], out[b + "b_down"] = t[a + "down"], t[a + "down.b"]
            else:
                out[b + "w_gate_up"] = torch.stack([_cat([t[f"{a}e{e}.gate"], t[f"{a}e{e}.up"]]) for e in range(f.experts)])
                out[b + "w_down"] = torch.stack([t[f"{a}e{e}.down"] for e in range(f.experts)])
                out[b + "table"] = t[a + "table"]
                if f.shared_ff:
                    out[b + "shared.w_gate_up"] = _cat([t[a + "shared.gate"], t[a + "shared.up"]])
                    out[b + "shared.w_down"] = t[a + "shared.down"]
        return out

    return WeightPlan(rules, [], assemble)


def fovezen_weight_plan(cfg) -> WeightPlan:
    """Tensor names and shapes of a Fovezen checkpoint: ``embed``, ``head``, ``final.norm`` and, for layer i, ``l<i>.norm1`` /
    ``l<i>.norm2``, with ``streams`` also ``l<i>.hc1.in`` / ``.out`` / ``.mix`` (and ``hc2`` with a feed-forward), the mixer's
    tensors under ``l<i>.mix.`` (a parallel mixer: under ``.left.`` and ``.right.``, with ``left.out`` and ``right.out``) and the
    feed-forward's under ``l<i>.mlp.``. Projections that read the same input become one product: [q; k; v] of an attention
    (their three convolutions likewise one), [q; k; v; g] of the gated linear attention, [gate; up] of the feed-forward. A
    model without ``streams`` runs the same block with one copy and unit weights."""
    D, V, S = cfg.width, cfg.vocab, cfg.streams
    zero = (0.0, 0.05)                   # the layers' norm weights are stored around zero
    rules = [TensorRule("embed", (V, D)), TensorRule("head", (V, D)), TensorRule("final.norm", (D,), "vector", zero)]
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        rules.append(TensorRule(p + "norm1", (D,), "vector", zero))
        q = p + "mix."
        if layer.type == "attention":
            rules += [TensorRule(q + "q", (m.heads * m.dim, D)), TensorRule(q + "k", (m.kv_heads * m.dim, D)),
                      TensorRule(q + "v", (m.kv_heads * m.vdim, D)), TensorRule(q + "q.norm", (m.heads * m.dim,), "vector"),
                      TensorRule(q + "k.norm", (m.kv_heads * m.dim,), "vector"), TensorRule(q + "o", (D, m.heads * m.vdim))]
        elif layer.type == "mamba2":
            rules += [TensorRule(q + "in", (2 * m.inner + 2 * m.groups * m.state + m.heads, D)),
                      TensorRule(q + "conv", (m.conv_channels, m.conv), "vector", (0.0, 0.4)),
                      TensorRule(q + "conv.b", (m.conv_channels,), "vector", (0.0, 0.1)),
                      TensorRule(q + "dt_bias", (m.heads,), "vector", ("uniform", -3.0, 0.5)),
                      TensorRule(q + "A_log", (m.heads,), "vector", ("uniform", -1.5, 1.0)),
                      TensorRule(q + "D", (m.heads,), "vector", (1.0, 0.2)),
                      TensorRule(q + "norm", (m.inner,), "vector"), TensorRule(q + "o", (D, m.inner))]
        else:
            a, g = m.left, m.right
            q = p + "mix.left."
            for name, rows in (("q", a.heads * a.dim), ("k", a.kv_heads * a.dim), ("v", a.kv_heads * a.vdim)):
                rules.append(TensorRule(q + name, (rows, D)))
                if a.conv is not None:
                    rules.append(TensorRule(q + name + ".conv", (rows, a.conv), "vector", (0.0, 0.5)))
            rules += [TensorRule(q + "q.norm", (a.dim,), "vector"), TensorRule(q + "k.norm", (a.dim,), "vector"),
                      TensorRule(q + "o", (D, a.heads * a.vdim))]
            q = p + "mix.right."
            rank = g.rank or -1
            rules += [TensorRule(q + "q", (g.heads * g.dim, D)), TensorRule(q + "k", (g.heads * g.dim, D)),
                      TensorRule(q + "v", (g.heads * g.vdim, D)), TensorRule(q + "g", (g.heads * g.vdim, D)),
                      TensorRule(q + "o", (D, g.heads * g.vdim)), TensorRule(q + "norm", (g.vdim,), "vector"),
                      TensorRule(q + "a1", (rank, D)), TensorRule(q + "a2", (g.heads * g.dim, rank), "matrix", (0.0, 0.3)),
                      TensorRule(q + "a2.b", (g.heads * g.dim,), "vector", ("uniform", 1.0, 5.0)),
                      TensorRule(p + "mix.left.out", (D,), "vector"), TensorRule(p + "mix.right.out", (D,), "vector")]
        if layer.ff is not None:
            rules += [TensorRule(p + "norm2", (D,), "vector", zero), TensorRule(p + "mlp.gate", (layer.ff, D)),
                      TensorRule(p + "mlp.up", (layer.ff, D)), TensorRule(p + "mlp.down", (D, layer.ff))]
        if S is not None:
            for c in ("hc1.", "hc2.") if layer.ff is not None else ("hc1.",):
                rules += [TensorRule(p + c + "in", (S,), "vector", (1.0 / S, 0.2)), TensorRule(p + c + "out", (S,), "vector", (1.0, 0.3)),
                          TensorRule(p + c + "mix", (S, S), "vector", (1.0 / S, 0.3))]

    def assemble(t: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
        out: Dict[str, torch.Tensor] = {"embedding.weight": t["embed"], "head.weight": t["head"], "final_norm.weight": t["final.norm"]}
        for i, layer in enumerate(cfg.layers):
            p, q = f"l{i}.", f"layers.{i}."
            out[q + "mixer_norm.weight"] = t[p + "norm1"]
            a, b = p + "mix.", q + "mixer."
            if layer.type == "attention":
                out[b + "w_qkv"] = _cat([t[a + "q"], t[a + "k"], t[a + "v"]])
                out[b + "q_norm"], out[b + "k_norm"], out[b + "w_o"] = t[a + "q.norm"], t[a + "k.norm"], t[a + "o"]
            elif layer.type == "mamba2":
                out[b + "w_in"], out[b + "w_o"], out[b + "norm"] = t[a + "in"], t[a + "o"], t[a + "norm"]
                out[b + "conv"], out[b + "conv_bias"] = t[a + "conv"], t[a + "conv.b"]
                out[b + "dt_bias"], out[b + "a_log"], out[b + "skip"] = t[a + "dt_bias"], t[a + "A_log"], t[a + "D"]
            else:
                a, b = p + "mix.left.", q + "mixer.left."
                out[b + "w_qkv"] = _cat([t[a + "q"], t[a + "k"], t[a + "v"]])
                if layer.mixer.left.conv is not None:
                    out[b + "conv"] = _cat([t[a + "q.conv"], t[a + "k.conv"], t[a + "v.conv"]])
                out[b + "q_norm"], out[b + "k_norm"], out[b + "w_o"] = t[a + "q.norm"], t[a + "k.norm"], t[a + "o"]
                a, b = p + "mix.right.", q + "mixer.right."
                out[b + "w_in"] = _cat([t[a + "q"], t[a + "k"], t[a + "v"], t[a + "g"]])
                out[b + "w_a1"], out[b + "w_a2"], out[b + "a2_bias"] = t[a + "a1"], t[a + "a2"], t[a + "a2.b"]
                out[b + "norm"], out[b + "w_o"] = t[a + "norm"], t[a + "o"]
                out[q + "mixer.left_out"], out[q + "mixer.right_out"] = t[p + "mix.left.out"], t[p + "mix.right.out"]
            if layer.ff is not None:
                out[q + "feed_forward_norm.weight"] = t[p + "norm2"]
                out[q + "feed_forward.w_gate_up"] = _cat([t[p + "mlp.gate"], t[p + "mlp.up"]])
                out[q + "feed_forward.w_down"] = t[p + "mlp.down"]
            for c in ("hc1.", "hc2.") if layer.ff is not None else ("hc1.",):
                for name, shape in (("in", (1,)), ("out", (1,)), ("mix", (1, 1))):
                    out[q + c + name] = t[p + c + name] if S is not None else torch.ones(shape, dtype=torch.float32)
        return out

    return WeightPlan(rules, [], assemble)


def _cat(parts: List[torch.Tensor]) -> torch.Tensor:
    """Concatenates rows; parts of different stored dtypes are widened to 32-bit first."""
    if len({p.dtype for p in parts}) > 1:
        parts = [p.float() for p in parts]
    return torch.cat(parts, dim=0)
