"""Configuration of the Pinorax design, read from its own config.json keys.

Keys: ``architecture`` ("Pinorax"), ``width``, ``vocab``, ``max_positions`` (rows of the learned position table: the
design's context length), ``norm.eps``, ``residual_mult``, ``logit_softcap`` and ``layers``, a list whose entries give
``type`` ("latent_attention"), the mixer's sizes under ``mixer`` (``heads``, ``dim``, ``vdim``, ``kv_rank``, ``scale``) and
the feed-forward under ``mlp``: null for none; ``kind`` "dense" with ``ff``; or "moe" with ``expert.ff``, ``expert.limit``,
``router.experts``, ``router.top`` and optionally ``shared`` (``ff``, ``limit``), an expert that every token runs. Every
size and constant that the file gives is kept as it stands.

Translation into parts (``model_spec``): the embedding's output gets a learned vector per position (``learned`` position
at the embedding). Every layer is a ``parallel`` block: one ``rmsnorm_scalar`` norm (unit RMS times a single number) whose
output both sublayers read, x <- x + residual_mult (mixer + feed-forward), followed by the depth mix: what goes on is a
weighted sum of the embedding's output and every layer's result so far, with the layer's own weights. The mixer is the
``latent_attention`` mixer without a query latent, without a rotated part and without a window, with a learned sink per
head and an element-wise sigmoid gate on the heads' outputs. A dense feed-forward is a ``gated_mlp`` with SiLU and
biases; a mixture a ``routed_experts`` whose experts are looked up per token id in a table (weight 1 / top each), with
the "capped_swish" activation and the shared expert. The head is a matrix of its own; the logits are soft-capped.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .nipadra import _int, _num, _obj

MIXER_TYPES = ("latent_attention",)


@dataclass(frozen=True)
class PinoraxMixer:
    heads: int
    dim: int
    vdim: int
    kv_rank: int
    scale: float

    def to_json(self):
        return {"dim": self.dim, "heads": self.heads, "kv_rank": self.kv_rank, "scale": self.scale, "vdim": self.vdim}


@dataclass(frozen=True)
class PinoraxFeedForward:
    kind: str                       # "dense" | "moe"
    ff: int                         # of the dense feed-forward, or of one expert
    limit: float = 0.0              # of the experts' activation
    experts: int = 0
    top: int = 0
    shared_ff: int = 0              # 0: no shared expert
    shared_limit: float = 0.0

    def to_json(self):
        if self.kind == "dense":
            return {"ff": self.ff, "kind": "dense"}
        out: Dict[str, Any] = {"expert": {"ff": self.ff, "limit": self.limit}, "kind": "moe",
                               "router": {"experts": self.experts, "top": self.top}}
        if self.shared_ff:
            out["shared"] = {"ff": self.shared_ff, "limit": self.shared_limit}
        return out


@dataclass(frozen=True)
class PinoraxLayer:
    type: str
    mixer: PinoraxMixer
    mlp: Optional[PinoraxFeedForward]

    def to_json(self):
        return {"mixer": self.mixer.to_json(), "mlp": None if self.mlp is None else self.mlp.to_json(), "type": self.type}


def _limit(j: Dict[str, Any], what: str) -> float:
    v = _num(j, "limit", what)
    if not v > 0:
        raise ConfigError(f"config.json: {what}.limit must be positive")
    return v


def _feed_forward(mlp: Any, what: str) -> Optional[PinoraxFeedForward]:
    if mlp is None:
        return None
    mlp = _obj(mlp, what)
    kind = mlp.get("kind")
    if kind == "dense":
        return PinoraxFeedForward("dense", _int(mlp, "ff", what))
    if kind == "moe":
        router = _obj(mlp.get("router"), what + ".router")
        experts, top = _int(router, "experts", what + ".router"), _int(router, "top", what + ".router")
        if top > experts:
            raise ConfigError(f"config.json: {what}.router.top exceeds the number of experts")
        expert = _obj(mlp.get("expert"), what + ".expert")
        shared_ff, shared_limit = 0, 0.0
        if mlp.get("shared") is not None:
            shared = _obj(mlp.get("shared"), what + ".shared")
            shared_ff, shared_limit = _int(shared, "ff", what + ".shared"), _limit(shared, what + ".shared")
        return PinoraxFeedForward("moe", _int(expert, "ff", what + ".expert"), _limit(expert, what + ".expert"), experts, top,
                                  shared_ff, shared_limit)
    raise ConfigError(f"config.json: {what} has the unknown kind {kind!r} (known: dense, moe)")


@dataclass(frozen=True)
class PinoraxConfig:
    width: int
    vocab: int
    max_positions: int
    eps: float
    residual_mult: float
    logit_softcap: float
    layers: Tuple[PinoraxLayer, ...]

    architecture = "Pinorax"
    model_type = "pinorax"

    @classmethod
    def from_json(cls, j: Any) -> "PinoraxConfig":
        j = _obj(j, "the configuration")
        width, vocab = _int(j, "width", "the model"), _int(j, "vocab", "the model")
        max_positions = _int(j, "max_positions", "the model")
        eps = _num(_obj(j.get("norm"), "norm"), "eps", "norm")
        if not eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        mult, cap = _num(j, "residual_mult", "the model"), _num(j, "logit_softcap", "the model")
        if not cap > 0:
            raise ConfigError("config.json: logit_softcap must be positive")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[PinoraxLayer] = []
        for i, entry in enumerate(raw):
            what = f"layer {i}"
            entry = _obj(entry, what)
            kind = entry.get("type")
            if kind not in MIXER_TYPES:
                raise ConfigError(f"config.json: {what} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            m = _obj(entry.get("mixer"), what + ".mixer")
            heads, dim, vdim, kv_rank = (_int(m, k, what + ".mixer") for k in ("heads", "dim", "vdim", "kv_rank"))
            mixer = PinoraxMixer(heads, dim, vdim, kv_rank, _num(m, "scale", what + ".mixer"))
            layers.append(PinoraxLayer(kind, mixer, _feed_forward(entry.get("mlp"), what + ".mlp")))
        return cls(width, vocab, max_positions, eps, mult, cap, tuple(layers))

    def to_json(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "layers": [l.to_json() for l in self.layers],
                "logit_softcap": self.logit_softcap, "max_positions": self.max_positions, "norm": {"eps": self.eps},
                "residual_mult": self.residual_mult, "vocab": self.vocab, "width": self.width}

    # ------------------------------------------------------------------ translation into parts
    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = PartSpec("rmsnorm_scalar", {"size": D, "eps": self.eps})
        specs, schedule = [], []
        for i, layer in enumerate(self.layers):
            m = layer.mixer
            mixer = PartSpec("latent_attention", {
                "hidden_size": D, "num_heads": m.heads, "head_dim": m.dim, "rotary_dim": 0, "value_dim": m.vdim, "q_rank": None,
                "kv_rank": m.kv_rank, "scale": m.scale, "window": None, "norm_eps": self.eps, "position": None,
                "sink": "learned", "output_gate": True})
            f, ffn = layer.mlp, None
            if f is not None and f.kind == "dense":
                ffn = PartSpec("gated_mlp", {"hidden_size": D, "intermediate_size": f.ff, "activation": "silu", "bias": True})
            elif f is not None:
                shared = None
                if f.shared_ff:
                    shared = {"hidden_size": D, "intermediate_size": f.shared_ff, "activation": "capped_swish",
                              "activation_limit": f.shared_limit}
                ffn = PartSpec("routed_experts", {"hidden_size": D, "intermediate_size": f.ff, "experts": f.experts, "top": f.top,
                                                  "activation": "capped_swish", "activation_limit": f.limit, "router": "table",
                                                  "vocab_size": self.vocab, "shared": shared})
            specs.append(LayerSpec(mixer=mixer, feed_forward=ffn, mixer_norm=norm, feed_forward_norm=None, block="parallel",
                                   block_params={"residual_mult": self.residual_mult, "depth_slot": i + 1,
                                                 "depth_slots": len(self.layers) + 1}))
            schedule.append(ScheduleEntry(i))
        return ModelSpec(architecture=self.architecture, hidden_size=D, vocab_size=self.vocab, max_position=self.max_positions,
                         layers=specs, schedule=schedule, final_norm=norm, tie_word_embeddings=False,
                         embedding_position=PartSpec("learned", {"size": D, "positions": self.max_positions}),
                         logit_transform=PartSpec("softcap", {"cap": self.logit_softcap}))
