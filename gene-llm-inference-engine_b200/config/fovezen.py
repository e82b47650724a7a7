"""Configuration of the Fovezen design, read from its own config.json keys.

Keys: ``architecture`` ("Fovezen"), ``width``, ``vocab``, ``norm.eps``, ``streams`` (copies of the residual stream; absent:
one plain stream), ``logit_scale`` (1 when absent), ``loop`` (``start``, ``stop``, ``times``: layers start .. stop-1 run that
many times in a row on the same weights, every pass with a cache and state of its own; absent: every layer once) and
``layers``, a list whose entries give ``type``, the mixer's sizes under ``mixer`` and the feed-forward under ``mlp`` (null
for none; ``kind`` "dense" with ``ff`` and ``limit``). Mixer types:

* "attention": ``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and optionally ``rot`` (``base``, ``dims`` and optionally
  ``scaling`` with ``factor``, ``low``, ``high``, ``original``);
* "mamba2": ``heads``, ``vdim``, ``state``, ``groups``, ``conv``, ``norm_groups``;
* "parallel": ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale`` and optionally ``mask.size``, ``conv`` and
  ``softcap``) beside ``right`` (``heads``, ``dim``, ``vdim``, ``tau``; the rank of its decay projection is read off the
  checkpoint's shapes by the weight plan and may be given as ``rank``).

Every size and constant that the file gives is kept as it stands; nothing is assumed equal to anything else. The design
has no context length of its own: ``max_position`` (optional) only sets the engine's default.

Translation into parts (``model_spec``): every layer is a ``hyper_connections`` block with ``rmsnorm`` norms whose weights
are stored around zero. "attention" becomes the ``attention`` mixer with one norm over the whole query projection and one
over the whole key projection, a half-split partial rotation whose angles are computed on the device (frequencies scaled
by wavelength) and all earlier keys visible; "mamba2" the ``state_space`` mixer; "parallel" a ``parallel`` mixer that
takes the mean of its branches' outputs, each brought to unit RMS over the width and weighted: a windowed ``attention``
mixer with a short convolution on its projections, per-head query/key norm, no rotation and soft-capped scores, beside a
``gated_linear_attention`` mixer. The feed-forward is a ``gated_mlp`` with the "capped_swish" activation. A layer that the
loop runs again gets one further (weightless) layer per extra pass, which runs the owner's parts on a cache of its own.
The head is a matrix of its own; the logits are multiplied by ``logit_scale``.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Tuple

from .base import ConfigError, LayerSpec, ModelSpec, PartSpec, ScheduleEntry
from .nipadra import DEFAULT_CONTEXT, StateSpaceSizes, _int, _num, _obj, _state_space

MIXER_TYPES = ("attention", "mamba2", "parallel")


@dataclass(frozen=True)
class RotaryAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_base: Optional[float] = None        # None: no rotation
    rot_dims: int = 0
    rot_scaling: Optional[Tuple[float, float, float, float]] = None      # factor, low, high, original

    def to_json(self):
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.rot_base is not None:
            out["rot"] = {"base": self.rot_base, "dims": self.rot_dims}
            if self.rot_scaling is not None:
                f, lo, hi, orig = self.rot_scaling
                out["rot"]["scaling"] = {"factor": f, "high": hi, "low": lo, "original": orig}
        return out


@dataclass(frozen=True)
class ConvWindowAttentionSizes:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]                   # None: every earlier key
    conv: Optional[int] = None              # taps (one tap: a factor per channel); None: no convolution, no such tensors
    softcap: Optional[float] = None

    def to_json(self):
        out: Dict[str, Any] = {"dim": self.dim, "heads": self.heads, "kv_heads": self.kv_heads, "scale": self.scale, "vdim": self.vdim}
        if self.window is not None:
            out["mask"] = {"size": self.window}
        if self.conv is not None:
            out["conv"] = self.conv
        if self.softcap is not None:
            out["softcap"] = self.softcap
        return out


@dataclass(frozen=True)
class GatedLinearSizes:
    heads: int
    dim: int
    vdim: int
    tau: float
    rank: int                               # of the decay's two-step projection; 0: whatever the checkpoint's shapes say

    def to_json(self):
        out = {"dim": self.dim, "heads": self.heads, "tau": self.tau, "vdim": self.vdim}
        if self.rank:
            out["rank"] = self.rank
        return out


@dataclass(frozen=True)
class ParallelPairSizes:
    left: ConvWindowAttentionSizes
    right: GatedLinearSizes

    def to_json(self):
        return {"left": self.left.to_json(), "right": self.right.to_json()}


@dataclass(frozen=True)
class FovezenLayer:
    type: str                          # one of MIXER_TYPES
    mixer: Any
    ff: Optional[int]                  # None: the layer has no feed-forward
    limit: float = 0.0

    def to_json(self):
        return {"type": self.type, "mixer": self.mixer.to_json(),
                "mlp": None if self.ff is None else {"ff": self.ff, "kind": "dense", "limit": self.limit}}


def _heads(m: Dict[str, Any], what: str):
    heads, kv_heads, dim, vdim = (_int(m, k, what) for k in ("heads", "kv_heads", "dim", "vdim"))
    if heads % kv_heads:
        raise ConfigError(f"config.json: {what}: heads must be a multiple of kv_heads")
    return heads, kv_heads, dim, vdim


def _rotary_attention(m: Dict[str, Any], what: str) -> RotaryAttentionSizes:
    heads, kv_heads, dim, vdim = _heads(m, what)
    base, dims, scaling = None, 0, None
    if m.get("rot") is not None:
        rot = _obj(m["rot"], what + ".rot")
        dims = _int(rot, "dims", what + ".rot")
        if dims % 2 or dims > dim:
            raise ConfigError(f"config.json: {what}.rot.dims must be even and at most dim")
        base = _num(rot, "base", what + ".rot")
        if not base > 0:
            raise ConfigError(f"config.json: {what}.rot.base must be positive")
        if rot.get("scaling") is not None:
            sc = _obj(rot["scaling"], what + ".rot.scaling")
            scaling = tuple(_num(sc, k, what + ".rot.scaling") for k in ("factor", "low", "high", "original"))
            if not all(v > 0 for v in scaling) or scaling[1] == scaling[2]:
                raise ConfigError(f"config.json: {what}.rot.scaling needs positive numbers with low and high apart")
    return RotaryAttentionSizes(heads, kv_heads, dim, vdim, _num(m, "scale", what), base, dims, scaling)


def _conv_window_attention(m: Dict[str, Any], what: str) -> ConvWindowAttentionSizes:
    heads, kv_heads, dim, vdim = _heads(m, what)
    window = None if m.get("mask") is None else _int(_obj(m["mask"], what + ".mask"), "size", what + ".mask")
    conv = None if m.get("conv") is None else _int(m, "conv", what)
    softcap = None
    if m.get("softcap") is not None:
        softcap = _num(m, "softcap", what)
        if not softcap > 0:
            raise ConfigError(f"config.json: {what}.softcap must be positive")
    return ConvWindowAttentionSizes(heads, kv_heads, dim, vdim, _num(m, "scale", what), window, conv, softcap)


def _gated_linear(m: Dict[str, Any], what: str) -> GatedLinearSizes:
    heads, dim, vdim = (_int(m, k, what) for k in ("heads", "dim", "vdim"))
    tau = _num(m, "tau", what)
    if not tau > 0:
        raise ConfigError(f"config.json: {what}.tau must be positive")
    rank = 0 if m.get("rank") is None else _int(m, "rank", what)        # 0: as the checkpoint's shapes say
    return GatedLinearSizes(heads, dim, vdim, tau, rank)


@dataclass(frozen=True)
class FovezenConfig:
    width: int
    vocab: int
    eps: float
    layers: Tuple[FovezenLayer, ...]
    streams: Optional[int] = None                       # None: one plain residual stream
    logit_scale: float = 1.0
    loop: Optional[Tuple[int, int, int]] = None         # start, stop, times
    max_position: int = DEFAULT_CONTEXT

    architecture = "Fovezen"
    model_type = "fovezen"

    @classmethod
    def from_json(cls, j: Any) -> "FovezenConfig":
        j = _obj(j, "the configuration")
        width, vocab = _int(j, "width", "the model"), _int(j, "vocab", "the model")
        eps = _num(_obj(j.get("norm"), "norm"), "eps", "norm")
        if not eps >= 0:
            raise ConfigError("config.json: norm.eps must be >= 0")
        raw = j.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a list with at least one layer")
        layers: List[FovezenLayer] = []
        for i, entry in enumerate(raw):
            what = f"layer {i}"
            entry = _obj(entry, what)
            kind = entry.get("type")
            m = _obj(entry.get("mixer"), what + ".mixer")
            if kind == "attention":
                mixer = _rotary_attention(m, what + ".mixer")
            elif kind == "mamba2":
                mixer = _state_space(m, what + ".mixer")
            elif kind == "parallel":
                mixer = ParallelPairSizes(_conv_window_attention(_obj(m.get("left"), what + ".mixer.left"), what + ".mixer.left"),
                                          _gated_linear(_obj(m.get("right"), what + ".mixer.right"), what + ".mixer.right"))
            else:
                raise ConfigError(f"config.json: {what} has the unknown type {kind!r} (known: {', '.join(MIXER_TYPES)})")
            ff, limit = None, 0.0
            if entry.get("mlp") is not None:
                mlp = _obj(entry["mlp"], what + ".mlp")
                if mlp.get("kind") != "dense":
                    raise ConfigError(f"config.json: {what}.mlp has the unknown kind {mlp.get('kind')!r} (known: dense)")
                ff, limit = _int(mlp, "ff", what + ".mlp"), _num(mlp, "limit", what + ".mlp")
                if not limit > 0:
                    raise ConfigError(f"config.json: {what}.mlp.limit must be positive")
            layers.append(FovezenLayer(kind, mixer, ff, limit))
        streams = None if j.get("streams") is None else _int(j, "streams", "the model")
        if streams is not None and streams > 8:
            raise ConfigError(f"config.json: {streams} streams are not supported (up to 8)")
        loop = None
        if j.get("loop") is not None:
            lp = _obj(j["loop"], "loop")
            start = lp.get("start")
            if isinstance(start, bool) or not isinstance(start, int) or start < 0:
                raise ConfigError("config.json: loop.start must be a layer index")
            stop, times = _int(lp, "stop", "loop"), _int(lp, "times", "loop")
            if not (start < stop <= len(layers)):
                raise ConfigError(f"config.json: loop {start} .. {stop} does not lie inside the {len(layers)} layers")
            loop = (start, stop, times)
        scale = 1.0 if j.get("logit_scale") is None else _num(j, "logit_scale", "the model")
        max_position = DEFAULT_CONTEXT if j.get("max_position") is None else _int(j, "max_position", "the model")
        return cls(width, vocab, eps, tuple(layers), streams, scale, loop, max_position)

    def to_json(self) -> Dict[str, Any]:
        out: Dict[str, Any] = {"architecture": self.architecture, "width": self.width, "vocab": self.vocab, "norm": {"eps": self.eps},
                               "layers": [l.to_json() for l in self.layers]}
        if self.streams is not None:
            out["streams"] = self.streams
        if self.logit_scale != 1.0:
            out["logit_scale"] = self.logit_scale
        if self.loop is not None:
            out["loop"] = {"start": self.loop[0], "stop": self.loop[1], "times": self.loop[2]}
        if self.max_position != DEFAULT_CONTEXT:
            out["max_position"] = self.max_position
        return out

    # ------------------------------------------------------------------ the order of runs
    def runs(self) -> List[Tuple[int, int]]:
        """(layer, pass) in the order they run."""
        n = len(self.layers)
        if self.loop is None:
            return [(i, 0) for i in range(n)]
        start, stop, times = self.loop
        return [(i, 0) for i in range(start)] + [(i, p) for p in range(times) for i in range(start, stop)] + \
               [(i, 0) for i in range(stop, n)]

    # ------------------------------------------------------------------ translation into parts
    def _mixer_spec(self, layer: FovezenLayer) -> PartSpec:
        D, m = self.width, layer.mixer
        if layer.type == "attention":
            position = PartSpec("none", {})
            if m.rot_base is not None:
                p = {"head_dim": m.dim, "rotary_dim": m.rot_dims, "theta": m.rot_base, "pairing": "half_split"}
                if m.rot_scaling is not None:
                    p["wavelength_scaling"] = dict(zip(("factor", "low", "high", "original"), m.rot_scaling))
                position = PartSpec("rope_on_device", p)
            return PartSpec("attention", {
                "hidden_size": D, "num_heads": m.heads, "num_kv_heads": m.kv_heads, "head_dim": m.dim, "value_dim": m.vdim,
                "scale": m.scale, "window": None, "position": position, "qk_norm_eps": self.eps, "qk_norm_wide": True})
        if layer.type == "mamba2":
            return PartSpec("state_space", {
                "hidden_size": D, "num_heads": m.heads, "head_dim": m.vdim, "state_size": m.state, "groups": m.groups,
                "conv_taps": m.conv, "norm_groups": m.norm_groups, "norm_eps": self.eps})
        a, g = m.left, m.right
        left = PartSpec("attention", {
            "hidden_size": D, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": a.dim, "value_dim": a.vdim,
            "scale": a.scale, "window": a.window, "position": PartSpec("none", {}), "qk_norm_eps": self.eps,
            "conv_taps": a.conv, "softcap": a.softcap})
        right = PartSpec("gated_linear_attention", {
            "hidden_size": D, "num_heads": g.heads, "key_dim": g.dim, "value_dim": g.vdim, "tau": g.tau, "decay_rank": g.rank or None,
            "norm_eps": self.eps})
        return PartSpec("parallel", {"branches": [("left", left, 1.0), ("right", right, 1.0)], "combine": "mean_normed",
                                     "combine_eps": self.eps, "hidden_size": D})

    def model_spec(self) -> ModelSpec:
        D = self.width
        norm = PartSpec("rmsnorm", {"size": D, "eps": self.eps, "weight_offset": 1.0})
        specs = []
        for layer in self.layers:
            ffn = None if layer.ff is None else PartSpec("gated_mlp", {
                "hidden_size": D, "intermediate_size": layer.ff, "activation": "capped_swish", "activation_limit": layer.limit})
            specs.append(LayerSpec(mixer=self._mixer_spec(layer), feed_forward=ffn, mixer_norm=norm,
                                   feed_forward_norm=None if ffn is None else norm, block="hyper_connections",
                                   block_params={"streams": self.streams or 1}))
        # a further pass of a looped layer: a layer of its own for the cache manager, the owner's parts and weights
        schedule, shared = [], {}
        for i, p in self.runs():
            if p == 0:
                schedule.append(ScheduleEntry(i))
            else:
                specs.append(specs[i])
                shared[len(specs) - 1] = i
                schedule.append(ScheduleEntry(i, cache_of=len(specs) - 1))
        return ModelSpec(architecture=self.architecture, hidden_size=D, vocab_size=self.vocab, max_position=self.max_position,
                         layers=specs, schedule=schedule, final_norm=norm, tie_word_embeddings=False,
                         logit_transform=None if self.logit_scale == 1.0 else PartSpec("scale", {"factor": self.logit_scale}),
                         open_ended=True, shared_layers=shared)
