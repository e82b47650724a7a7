"""Position encodings."""
from __future__ import annotations

import math

import numpy as np
import torch

from .registry import register_logit_transform, register_position_encoding


def rope_frequencies(head_dim: int, theta: float, scaling, rotary_dim=None, round_theta: bool = True) -> np.ndarray:
    """Rotation frequency of each pair in double precision: 1/theta^(2k/rotary_dim), with the
    "llama3" scaling when given (src/kernels/kernels.cpp:142-163). theta is rounded to 32-bit
    first, as the reference stores it so (src/loader/hf_checkpoint.cpp:125)."""
    rd = rotary_dim or head_dim
    theta = float(np.float32(theta)) if round_theta else float(theta)
    k = np.arange(rd // 2, dtype=np.float64)
    freq = 1.0 / np.power(theta, 2.0 * k / rd)
    if scaling:
        factor = float(scaling["factor"])
        low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
        original = float(scaling["original_max_position"])
        wavelength = 6.283185307179586476925 / freq
        out = freq.copy()
        slow = wavelength > original / low
        out[slow] = freq[slow] / factor
        mid = ~slow & ~(wavelength < original / high)
        smooth = (original / wavelength - low) / (high - low)
        out[mid] = ((1.0 - smooth) * freq / factor + smooth * freq)[mid]
        freq = out
    return freq


@register_position_encoding("rope")
class RotaryPosition:
    """Rotary position encoding applied to queries and keys before the key is stored. Owns the
    cos/sin table [max_position, rotary_dim/2], computed on the host in double precision and
    rounded to 32-bit once (src/kernels/kernels.cpp:159-161). Params: ``head_dim``, ``theta``,
    ``pairing`` ("half_split": pair k is (v[k], v[k+rd/2]); "interleaved": (v[2k], v[2k+1])),
    ``scaling`` (None or the four llama3 numbers), optional ``rotary_dim`` (< head_dim rotates only
    the first dims)."""

    applies = "qk_before_store"
    not_weights = ("cos", "sin")        # tables computed from constants: not counted among a model's weight bytes

    def __init__(self, params, weights, build):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        pairing = params.get("pairing", "half_split")
        if pairing not in ("half_split", "interleaved"):
            raise ValueError(f"rope: unknown pairing '{pairing}'")
        self.interleaved = pairing == "interleaved"
        freq = rope_frequencies(self.head_dim, params["theta"], params.get("scaling"), self.rotary_dim)
        pos = np.arange(build.max_position, dtype=np.float64)[:, None]
        angle = pos * freq[None, :]
        self.cos = torch.from_numpy(np.cos(angle).astype(np.float32)).to(build.device).contiguous()
        self.sin = torch.from_numpy(np.sin(angle).astype(np.float32)).to(build.device).contiguous()


@register_position_encoding("none")
class NoPosition:
    """No position encoding: queries and keys are stored as they are."""

    applies = "none"
    interleaved = False
    cos = None
    sin = None

    def __init__(self, params, weights, build):
        pass


@register_position_encoding("rope_on_device")
class RotaryOnDevice:
    """Rotary position encoding whose angles are computed where they are applied: the kernel multiplies
    the 32-bit position by the pair's 32-bit frequency and takes sine and cosine, so no table of
    ``max_position`` rows exists and no position is too far. Params: ``head_dim``, ``theta``, ``pairing``
    ("interleaved" or "half_split"), optional ``rotary_dim`` (< head_dim rotates only the first dims).
    ``freq`` [rotary_dim / 2] = theta^(-2i / rotary_dim), taken in double and rounded once.

    Optional ``ramp_scaling`` {factor, original, fast, slow} stretches the slow pairs for contexts longer than
    ``original`` positions: with n(t) = rotary_dim ln(original / (2 pi t)) / (2 ln theta) the index of the pair that
    turns t times within ``original`` positions, lo = max(floor(n(fast)), 0), hi = min(ceil(n(slow)), rotary_dim - 1)
    and r_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at f_i (1 - r_i) + f_i r_i / factor, and
    cos and sin are multiplied by ``amplitude`` = 0.1 ln(factor) + 1 (1 without scaling).

    Optional ``wavelength_scaling`` {factor, low, high, original}: a pair whose wavelength 2 pi / f is shorter than
    original / high keeps f, one whose wavelength is longer than original / low turns at f / factor, and between the two
    f (1 - s) / factor + f s with s = (original / wavelength - low) / (high - low) (the frequencies of ``rope_frequencies``
    with its "llama3" scaling, computed once in double)."""

    applies = "qk_before_store"
    cos = None
    sin = None
    not_weights = ("freq",)

    def __init__(self, params, weights, build):
        self.head_dim = int(params["head_dim"])
        self.rotary_dim = int(params.get("rotary_dim") or self.head_dim)
        if self.rotary_dim % 2 or self.rotary_dim > self.head_dim:
            raise ValueError(f"rope: rotary_dim {self.rotary_dim} must be even and at most head_dim {self.head_dim}")
        pairing = params.get("pairing", "half_split")
        if pairing not in ("half_split", "interleaved"):
            raise ValueError(f"rope: unknown pairing '{pairing}'")
        self.interleaved = pairing == "interleaved"
        i = np.arange(self.rotary_dim // 2, dtype=np.float64)
        freq = np.power(float(params["theta"]), -2.0 * i / self.rotary_dim)
        self.amplitude = 1.0
        ramp = params.get("ramp_scaling")
        if ramp:
            factor, original = float(ramp["factor"]), float(ramp["original"])
            if not (factor > 0 and original > 0 and float(ramp["fast"]) > 0 and float(ramp["slow"]) > 0):
                raise ValueError("rope: the numbers of ramp_scaling must be positive")

            def pair_index(turns: float) -> float:
                return self.rotary_dim * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(float(params["theta"])))

            lo = max(math.floor(pair_index(float(ramp["fast"]))), 0)
            hi = min(math.ceil(pair_index(float(ramp["slow"]))), self.rotary_dim - 1)
            r = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
            freq = freq / factor * r + freq * (1.0 - r)
            self.amplitude = 0.1 * math.log(factor) + 1.0
        wave = params.get("wavelength_scaling")
        if wave:
            if ramp:
                raise ValueError("rope: ramp_scaling and wavelength_scaling exclude one another")
            freq = rope_frequencies(self.head_dim, float(params["theta"]), {
                "factor": wave["factor"], "low_freq_factor": wave["low"], "high_freq_factor": wave["high"],
                "original_max_position": wave["original"]}, self.rotary_dim, round_theta=False)
        self.freq = torch.from_numpy(freq.astype(np.float32)).to(build.device).contiguous()


@register_position_encoding("learned")
class LearnedPosition:
    """A table of learned vectors, one per position, added as they are to the embedding's output; queries and keys are not rotated.
    Params: ``size`` (the model's width), ``positions`` (rows of the table: no position beyond it exists). Weights:
    ``table`` [positions, size]. The model calls ``add_to(ctx, x)`` once per step, after the embedding."""

    applies = "embedding"
    cos = sin = None
    interleaved = False

    def __init__(self, params, weights, build):
        size, rows = int(params["size"]), int(params["positions"])
        table = weights["table"]
        if tuple(table.shape) != (rows, size):
            raise ValueError(f"learned positions: the table has shape {tuple(table.shape)}, expected ({rows}, {size})")
        if build.max_position > rows:
            raise ValueError(f"learned positions: the table has {rows} rows, the context length is {build.max_position}")
        self.table = table.to(device=build.device, dtype=build.compute_dtype).contiguous()

    def add_to(self, ctx, x: torch.Tensor) -> None:
        from ..ops import kernels
        kernels.add_rows_at(x, self.table, ctx.positions)


@register_logit_transform("softcap")
class SoftCap:
    """logits <- cap * tanh(logits / cap), in place, 32-bit. Params: ``cap`` (> 0)."""

    def __init__(self, params, weights, build):
        self.cap = float(params["cap"])
        if not self.cap > 0:
            raise ValueError("softcap: the cap must be positive")

    def forward(self, ctx, logits: torch.Tensor) -> None:
        from ..ops import kernels
        kernels.softcap(logits, self.cap)


@register_logit_transform("scale")
class LogitScale:
    """logits <- factor * logits, in place, 32-bit. Params: ``factor``."""

    def __init__(self, params, weights, build):
        self.factor = float(params["factor"])

    def forward(self, ctx, logits: torch.Tensor) -> None:
        from ..ops import kernels
        kernels.scale(logits, self.factor)
