"""Rotary position encoding, NeoX pairing over the whole head."""
from __future__ import annotations

import math

import torch

from .base import POSITIONS, PositionEncoding


@POSITIONS.register("rope_neox")
class NeoxRope(PositionEncoding):
    """Pairs (i, i + d/2) of a head are rotated by pos * theta^(-2i/d)
    (maeddesg/ROCmForge hip_kernels/rope.hip:57-90, src/cpu/ops.rs:69-98 with neox=true).

    ``rotary_dim`` (default: the whole head) limits the rotation to the first elements of a head, d then being
    ``rotary_dim``; ``interleaved`` pairs (2i, 2i+1) instead (the reference's neox=false branch, src/cpu/ops.rs:86-96).

    The reference evaluates powf in the kernel; here the d/2 frequencies are computed
    once in double precision, rounded to float32 and shared by every kernel, so that
    all of them (and the plain implementation) rotate by the same angle
    float32(pos) * float32(freq).

    ``scaling`` (a dict factor, low, high, original) stretches the frequencies by wavelength l = 2 pi / f, as the
    Llama 3.1 models do: f stays where l < original/high, becomes f / factor where l > original/low, and in between
    (1 - s) f / factor + s f with s = (original/l - low) / (high - low).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, interleaved: bool = False, scaling=None):
        rot = head_dim if rotary_dim is None else int(rotary_dim)
        if head_dim % 2 or rot % 2 or not 0 < rot <= head_dim:
            raise ValueError(f"rotary encoding needs an even head_dim and an even rotary_dim in (0, head_dim]; "
                             f"got {head_dim} and {rot}")
        self.head_dim, self.rotary_dim, self.interleaved = head_dim, rot, bool(interleaved)
        self.theta = float(theta)
        i = torch.arange(rot // 2, dtype=torch.float64)
        freq = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / rot)
        self.scaling = None if scaling is None else {k: float(scaling[k]) for k in ("factor", "low", "high", "original")}
        if self.scaling is not None:
            freq = self.scaled_by_wavelength(freq, **self.scaling)
        self.inv_freq_host = freq.to(torch.float32)
        self.inv_freq = None

    @staticmethod
    def scaled_by_wavelength(freq: torch.Tensor, factor: float, low: float, high: float, original: float) -> torch.Tensor:
        if not (factor > 0 and high > low and original > 0):
            raise ValueError(f"frequency scaling needs factor > 0, high > low and original > 0; got {factor}, {low}, {high}, {original}")
        wave = 2.0 * math.pi / freq
        blend = (original / wave - low) / (high - low)
        mixed = (1.0 - blend) * freq / factor + blend * freq
        return torch.where(wave < original / high, freq, torch.where(wave > original / low, freq / factor, mixed))

    def prepare(self, device):
        self.inv_freq = self.inv_freq_host.to(device)

    def rotation(self):
        return dict(inv_freq=self.inv_freq, rot_dim=self.rotary_dim, interleaved=self.interleaved)


@POSITIONS.register("rope_yarn")
class YarnRope(NeoxRope):
    """The same rotation with frequencies stretched over a ramp of pair indices and with longer pairs (YaRN).

    With f_i = theta^(-2i/d), d the rotary size, and index(t) = d ln(original / (2 pi t)) / (2 ln theta), the pair index
    at which a pair makes t turns over ``original`` positions:

        lo = max(floor(index(fast)), 0),  hi = min(ceil(index(slow)), d - 1)
        ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1)
        frequency_i = (f_i / factor) ramp_i + f_i (1 - ramp_i)

    so pairs that turn more than ``fast`` times keep their frequency and pairs that turn less than ``slow`` times turn
    ``factor`` times slower.  Sine and cosine are multiplied by ``magnitude`` = 0.1 ln(factor) + 1, which the rotation
    kernel receives beside the frequencies (a pair grows by that factor: it is no pure rotation).
    """

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, interleaved: bool = False, *, factor: float,
                 original: float, fast: float, slow: float):
        super().__init__(head_dim, theta, rotary_dim, interleaved)
        if not (factor > 0 and original > 0 and fast > 0 and slow > 0 and theta > 1):
            raise ValueError(f"rope_yarn needs positive factor, original, fast and slow and theta > 1; got {factor}, "
                             f"{original}, {fast}, {slow}, {theta}")
        d = self.rotary_dim
        self.yarn = dict(factor=float(factor), original=float(original), fast=float(fast), slow=float(slow))

        def index_of(turns: float) -> float:
            return d * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(self.theta))
        lo = max(math.floor(index_of(fast)), 0)
        hi = min(math.ceil(index_of(slow)), d - 1)
        i = torch.arange(d // 2, dtype=torch.float64)
        f = 1.0 / torch.pow(torch.tensor(self.theta, dtype=torch.float64), 2.0 * i / d)
        ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
        self.inv_freq_host = (f / factor * ramp + f * (1.0 - ramp)).to(torch.float32)
        self.magnitude = 0.1 * math.log(factor) + 1.0

    def rotation(self):
        return dict(super().rotation(), magnitude=self.magnitude)
