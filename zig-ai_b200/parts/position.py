"""Position encodings.

Rotary embedding in the half-split pairing: for i < rotary_dim/2 the pair (x[i], x[i + rotary_dim/2])
is rotated by the angle pos * theta^(-2i/rotary_dim) (the reference's device kernel,
src/cuda/layer_kernels.cu:343-366; its host version pairs (2i, 2i+1), src/transformer/rope.zig:41-53).
The position is the token's absolute position in its request.  Angles are computed in 32-bit.
"""
from __future__ import annotations

from .base import PositionEncoding, register_part


class RotaryHalfSplit(PositionEncoding):
    """`scaling` = {factor, original, fast, slow} stretches the rotation for contexts longer than `original`
    positions: with where(t) = n ln(original / (2 pi t)) / (2 ln theta), lo = max(floor(where(fast)), 0),
    hi = min(ceil(where(slow)), n - 1) and ramp_i = clamp((i - lo) / max(hi - lo, 0.001), 0, 1), pair i turns at
    f_i (1 - ramp_i) + f_i ramp_i / factor, and cosines and sines are multiplied by 0.1 ln(factor) + 1."""
    pairing = "half_split"

    def __init__(self, head_dim: int, theta: float, rotary_dim: int = None, scaling=None):
        self.head_dim = int(head_dim)
        self.rotary_dim = int(head_dim if rotary_dim is None else rotary_dim)
        self.theta = float(theta)
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} should be even and at most head_dim {self.head_dim}")
        self.scaling = None
        if scaling is not None and scaling.get("kind") == "wavelength":
            # frequencies stretched by their wavelength l = 2 pi / f: kept where l < original / high, divided by `factor`
            # where l > original / low, and between the two mixed by s = (original / l - low) / (high - low):
            # (1 - s) f / factor + s f.  Cosines and sines keep their size.
            self.scaling = ("wavelength",) + tuple(float(scaling[k]) for k in ("factor", "low", "high", "original"))
        elif scaling is not None:
            self.scaling = tuple(float(scaling[k]) for k in ("factor", "original", "fast", "slow"))

    def rotary(self):
        """(rotary_dim, theta) for the kernels that make the plain rotation's table themselves; a stretched
        rotation has none and is applied from `table`."""
        return (self.rotary_dim, self.theta) if self.scaling is None else None

    def table(self, step, device):
        """(rotated dimensions, (cos, sin) per row of the step and pair [N, dims/2, 2] in 32-bit), made once per
        step and rotation."""
        return self.rotary_dim, step.ops.rope_table(step, self.rotary_dim, self.theta, device, self.scaling)

    def to_half_split(self, head_dim: int):
        """The order of a head's dimensions in which this rotation pairs (i, i + dims/2); None: as stored."""
        return None


class RotaryInterleaved(RotaryHalfSplit):
    """Pairs (2i, 2i + 1) of the first `rotary_dim` dimensions turn by position * theta^(-2i/rotary_dim).  A dot
    product does not change when both vectors' dimensions are reordered alike, so a mixer reorders the rows of
    its q and k projections once at load (`to_half_split`) and the kernels rotate pairs (i, i + dims/2)."""
    pairing = "interleaved"

    def to_half_split(self, head_dim: int):
        n = self.rotary_dim
        return list(range(0, n, 2)) + list(range(1, n, 2)) + list(range(n, int(head_dim)))


class NoPosition(PositionEncoding):
    def __init__(self, head_dim: int = 0):
        self.head_dim = head_dim

    def rotary(self):
        return 0, 1.0

    def table(self, step, device):
        return 0, None

    def to_half_split(self, head_dim: int):
        return None


register_part("position", "rotary_half_split", RotaryHalfSplit)
register_part("position", "rotary_interleaved", RotaryInterleaved)
register_part("position", "none", NoPosition)
