"""Number-format descriptors (plain Python; no arithmetic happens here).

API-compatible with the reference's ``mptorch/number.py`` (classes, constructor arguments and the
public attributes the quantization layer reads): ``FloatingPoint`` (number.py:114-179),
``SuperNormalFloat`` (:182-246), ``Binary8`` (:279-383), ``FixedPoint`` (:44-111) and
``BlockFloatingPoint`` (:249-276).  The last two are kept as descriptors only: fixed-point and
block-floating-point arithmetic is outside this library's hot path.
"""
from __future__ import annotations

__all__ = ["Number", "FloatType", "FixedPoint", "FloatingPoint", "BlockFloatingPoint", "SuperNormalFloat", "Binary8"]


class Number:
    """Base class of every format descriptor."""

    def __str__(self) -> str:
        raise NotImplementedError

    def __repr__(self) -> str:
        raise NotImplementedError


class FloatType(Number):
    """Marker base class of the float-like formats."""


class FixedPoint(Number):
    """Fixed point: word length ``wl``, fractional length ``fl`` (descriptor only)."""

    def __init__(self, wl: int, fl: int, clamp: bool = True, symmetric: bool = False):
        assert wl > 0, "invalid bits for word length:{}".format(wl)
        assert fl >= 0, "invalid bits for fractional length: {}".format(fl)
        assert isinstance(clamp, bool), "invalid type for clamping choice: {}".format(type(clamp))
        assert isinstance(symmetric, bool), "invalid type for symmetric: {}".format(type(symmetric))
        self.wl, self.fl, self.clamp, self.symmetric = wl, fl, clamp, symmetric

    def __str__(self):
        return "FixedPoint (wl={:d}, fl={:d})".format(self.wl, self.fl)

    __repr__ = __str__


class FloatingPoint(FloatType):
    """IEEE-754-like format with ``exp`` exponent bits (bias 2^(exp-1) - 1) and ``man`` stored mantissa bits.

    The all-ones exponent is reserved, so e.g. (exp=4, man=3) tops out at 240, not at OCP E4M3's 448.
    """

    def __init__(self, exp: int, man: int, subnormals: bool = False, saturate: bool = True):
        assert 8 >= exp > 0, "invalid bits for exponent:{}".format(exp)
        assert 23 >= man >= 0, "invalid bits for mantissa:{}".format(man)
        self.exp, self.man, self.subnormals, self.saturate = exp, man, subnormals, saturate
        emin = 2 - 2 ** (exp - 1)
        emax = 2 ** (exp - 1) - 1
        self.normal_min = 2.0 ** emin
        self.normal_max = 2.0 ** emax * (2.0 - 2.0 ** (-man))
        self.subnormal_min = 2.0 ** (emin - man) if subnormals else None
        self.subnormal_max = 2.0 ** emin * (1.0 - 2.0 ** (-man)) if subnormals else None

    def __str__(self):
        return "FloatingPoint (exponent={:d}, mantissa={:d})".format(self.exp, self.man)

    __repr__ = __str__

    @property
    def is_fp32(self) -> bool:
        return self.man == 23 and self.exp == 8

    @property
    def is_fp16(self) -> bool:
        return self.man == 10 and self.exp == 5

    @property
    def is_bfloat16(self) -> bool:
        return self.man == 7 and self.exp == 8


class SuperNormalFloat(FloatType):
    """Floating point whose lowest ``binades_l`` and highest ``binades_u`` binades are re-used as
    logarithmic ("supernormal") ranges."""

    def __init__(self, exp: int, man: int, binades: int | tuple[int] | tuple[int, int], saturate: bool = False):
        assert 8 >= exp > 0, "invalid bits for exponent:{}".format(exp)
        assert 23 >= man >= 0, "invalid bits for mantissa:{}".format(man)
        self.exp, self.man = exp, man
        if isinstance(binades, int):
            self.binades_l = self.binades_u = binades
        elif len(binades) == 1:
            self.binades_l = self.binades_u = binades[0]
        else:
            self.binades_l, self.binades_u = binades[0], binades[1]
        self.binades = (self.binades_l, self.binades_u)
        self.saturate = saturate
        min_exp = 1 - 2 ** (exp - 1) + (self.binades_l - 1)
        max_exp = 2 ** (exp - 1) - 2 - (self.binades_u - 1)
        self.subnormal_min = 2 ** (min_exp - self.binades_l * (2 ** man) + 1)
        self.subnormal_max = 2 ** (min_exp - 1)
        self.normal_min = 2 ** min_exp
        self.normal_max = 2 ** max_exp
        self.supernormal_min = 2 ** (max_exp + 1)
        self.supernormal_max = 2 ** (max_exp + self.binades_u * (2 ** man) - 1)

    def __str__(self):
        return "SuperNormalFloat (exponent={:d}, mantissa={:d}, binades={})".format(self.exp, self.man, self.binades)

    __repr__ = __str__


class BlockFloatingPoint(Number):
    """Block floating point with a shared exponent along ``dim`` (descriptor only)."""

    def __init__(self, wl: int, dim: int = -1):
        assert wl > 0 and isinstance(wl, int), "invalid bits for word length:{}".format(wl)
        assert dim >= -1 and isinstance(dim, int), "invalid dimension"
        self.wl, self.dim = wl, dim

    def __str__(self):
        return "BlockFloatingPoint (wl={:d}, dim={:d})".format(self.wl, self.dim)

    __repr__ = __str__


class Binary8(FloatType):
    """IEEE P3109 ``binary8`` with precision ``P``: ``P - 1`` mantissa bits and ``8 - P`` (signed) or
    ``9 - P`` (unsigned) exponent bits."""

    POLICIES = ("saturate_infty", "saturate_maxfloat", "saturate_maxfloat2")

    def __init__(self, P: int, signed: bool = True, subnormals: bool = True,
                 overflow_policy: str = "saturate_maxfloat2"):
        assert 8 > P > 0, "Invalid P: {}".format(P)
        assert overflow_policy in self.POLICIES, "Invalid overflow policy: {}".format(overflow_policy)
        self.P = P
        self.man = P - 1
        self.exp = (8 - P) if signed else (9 - P)
        max_exp = 2 ** (self.exp - 1) - 1
        min_exp = -max_exp + (1 if P == 1 else 0)
        man = self.man
        if man != 1 and subnormals:
            self.subnormal_min = (2 ** -man) * (2 ** min_exp)
            self.subnormal_max = (1 - 2 ** -man) * (2 ** min_exp)
        else:
            self.subnormal_min = self.subnormal_max = None
        self.normal_min = 2 ** min_exp if (subnormals or man == 1) else (1 + 2 ** -man) * (2 ** (min_exp - 1))
        # How many of the top code points are reserved (NaN, and infinity where the policy keeps one)
        # decides the largest finite value.
        wide = overflow_policy == "saturate_maxfloat2"
        if signed:
            if wide:
                self.normal_max = (2 - 2 ** -man) * 2 ** max_exp if man > 0 else 2 ** (max_exp + 1)
            else:
                self.normal_max = (2 - 2 ** -(man - 1)) * 2 ** max_exp if man > 0 else 2 ** max_exp
        else:
            if wide:
                self.normal_max = (2 - 2 ** -(man - 1)) * 2 ** max_exp if man > 0 else 2 ** max_exp
            else:
                self.normal_max = (2 - 2 ** -man - 2 ** -(man - 1)) * 2 ** max_exp if man > 0 else 2 ** (max_exp - 1)
        self.signed, self.subnormals, self.overflow_policy = signed, subnormals, overflow_policy

    def __repr__(self):
        return (f"Binary8 (P={self.P}, exp={self.exp}, man={self.man}, signed={self.signed}, "
                f"subnormals={self.subnormals}, overflow_policy={self.overflow_policy})")

    __str__ = __repr__
