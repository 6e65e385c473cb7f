"""Level arithmetic and the enums of the reference's `hattention/base.py` (lines 12-46).

The reference materialises a T x T int64 lookup table of Fenwick levels
(`make_levels_matrix`, base.py:101-161); the kernels here evaluate the closed form
bit_length(t XOR s) instead, so no table exists and no length limit applies.
"""
from enum import Enum


class HType(Enum):
    WEAK = 0
    STRONG = 1


class HStruct(Enum):
    MAMBA2 = 0
    GDELTA = 1


def ceil_log(x: int, b: int) -> int:
    """ceil(log_b(x)) in exact integer arithmetic (base.py:29-30)."""
    if b != 2:
        raise NotImplementedError("only level_base=2 is supported")
    return (int(x) - 1).bit_length()


def get_num_levels(length: int, base: int) -> int:
    """Levels needed for `length` positions (base.py:37-38)."""
    return ceil_log(length, base) + 1


def get_level_index(t: int, s: int, b: int = 2, htype: HType = HType.WEAK) -> int:
    """Bucket of source s for target t > s (base.py:41-72, WEAK hierarchy only)."""
    if t <= s:
        raise ValueError
    if htype != HType.WEAK or b != 2:
        raise NotImplementedError
    return (t ^ s).bit_length()
