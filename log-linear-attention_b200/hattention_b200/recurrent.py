"""Decode-time level states, with the interface of the reference's `hattention/recurrent.py`
(`HState` :9-131).  The token recurrence itself (`step_state` / `step_output` :134-166) runs in one CUDA
kernel behind `hattention_b200.kernel.hattention_step`."""
import torch

from .base import HStruct, HType


class HState:
    """Level states of one layer for decoding, with the fields of the reference's `HState`
    (hattention/recurrent.py:9-131): `states` (B,H,K,V,L) in `dtype` and one token count per level.
    The counts are identical for every sequence and are kept on the host, so that the cascade
    (recurrent.py:42-54) costs no device synchronisation."""

    def __init__(self, base: int, htype: HType, hstruct: HStruct, shape, dtype: torch.dtype, device) -> None:
        if base != 2 or htype != HType.WEAK:
            raise NotImplementedError
        self.base, self.htype, self.hstruct = base, htype, hstruct
        self.shape, self.dtype, self.device = tuple(shape), dtype, device
        self.max_num_levels = self.shape[-1]
        self.states = torch.zeros(self.shape, dtype=dtype, device=device)
        self.counts = [0] * self.max_num_levels

    def cascade_counts(self) -> int:
        """Runs the cascade on the counts; returns the level that receives the merged levels."""
        for level in range(self.max_num_levels):
            cap = 1 << level
            if self.counts[level] == cap:
                if level + 1 >= self.max_num_levels:
                    raise ValueError("more tokens than the levels can hold")
                self.counts[level + 1] += self.counts[level]
                self.counts[level] = 0
            elif self.counts[level] < cap:
                return level
            else:
                raise ValueError
        return self.max_num_levels - 1

    def set_counts_after(self, T: int) -> None:
        """Counts after T tokens: level 0 holds the last token, level j+1 holds 2^j tokens for each set
        bit j of T-1 (the bookkeeping at the end of kernel.py:452-463)."""
        self.counts = [0] * self.max_num_levels
        if T <= 0:
            return
        self.counts[0] = 1
        m = T - 1
        for j in range(m.bit_length()):
            if (m >> j) & 1:
                if j + 1 >= self.max_num_levels:
                    raise ValueError("more tokens than the levels can hold")
                self.counts[j + 1] = 1 << j

    def set_counts_before(self, t: int) -> None:
        """Counts as the cascade leaves them just before token t (0-based) is inserted: level 0 empty, level j+1
        holds 2^j tokens for each set bit j of t."""
        self.counts = [0] * self.max_num_levels
        for j in range(max(t, 0).bit_length()):
            if (t >> j) & 1:
                if j + 1 >= self.max_num_levels:
                    raise ValueError("more tokens than the levels can hold")
                self.counts[j + 1] = 1 << j

    def reset_states(self) -> None:
        """recurrent.py:102-103; the token counts restart with the states."""
        self.states = torch.zeros_like(self.states)
        self.counts = [0] * self.max_num_levels

    def replace(self, other: "HState") -> None:
        """Adopt another state of the same shape (recurrent.py:105-115), token counts included: the cascade
        of the next decode step depends on them."""
        if not (tuple(self.shape) == tuple(other.shape) and self.base == other.base and self.htype == other.htype
                and self.dtype == other.dtype and torch.device(self.device) == torch.device(other.device)):
            raise ValueError("Shape, dtype or device mismatch")
        self.states = other.states
        self.counts = list(other.counts)

    def to(self, dtype=None, device=None) -> "HState":
        """recurrent.py:117-131.  The states stay fp32 (the decode kernel reads fp32 states and casts its
        output), so only fp32 / the same device is a no-op copy; other targets are not supported."""
        if (dtype is not None and dtype != self.dtype) or (device is not None and torch.device(device) != torch.device(self.device)):
            raise NotImplementedError("level states are kept in fp32 on their device")
        new = HState(self.base, self.htype, self.hstruct, self.shape, self.dtype, self.device)
        new.states = self.states
        new.counts = list(self.counts)
        return new
