"""Splitting the op over GPUs: (batch, kv-head) units are independent, so a rank takes a
contiguous run of units, slices its inputs and runs the same kernels; nothing is exchanged on
the data path (the reference has no distributed code to mirror: every kernel's outer grid
dimension is B*Hkv, nsa_selection_kernel.py:119-122)."""


def unit_range(n_units: int, world: int, rank: int):
    """[first, last) units of `rank` when n_units are dealt out as evenly as possible."""
    base, extra = divmod(n_units, world)
    first = rank * base + min(rank, extra)
    return first, first + base + (1 if rank < extra else 0)


def slice_units(t, Hkv: int, first: int, last: int):
    """View of the units [first, last) of a [B, H, T, X] tensor with H = Hkv * G heads, as a
    [n_units, G, T, X] tensor (batch and kv-head folded into the leading dimension; for the op
    a unit is simply a batch entry with one kv head)."""
    B, H, T, X = t.shape
    G = H // Hkv
    return t.reshape(B * Hkv, G, T, X)[first:last]


def merge_units(parts, B: int, Hkv: int):
    """Inverse of slice_units over the concatenation of all ranks' parts, in rank order."""
    import torch
    full = torch.cat(list(parts), dim=0)
    n, G, T, X = full.shape
    assert n == B * Hkv
    return full.reshape(B, Hkv * G, T, X)
