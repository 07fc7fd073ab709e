"""Names of the reference module ``ops3d/flash_deform_attn.py`` that callers import: the autograd
function (``:65-136``) and the launch-hint helpers (``:17-62``)."""
from ops3d_b200.flash_deform_attn import FlashDeformAttnFunction, findspec, findspec_bwd

from ._extension import _C  # noqa: F401


def factors(N):
    """All positive divisors of ``N`` in increasing order (reference ``:17-23``), found in O(sqrt(N))."""
    small, large = [], []
    i = 1
    while i * i <= N:
        if N % i == 0:
            small.append(i)
            if i != N // i:
                large.append(N // i)
        i += 1
    return small + large[::-1]


__all__ = ["FlashDeformAttnFunction", "findspec", "findspec_bwd", "factors"]
