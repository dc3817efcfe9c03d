"""Backend status record shared by the public status functions.

Same fields, order and immutability as the reference's ``BackendStatus``
(``gfx1010_kernels/attention.py:14-19`` of T-vaccari/gfx1010-kernels), which
the residual LayerNorm path imports at ``gfx1010_kernels/normalization.py:7``.
Only the record is carried over; the attention operator it lives beside in the
reference is a different path and is not part of this build.
"""

from dataclasses import dataclass
from typing import Optional


@dataclass(frozen=True)
class BackendStatus:
    available: bool
    device: Optional[str]
    architecture: Optional[str]
    reason: str
