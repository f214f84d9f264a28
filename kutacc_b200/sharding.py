"""Row partition used when the batch rows of an attention call are spread over several GPUs.

Same formula as the reference's collectives (include/kutacc.h:58-74, src/comm/all_gather.cpp:35,48):
block(x) = ceil(x / world), rank r owns rows [r*block, min((r+1)*block, x)).
"""
from __future__ import annotations

from typing import Tuple


def block(x: int, world: int) -> int:
    return (x + world - 1) // world


def chunk(x: int, world: int, rank: int) -> int:
    return max(0, min(block(x, world), x - rank * block(x, world)))


def row_range(x: int, world: int, rank: int) -> Tuple[int, int]:
    b = block(x, world)
    lo = min(x, rank * b)
    return lo, lo + chunk(x, world, rank)
