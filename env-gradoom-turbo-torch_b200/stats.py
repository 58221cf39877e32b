"""Lane sharding across ranks and the one collective of the path.

Lanes are independent, so the render path shards them over the GPUs of a box
with no communication: rank r owns the contiguous global lanes
``[r*lanes_per_rank, (r+1)*lanes_per_rank)`` and holds its own copy of the
scene blob.  The only exchange is an occasional ``all_gather`` of four
per-lane episode statistics taken from the producer's signal buffer (columns of
the reference's ``DEVICE_SIGNAL_NAMES``, src/gradoom/engine.py:509-539):
killcount, episode_time, episode_return, player_killcount.  The reference is
single-device and has no counterpart for it.
"""

from __future__ import annotations

import torch
import torch.distributed as dist

STAT_COLUMNS = (0, 17, 18, 26)
STAT_NAMES = ("killcount", "episode_time", "episode_return", "player_killcount")


def lane_slice(rank: int, world_size: int, lanes_per_rank: int) -> range:
    """Global lane ids owned by ``rank``."""

    if not 0 <= rank < world_size:
        raise ValueError("rank outside the world")
    return range(rank * lanes_per_rank, (rank + 1) * lanes_per_rank)


def local_stats(signal_buffer: torch.Tensor) -> torch.Tensor:
    """``(lanes, 4) float32`` statistics block of this rank."""

    index = torch.as_tensor(STAT_COLUMNS, device=signal_buffer.device)
    return signal_buffer.index_select(1, index).contiguous().to(torch.float32)


def gather_lane_stats(signal_buffer: torch.Tensor, group=None) -> torch.Tensor:
    """All-gather the statistics of every rank: ``(world*lanes, 4)`` in global lane order.

    Without an initialised process group (single GPU) it returns the local block.
    """

    block = local_stats(signal_buffer)
    if not (dist.is_available() and dist.is_initialized()):
        return block
    world = dist.get_world_size(group)
    out = torch.empty((world * block.shape[0], block.shape[1]), dtype=block.dtype, device=block.device)
    dist.all_gather_into_tensor(out, block, group=group)
    return out
