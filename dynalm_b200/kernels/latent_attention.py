"""Chooses the latent-attention kernel for a step, and cuts the step into query tiles for the tensor-core one.

float32 always runs the plain kernel (csrc/latent_attention.cu), whose arithmetic for a row is fixed by the row
alone. bfloat16 runs the tensor-core kernel (csrc/latent_attention_flash.cu) when the record's two pieces are
multiples of 8 numbers and the latent has at most 512: its blocks take 32 query units, a unit being (row, head), so
the host cuts every request of the step into tiles of 32 / heads-to-a-block consecutive rows (a step plan, sent with
the step's integers). Prompt portions and single decoded tokens go through the same launch.
"""

from __future__ import annotations

import torch

from . import ops
from .device import sm_count

UNITS = 32          # query units (row, head) to a block of the tensor-core kernel


def heads_per_block(heads: int) -> int:
    """Heads to a block: all of them up to 32, else the heads dealt evenly over the fewest blocks."""
    groups = -(-heads // UNITS)
    return -(-heads // groups)


class LatentTilePlan:
    """Every request of the step cut into tiles of at most `rows` consecutive rows: int32 [tiles, 4] = (request slot,
    first row of the step, rows, first position), the tiles that see the most keys first. `fill` returns the number
    of tiles."""

    def __init__(self, rows: int):
        self.rows = int(rows)
        self.name = f"latent_query_tiles:{self.rows}"

    def ints(self, max_tokens: int, max_requests: int) -> int:
        return 4 * (max_tokens // self.rows + max_requests)

    def fill(self, host, shape) -> int:
        tiles = []
        for n, r0, start, slot in zip(shape.q_len, shape.q_start, shape.pos_start, shape.slots):
            for t0 in range(0, n, self.rows):
                tiles.append((slot, r0 + t0, min(self.rows, n - t0), start + t0))
        tiles.sort(key=lambda t: -(t[3] + t[2]))
        flat = [v for t in tiles for v in t]
        host[:len(flat)] = flat
        return len(tiles)


_plans = {}


def tile_plan(spec) -> LatentTilePlan:
    rows = max(1, UNITS // heads_per_block(spec.num_heads))
    plan = _plans.get(rows)
    if plan is None:
        plan = _plans[rows] = LatentTilePlan(rows)
    return plan


def flash_applies(spec, dtype) -> bool:
    return (dtype == torch.bfloat16 and spec.kv_rank % 8 == 0 and spec.rot_dim % 8 == 0 and spec.kv_rank <= 512
            and ops.latent_flash_fits(spec.kv_rank, spec.rot_dim))


KEY_TILE = 64           # keys to a tile of the tensor-core kernel
PART_ROWS = 64          # steps of single tokens up to this many rows may deal their keys over several blocks
MAX_PARTS = 16


def key_parts(ctx, spec, sms: int = 0) -> int:
    """Into how many parts the keys of every query tile are dealt. Only steps in which every request brings one token,
    and few of them: such a step has one block per request and group of heads, each walking all of its keys alone. The
    count follows the step's longest span of keys in powers of two (cut off at the window), so that a growing context
    keeps its launch shape, gives every part at least two key tiles, and aims at two blocks per SM."""
    if not ctx.decode_only or ctx.num_tokens > PART_ROWS:
        return 1
    window = int(spec.get("window", 0))
    span = 256
    while span < ctx.max_kv_len:
        span *= 2
    if window > 0:
        span = min(span, window)
    tiles = span // KEY_TILE + 1
    blocks = ctx.num_tokens * -(-spec.num_heads // heads_per_block(spec.num_heads))
    want = -(-2 * (sms or sm_count()) // blocks)
    return max(1, min(want, tiles // 2, MAX_PARTS))


def attend(wide: torch.Tensor, cache, ctx, out: torch.Tensor, spec, sink, runtime=None) -> bool:
    """The tensor-core kernel over the step's tiles; False (nothing done) when it does not take this model or step."""
    if not flash_applies(spec, wide.dtype):
        return False
    planned = ctx.extras.get(tile_plan(spec).name)
    if planned is None:
        return False
    tiles, n_tiles = planned
    (records,) = cache.arrays
    parts = key_parts(ctx, spec) if runtime is not None else 1
    scratch = None
    if parts > 1:
        scratch = runtime.flat(f"latent_parts_{spec.num_heads}_{spec.kv_rank}",
                               PART_ROWS * spec.num_heads * MAX_PARTS * (spec.kv_rank + 2))
    ops.latent_attention_flash(wide, records, cache.block_table, tiles, n_tiles, sink, out, spec.num_heads, spec.kv_rank,
                               spec.rot_dim, cache.page_size, float(spec.scale), int(spec.get("window", 0)),
                               heads_per_block(spec.num_heads), parts, scratch)
    return True
