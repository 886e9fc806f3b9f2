"""Chooses the differential-attention kernel for a step.

float32 always runs the plain kernel (csrc/attention_diff.cu), whose arithmetic for a row is fixed by the row alone.
bfloat16 with map and value sizes that are multiples of 16 up to 128 runs the tensor-core kernels
(csrc/attention_diff_flash.cu): the rows at the head of a step that bring a single token each go through the
split-KV kernel, prompt portions through the flash kernel, cut into the step's query tiles
(kernels/attention.QueryTilePlan). Every other shape runs the plain kernel.
"""

from __future__ import annotations

import torch

from . import ops
from .attention import QUERY_TILES, query_tiles
from .device import sm_count

MAX_SPLITS = 32           # the merge kernel holds one part per lane
PART_MIN_KEYS = 256       # fewest keys of a part: four tiles, one 16-key group of each for every warp
TILE_KEYS = 64
BLOCKS_PER_SM = 3         # blocks of the single-token kernel that share an SM (registers allow three at every size)
BLOCK_OVERHEAD_TILES = 2  # what a block costs besides its tiles (first loads, the merge of its warps), in tiles
MERGE_TILES = 2           # what the kernel that merges the parts costs, in tiles


def fast_applies(spec, q: torch.Tensor, records: torch.Tensor, page_size: int) -> bool:
    return (q.dtype == torch.bfloat16 and spec.head_dim % 16 == 0 and spec.value_dim % 16 == 0 and spec.head_dim <= 128
            and spec.value_dim <= 128 and page_size & (page_size - 1) == 0 and q.stride(0) % 8 == 0
            and records.shape[-1] % 8 == 0 and (spec.num_kv_heads * 2 * spec.head_dim) % 8 == 0)


def split_count(rows: int, n_heads: int, n_kv_heads: int, span: int, sms: int = 0) -> int:
    """Parts every single-token row's keys are dealt into. A block walks its tiles one after the other (1.8 us a tile
    measured), so the kernel takes (rounds of blocks over the GPU) x (tiles of a block + what a block costs besides),
    plus the merge when there are parts: the count with the least of that, every part keeping PART_MIN_KEYS keys.
    Measured on B200, 8 rows of 2,048 keys on 4 KV heads: 75 us in one part, 35 us in five, 32 us in eight. The span
    is taken in powers of two, so that a growing context changes the launch shape (and the CUDA graph) only now and then."""
    bucket = PART_MIN_KEYS
    while bucket < span:
        bucket *= 2
    blocks = rows * n_kv_heads * -(-(n_heads // n_kv_heads) // 16)
    slots = BLOCKS_PER_SM * (sms or sm_count())
    tiles = bucket // TILE_KEYS
    best, least = 1, None
    for parts in range(1, min(MAX_SPLITS, bucket // PART_MIN_KEYS) + 1):
        cost = -(-blocks * parts // slots) * (-(-tiles // parts) + BLOCK_OVERHEAD_TILES) + (MERGE_TILES if parts > 1 else 0)
        if least is None or cost < least:
            best, least = parts, cost
    return best


def step_plans() -> list:
    return [QUERY_TILES]


def _single(q, records, k_off, cache, ctx, out, spec, lam, out_scale, eps, runtime, rows, n_split=None):
    if n_split is None:
        n_split = split_count(rows, spec.num_heads, spec.num_kv_heads, ctx.max_kv_len)
    scratch = None
    if n_split > 1:
        most = max(runtime.max_requests, rows)
        scratch = runtime.flat(f"diff_split_scratch_{spec.num_heads}x{spec.value_dim}",
                               ops.diff_decode_scratch_floats(most, spec.num_heads, spec.value_dim, MAX_SPLITS))
    ops.diff_attention_decode(q[:rows], records, 0, k_off, cache.block_table, ctx.positions[:rows], ctx.row_slot[:rows],
                              out[:rows], scratch, spec.num_heads, spec.num_kv_heads, spec.head_dim, spec.value_dim,
                              cache.page_size, float(spec.scale), float(spec.get("softcap", 0.0)), lam, out_scale, eps, n_split)


def attend(q: torch.Tensor, cache, ctx, out: torch.Tensor, spec, lam: torch.Tensor, out_scale: float, eps: float,
           runtime) -> bool:
    """Run the tensor-core kernel(s) for this step if they apply; False means the caller runs the plain one."""
    (records,) = cache.arrays
    if not fast_applies(spec, q, records, cache.page_size) or out.stride(0) % 2:
        return False
    k_off = spec.num_kv_heads * 2 * spec.head_dim
    if ctx.decode_only:
        _single(q, records, k_off, cache, ctx, out, spec, lam, out_scale, eps, runtime, q.shape[0])
        return True
    planned = query_tiles(ctx)
    if planned is None:
        return False
    q_tiles, n_tiles, n_prompt_tiles, leading = planned
    if leading > 0:
        _single(q, records, k_off, cache, ctx, out, spec, lam, out_scale, eps, runtime, leading)
        n_tiles = n_prompt_tiles
    if n_tiles > 0:
        ops.diff_attention_prefill(q, records, 0, k_off, cache.block_table, q_tiles, n_tiles, out, spec.num_heads,
                                   spec.num_kv_heads, spec.head_dim, spec.value_dim, cache.page_size, float(spec.scale),
                                   float(spec.get("softcap", 0.0)), lam, out_scale, eps)
    return True


def run_for_test(kind: str, q, records, k_off, table, positions, row_slot, out, heads, groups, dim, vdim, page, scale, cap,
                 lam, out_scale, eps) -> None:
    """One tensor-core kernel on rows given by hand, every row a request position of its own: "flash" runs each row as
    a one-row query tile, "split" the single-token kernel with several parts (and once more with one part)."""
    rows = q.shape[0]
    if kind == "flash":
        tiles = torch.stack([row_slot[:rows], torch.arange(rows, dtype=torch.int32, device=q.device),
                             torch.ones(rows, dtype=torch.int32, device=q.device), positions[:rows]], dim=1).contiguous()
        ops.diff_attention_prefill(q, records, 0, k_off, table, tiles, rows, out, heads, groups, dim, vdim, page, scale, cap, lam,
                                   out_scale, eps)
        return
    for n_split in (1, 3):
        scratch = torch.zeros(max(1, ops.diff_decode_scratch_floats(rows, heads, vdim, n_split)), dtype=torch.float32,
                              device=q.device)
        ops.diff_attention_decode(q, records, 0, k_off, table, positions, row_slot, out, scratch, heads, groups, dim, vdim, page,
                                  scale, cap, lam, out_scale, eps, n_split)
