"""Multi-GPU scaled_mm: output rows are split across the ranks of a process group, every rank computes its slab with
the single-GPU kernel, and the slabs are assembled with one all-gather.

Why this is exact: an output element depends only on its own row of `input`, its own column of `mat2`, the scales and
the accumulation plan (the reference replays sub-matrices of hardware outputs on the same ground, astding/mmaemu
tests/test_epilogue.py:81-83). The plan, however, is a property of the WHOLE call -- cuBLASLt picks split-K from the
full (M, N, K) -- so the split decision is resolved once on the full shape and handed to every rank explicitly; a rank
never resolves it on its slab. K is never split across GPUs.

The reference has no multi-GPU path (one process, one device); this module is new. One process per GPU,
torch.distributed for the plumbing (NCCL over NVLink on GPUs; gloo works for host-side tests).
"""
from __future__ import annotations

import torch

from .splitk import resolve_splitk

ROW_ALIGN = 128     # slabs start on multiples of the largest CTA tile height


def shard_rows(M: int, world: int, rank: int, align: int = ROW_ALIGN) -> tuple:
    """[m0, m1) of `rank`: contiguous slabs of ceil(ceil(M / align) / world) * align rows; trailing ranks may get
    fewer rows or none."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    tiles = -(-M // align)
    per = -(-tiles // world) * align
    m0 = min(rank * per, M)
    return m0, min(m0 + per, M)


def sharded_scaled_mm(input, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None,
                      use_fast_accum=False, *, profile=None, splitk="auto", backend="auto", group=None, gather=True,
                      compute=None, input_is_local=False, full_rows=None):
    """scaled_mm over the ranks of `group` (default: the world).

    input: the full [M, K] operand on every rank, or -- with input_is_local=True and full_rows=M -- only this rank's
    row slab. mat2, the scales and every keyword are as in scaled_mm and must be equal on all ranks. Returns the full
    [M, N] result on every rank (gather=True: one all-gather of row slabs) or this rank's slab (gather=False).
    `compute` replaces the per-rank scaled_mm (tests run the sharding logic on CPU ranks with a stand-in)."""
    import torch.distributed as dist
    if compute is None:
        from .api import scaled_mm as compute
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    M = int(full_rows) if input_is_local else input.shape[0]
    K, N = input.shape[1], mat2.shape[1]
    od = out_dtype if out_dtype is not None else input.dtype
    split = splitk
    if M and N and K and isinstance(splitk, str) and splitk == "auto":
        d = resolve_splitk(M, N, K, a_dtype=input.dtype, b_dtype=mat2.dtype, out_dtype=od,
                           use_fast_accum=bool(use_fast_accum), profile=profile, splitk="auto",
                           layout_std=input.is_contiguous() and mat2.t().is_contiguous())
        split = 1 if d.S == 1 else (d.S, d.scheme)
    m0, m1 = shard_rows(M, world, rank)
    local = input if input_is_local else input[m0:m1]
    if local.shape[0] != m1 - m0:
        raise ValueError(f"rank {rank} owns rows [{m0}, {m1}) but was given {local.shape[0]} rows")
    y = compute(local, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, profile=profile,
                splitk=split, backend=backend)
    if not gather or world == 1:
        return y
    per = shard_rows(M, world, 0)[1]
    es = y.element_size()
    if per * world == M:                                     # equal slabs: gather straight into the result
        out = torch.empty((M, N), dtype=od, device=y.device)
        dist.all_gather_into_tensor(out.view(torch.uint8).view(-1), y.contiguous().view(torch.uint8).view(-1),
                                    group=group)
        return out
    buf = torch.zeros((per, N * es), dtype=torch.uint8, device=y.device)     # ragged tail: pad the last slabs
    buf[: m1 - m0] = y.contiguous().view(torch.uint8).view(m1 - m0, N * es)
    full = torch.empty((world * per, N * es), dtype=torch.uint8, device=y.device)
    dist.all_gather_into_tensor(full.view(-1), buf.view(-1), group=group)
    return full[:M].view(od)
