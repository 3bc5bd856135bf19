"""Multi-GPU scaled_mm: output rows are split across the ranks of a process group, every rank computes its slab with
the single-GPU kernel, and every rank ends up with the whole result.

Why this is exact: an output element depends only on its own row of `input`, its own column of `mat2`, the scales and
the accumulation plan (the reference replays sub-matrices of hardware outputs on the same ground, astding/mmaemu
tests/test_epilogue.py:81-83). The plan, however, is a property of the WHOLE call -- cuBLASLt picks split-K from the
full (M, N, K) -- so the call is validated and its split decision resolved once on the full shape, identically on
every rank, and handed to the per-rank kernels explicitly; a rank never resolves it on its slab. K is never split
across GPUs.

Assembly, two ways:
  "peer"  the kernel's epilogue stores every output element into this rank's copy of the result AND into every other
          rank's copy, through peer-mapped pointers into symmetric memory (plain stores over NVLink while the kernel
          computes; no collective afterwards, only a device-side barrier of the group before the result is read);
  "nccl"  every rank computes into its own slab and one all-gather (NCCL over NVLink, or gloo on CPU ranks) follows.
"auto" uses "peer" on CUDA devices when symmetric memory can be set up for the group and falls back to "nccl" with a
warning otherwise.

The reference has no multi-GPU path (one process, one device; docs/limitations.md:100); this module is new. One
process per GPU, torch.distributed for the plumbing.
"""
from __future__ import annotations

import warnings

import torch

ROW_ALIGN = 128     # slabs start on multiples of the CTA tile height
_symm_cache: dict = {}
_symm_failed: dict = {}


def shard_rows(M: int, world: int, rank: int, align: int = ROW_ALIGN) -> tuple:
    """[m0, m1) of `rank`: contiguous slabs of ceil(ceil(M / align) / world) * align rows; trailing ranks may get
    fewer rows or none."""
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} of {world}")
    tiles = -(-M // align)
    per = -(-tiles // world) * align
    m0 = min(rank * per, M)
    return m0, min(m0 + per, M)


def _meta_like(t, rows=None, ld=None):
    """A meta tensor with t's dtype, strides and requires_grad (and `rows` rows of leading dimension `ld`): what the
    validation of the full call needs from an operand, without its data."""
    if t is None:
        return None
    size, stride = list(t.shape), list(t.stride())
    if rows is not None:
        size[0] = rows
        if ld is not None:
            stride[0] = ld
    m = torch.empty_strided(size, stride, dtype=t.dtype, device="meta")
    return m.requires_grad_(True) if t.requires_grad else m


def validate_full_call(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, profile, splitk,
                       backend, full_rows=None):
    """Validate the WHOLE call from metadata only and resolve its split-K decision -- the same answer, or the same
    exception, on every rank, whatever rows the rank owns (an empty or one-row slab must not change which checks run).
    `input` may be this rank's slab; `full_rows` is then the row count of the whole operand. Returns the validated call
    (shapes, output dtype, split decision, early = zero-size result)."""
    from .api import _prepare
    M = input.shape[0] if full_rows is None else int(full_rows)
    K = input.shape[1] if input.dim() == 2 else 0
    ld = input.stride(0) if (input.dim() == 2 and input.shape[0] > 1) else max(K, 1)
    full = _meta_like(input, rows=M, ld=ld) if input.dim() == 2 else _meta_like(input)
    return _prepare(full, _meta_like(mat2), _meta_like(scale_a), _meta_like(scale_b), _meta_like(bias),
                    _meta_like(scale_result), out_dtype, use_fast_accum, None, profile, splitk, backend, dry=True)


def _symmetric_buffer(rows, N, dtype, device, group):
    """(buffer [rows, N], handle) in symmetric memory, set up once per (group, shape, dtype) -- a collective call."""
    import torch.distributed as dist
    import torch.distributed._symmetric_memory as symm
    g = group if group is not None else dist.group.WORLD
    key = (id(g), rows, N, dtype, str(device))
    hit = _symm_cache.get(key)
    if hit is None:
        buf = symm.empty((rows, N), dtype=dtype, device=device)
        hdl = symm.rendezvous(buf, group=g)
        hit = _symm_cache[key] = (buf, hdl)
    return hit


def _peer_mode_available(device, group) -> bool:
    """Whether the fused assembly can be used on this group: CUDA ranks and a working symmetric-memory rendezvous
    (probed once per group with a small buffer; all ranks take the same decision through an all-reduce)."""
    import torch.distributed as dist
    if device.type != "cuda":
        return False
    g = group if group is not None else dist.group.WORLD
    if id(g) in _symm_failed:
        return not _symm_failed[id(g)]
    ok = 1
    try:
        _symmetric_buffer(ROW_ALIGN, 16, torch.uint8, device, group)
    except Exception as e:  # noqa: BLE001 - any failure of the set-up means "use the collective"
        ok = 0
        why = f"{type(e).__name__}: {e}"
    flag = torch.tensor([ok], dtype=torch.int32, device=device)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    good = bool(int(flag.item()))
    _symm_failed[id(g)] = not good
    if not good:
        warnings.warn("symmetric memory is not available for this process group"
                      + (f" ({why})" if not ok else " (another rank could not set it up)")
                      + "; the output is assembled with an all-gather instead", RuntimeWarning, stacklevel=3)
    return good


def sharded_scaled_mm(input, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None,
                      use_fast_accum=False, *, profile=None, splitk="auto", backend="auto", group=None, gather=True,
                      compute=None, input_is_local=False, full_rows=None, assemble="auto", keep_symmetric=False):
    """scaled_mm over the ranks of `group` (default: the world).

    input: the full [M, K] operand on every rank, or -- with input_is_local=True and full_rows=M -- only this rank's
    row slab. mat2, the scales and every keyword are as in scaled_mm and must be equal on all ranks. Returns the full
    [M, N] result on every rank (gather=True) or this rank's slab (gather=False).

    assemble: "peer" | "nccl" | "auto" (module docstring). With "peer" the result is produced in a symmetric-memory
    buffer that later calls of the same shape reuse; it is returned as a copy unless keep_symmetric=True (then the
    returned tensor is only valid until the next call with this shape and group).
    `compute` replaces the per-rank scaled_mm (tests run the sharding logic on CPU ranks with a stand-in); it implies
    the all-gather assembly."""
    import torch.distributed as dist
    if assemble not in ("auto", "peer", "nccl"):
        raise ValueError(f"assemble must be 'auto', 'peer' or 'nccl', got {assemble!r}")
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    if input_is_local and full_rows is None:
        raise ValueError("input_is_local=True needs full_rows, the row count of the whole operand")
    # 1. the whole call, from metadata: same outcome on every rank
    c = validate_full_call(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, profile, splitk,
                           backend, full_rows if input_is_local else None)
    M, N, od = c.M, c.N, c.od
    m0, m1 = shard_rows(M, world, rank)
    local = input if input_is_local else input[m0:m1]
    if local.shape[0] != m1 - m0:
        raise ValueError(f"rank {rank} owns rows [{m0}, {m1}) but was given {local.shape[0]} rows")
    if c.early or c.unchanged_out:
        full = torch.zeros((M, N), dtype=od, device=input.device)
        return full if gather or world == 1 else full[m0:m1]
    split = 1 if c.decision.S == 1 else (c.decision.S, c.decision.scheme)
    kw = dict(profile=profile, splitk=split, backend=backend)
    custom = compute is not None
    if compute is None:
        from .api import scaled_mm as compute

    def slab():
        if m1 == m0:                                         # this rank owns no rows: nothing to compute
            return torch.empty((0, N), dtype=od, device=input.device)
        return compute(local, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, **kw)

    if not gather or world == 1:
        return slab()
    per = shard_rows(M, world, 0)[1]
    # 2. fused assembly: the kernel stores into every rank's copy of the result
    if not custom and assemble != "nccl" and (assemble == "peer" or _peer_mode_available(input.device, group)):
        from .api import scaled_mm_into
        buf, hdl = _symmetric_buffer(world * per, N, od, input.device, group)
        hdl.barrier(channel=0)                               # nobody still reads the buffer of an earlier call
        if m1 > m0:
            es = buf.element_size()
            peers = [int(hdl.buffer_ptrs[r]) + m0 * N * es for r in range(world) if r != rank]
            scaled_mm_into(buf[m0:m1], peers, local, mat2, scale_a, scale_b, scale_result, use_fast_accum, **kw)
        hdl.barrier(channel=1)                               # every rank's stores have landed everywhere
        full = buf[:M]
        return full if keep_symmetric else full.clone()
    # 3. all-gather of row slabs
    y = slab()
    es = y.element_size()
    if per * world == M:                                     # equal slabs: gather straight into the result
        out = torch.empty((M, N), dtype=od, device=y.device)
        dist.all_gather_into_tensor(out.view(torch.uint8).view(-1), y.contiguous().view(torch.uint8).view(-1),
                                    group=group)
        return out
    buf = torch.zeros((per, N * es), dtype=torch.uint8, device=y.device)     # ragged tail: pad the last slabs
    if m1 > m0:
        buf[: m1 - m0] = y.contiguous().view(torch.uint8).view(m1 - m0, N * es)
    full = torch.empty((world * per, N * es), dtype=torch.uint8, device=y.device)
    dist.all_gather_into_tensor(full.view(-1), buf.view(-1), group=group)
    return full[:M].view(od)
