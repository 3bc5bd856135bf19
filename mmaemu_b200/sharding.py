"""Multi-GPU scaled_mm: the output is cut into a grid of rectangles (row slabs by default; row groups x column groups
with grid=), one per rank of a process group, every rank computes its rectangle with the single-GPU kernel, and every
rank ends up with the whole result.

Why this is exact: an output element depends only on its own row of `input`, its own column of `mat2`, the scales and
the accumulation plan (the reference replays sub-matrices of hardware outputs on the same ground, astding/mmaemu
tests/test_epilogue.py:81-83). The plan, however, is a property of the WHOLE call -- cuBLASLt picks split-K from the
full (M, N, K) -- so the call is validated and its split decision resolved once on the full shape, identically on
every rank, and handed to the per-rank kernels explicitly; a rank never resolves it on its slab. K is never split
across GPUs. Column groups serve the row-poor shapes (a decode step has 16 rows and 8192 columns: there is nothing to
split along M) and halve what a rank reads of `mat2`.

Assembly, two ways:
  "peer"  the kernel's epilogue stores every output element into this rank's copy of the result AND into every other
          rank's copy, through peer-mapped pointers into symmetric memory (plain stores over NVLink while the kernel
          computes; no collective afterwards, only a device-side barrier of the group before the result is read);
  "nccl"  every rank computes into its own slab and one all-gather (NCCL over NVLink, or gloo on CPU ranks) follows
          (with column groups the gathered rectangles are then copied into place).
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


def shard_grid(M: int, N: int, world: int, grid=None) -> tuple:
    """(row groups, column groups) with row groups x column groups == world. None: row slabs only. "auto": the
    factorisation whose largest rectangle is smallest (ties: more row groups), so that row-poor shapes are cut along
    N. A pair is checked and returned."""
    if grid is None:
        return world, 1
    if grid == "auto":
        best = None
        for gm in range(world, 0, -1):
            if world % gm:
                continue
            gn = world // gm
            rows = min(shard_rows(M, gm, 0)[1], M)
            cols = min(shard_rows(N, gn, 0)[1], N)
            if best is None or rows * cols < best[0]:
                best = (rows * cols, gm, gn)
        return best[1], best[2]
    try:
        gm, gn = (int(g) for g in grid)
    except (TypeError, ValueError):
        raise ValueError(f"grid must be None, 'auto' or (row groups, column groups), got {grid!r}") from None
    if gm < 1 or gn < 1 or gm * gn != world:
        raise ValueError(f"grid {grid!r} does not cover the {world} ranks of the group")
    return gm, gn


def _meta_like(t, rows=None, ld=None, cols=None, ld_cols=None):
    """A meta tensor with t's dtype, strides and requires_grad (and `rows` rows of leading dimension `ld`, `cols`
    columns of leading dimension `ld_cols`): what the validation of the full call needs from an operand, without its
    data."""
    if t is None:
        return None
    size, stride = list(t.shape), list(t.stride())
    if rows is not None:
        size[0] = rows
        if ld is not None:
            stride[0] = ld
    if cols is not None:
        size[1] = cols
        if ld_cols is not None:
            stride[1] = ld_cols
    m = torch.empty_strided(size, stride, dtype=t.dtype, device="meta")
    return m.requires_grad_(True) if t.requires_grad else m


def validate_full_call(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, profile, splitk,
                       backend, full_rows=None, full_cols=None):
    """Validate the WHOLE call from metadata only and resolve its split-K decision -- the same answer, or the same
    exception, on every rank, whatever rectangle the rank owns (an empty or one-row slab must not change which checks
    run). `input` may be this rank's row slab and `mat2` its column slab; `full_rows` / `full_cols` are then the row
    count of the whole `input` and the column count of the whole `mat2`. Returns the validated call (shapes, output
    dtype, split decision, early = zero-size result)."""
    from .api import _prepare
    M = input.shape[0] if full_rows is None else int(full_rows)
    K = input.shape[1] if input.dim() == 2 else 0
    ld = input.stride(0) if (input.dim() == 2 and input.shape[0] > 1) else max(K, 1)
    full = _meta_like(input, rows=M, ld=ld) if input.dim() == 2 else _meta_like(input)
    if full_cols is not None and isinstance(mat2, torch.Tensor) and mat2.dim() == 2:
        ldb = mat2.stride(1) if mat2.shape[1] > 1 else max(mat2.shape[0], 1)
        mat2_full = _meta_like(mat2, cols=int(full_cols), ld_cols=ldb)
    else:
        mat2_full = _meta_like(mat2)
    return _prepare(full, mat2_full, _meta_like(scale_a), _meta_like(scale_b), _meta_like(bias),
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


def gather_rows(local, full_rows: int, group=None):
    """The whole row-sharded tensor on every rank: `local` holds this rank's rows [m0, m1) of shard_rows(full_rows, world,
    rank) (for instance the rows of mat2.t() that this rank has just copied from the host); one all-gather over the
    group's backend (NCCL over NVLink on CUDA ranks) assembles all of them. With it a replicated operand crosses the
    host link once per job instead of once per rank. FP8 tensors travel as bytes."""
    import torch.distributed as dist
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    m0, m1 = shard_rows(full_rows, world, rank)
    if local.shape[0] != m1 - m0:
        raise ValueError(f"rank {rank} owns rows [{m0}, {m1}) but was given {local.shape[0]} rows")
    if world == 1:
        return local
    per = shard_rows(full_rows, world, 0)[1]
    cols = tuple(local.shape[1:])
    row_bytes = local.element_size()
    for extent in cols:
        row_bytes *= extent
    pad = torch.zeros((per, row_bytes), dtype=torch.uint8, device=local.device)
    if m1 > m0:
        pad[: m1 - m0] = local.contiguous().view(torch.uint8).view(m1 - m0, row_bytes)
    full = torch.empty((world * per, row_bytes), dtype=torch.uint8, device=local.device)
    dist.all_gather_into_tensor(full.view(-1), pad.view(-1), group=group)
    return full[:full_rows].view(local.dtype).view((full_rows,) + cols)


def sharded_scaled_mm(input, mat2, scale_a, scale_b, bias=None, scale_result=None, out_dtype=None,
                      use_fast_accum=False, *, profile=None, splitk="auto", backend="auto", group=None, gather=True,
                      compute=None, input_is_local=False, full_rows=None, mat2_is_local=False, full_cols=None,
                      grid=None, assemble="auto", keep_symmetric=False):
    """scaled_mm over the ranks of `group` (default: the world).

    grid: None = one row slab per rank; (gm, gn) = gm row groups x gn column groups, rank r owning row group r // gn
    and column group r % gn; "auto" = the factorisation with the smallest rectangles (shard_grid).
    input: the full [M, K] operand on every rank, or -- with input_is_local=True and full_rows=M -- only the rows of
    this rank's row group. mat2: the full [K, N] operand, or -- with mat2_is_local=True and full_cols=N -- only the
    columns of this rank's column group. The scales and every keyword are as in scaled_mm and must be equal on all
    ranks. Returns the full [M, N] result on every rank (gather=True) or this rank's rectangle (gather=False).

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
    if mat2_is_local and full_cols is None:
        raise ValueError("mat2_is_local=True needs full_cols, the column count of the whole operand")
    # 1. the whole call, from metadata: same outcome on every rank
    c = validate_full_call(input, mat2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, profile, splitk,
                           backend, full_rows if input_is_local else None, full_cols if mat2_is_local else None)
    M, N, od = c.M, c.N, c.od
    gm, gn = shard_grid(M, N, world, grid)
    rm, rn = divmod(rank, gn)
    m0, m1 = shard_rows(M, gm, rm)
    n0, n1 = shard_rows(N, gn, rn) if gn > 1 else (0, N)
    local = input if input_is_local else input[m0:m1]
    local2 = mat2 if (mat2_is_local or gn == 1) else mat2[:, n0:n1]
    if local.shape[0] != m1 - m0:
        raise ValueError(f"rank {rank} owns rows [{m0}, {m1}) but was given {local.shape[0]} rows")
    if local2.shape[1] != n1 - n0:
        raise ValueError(f"rank {rank} owns columns [{n0}, {n1}) but was given {local2.shape[1]} columns")
    if c.early or c.unchanged_out:
        full = torch.zeros((M, N), dtype=od, device=input.device)
        return full if gather or world == 1 else full[m0:m1, n0:n1]
    split = 1 if c.decision.S == 1 else (c.decision.S, c.decision.scheme)
    kw = dict(profile=profile, splitk=split, backend=backend)
    custom = compute is not None
    if compute is None:
        from .api import scaled_mm as compute
    empty = m1 == m0 or n1 == n0                             # this rank owns no output: nothing to compute

    def slab():
        if empty:
            return torch.empty((m1 - m0, n1 - n0), dtype=od, device=input.device)
        return compute(local, local2, scale_a, scale_b, bias, scale_result, out_dtype, use_fast_accum, **kw)

    if not gather or world == 1:
        return slab()
    per = shard_rows(M, gm, 0)[1]
    per_n = shard_rows(N, gn, 0)[1] if gn > 1 else N
    # 2. fused assembly: the kernel stores into every rank's copy of the result
    if not custom and assemble != "nccl" and (assemble == "peer" or _peer_mode_available(input.device, group)):
        from .api import scaled_mm_into
        buf, hdl = _symmetric_buffer(gm * per, N, od, input.device, group)
        hdl.barrier(channel=0)                               # nobody still reads the buffer of an earlier call
        if not empty:
            es = buf.element_size()
            peers = [int(hdl.buffer_ptrs[r]) + (m0 * N + n0) * es for r in range(world) if r != rank]
            scaled_mm_into(buf[m0:m1, n0:n1], peers, local, local2, scale_a, scale_b, scale_result, use_fast_accum, **kw)
        hdl.barrier(channel=1)                               # every rank's stores have landed everywhere
        full = buf[:M]
        return full if keep_symmetric else full.clone()
    # 3. all-gather of the rectangles
    y = slab()
    es = y.element_size()
    if gn == 1 and per * world == M:                         # equal row slabs: gather straight into the result
        out = torch.empty((M, N), dtype=od, device=y.device)
        dist.all_gather_into_tensor(out.view(torch.uint8).view(-1), y.contiguous().view(torch.uint8).view(-1),
                                    group=group)
        return out
    buf = torch.zeros((per, per_n * es), dtype=torch.uint8, device=y.device)     # ragged edges: pad the last rectangles
    if not empty:
        buf[: m1 - m0, : (n1 - n0) * es] = y.contiguous().view(torch.uint8).view(m1 - m0, (n1 - n0) * es)
    full = torch.empty((world * per, per_n * es), dtype=torch.uint8, device=y.device)
    dist.all_gather_into_tensor(full.view(-1), buf.view(-1), group=group)
    if gn == 1:
        return full[:M].view(od)
    # [gm, gn, per, per_n] rectangles -> [gm * per, gn * per_n] rows (one copy), then the valid corner
    full = full.view(gm, gn, per, per_n * es).permute(0, 2, 1, 3).reshape(gm * per, gn * per_n * es)
    return full[:M, : N * es].contiguous().view(od)
