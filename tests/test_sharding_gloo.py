"""The multi-GPU sharding logic on two and four CPU ranks (gloo): row slabs and row x column grids, split-K decided
on the full shape, all-gather of equal and ragged rectangles. The per-rank compute is a stand-in that calls the CPU oracle, so the assembled result must
equal the oracle on the whole problem bit for bit."""
import os
import socket
import warnings

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from mmaemu_b200.sharding import shard_grid, shard_rows

F8 = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}


def test_shard_rows_cover_every_row_once():
    for M in (0, 1, 127, 128, 129, 1000, 4096, 32768):
        for world in (1, 2, 3, 4, 8):
            spans = [shard_rows(M, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == M
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            assert all(m0 % 128 == 0 or m0 == M for m0, _ in spans)
    with pytest.raises(ValueError):
        shard_rows(10, 2, 2)


def test_shard_grid():
    assert shard_grid(16384, 16384, 8) == (8, 1) and shard_grid(16, 8192, 8) == (8, 1)      # default: row slabs
    assert shard_grid(16384, 16384, 8, "auto") == (8, 1)                                    # ties keep the row slabs
    assert shard_grid(16, 8192, 8, "auto") == (1, 8)                                        # nothing to cut along M
    assert shard_grid(256, 8192, 8, "auto") == (2, 4)
    assert shard_grid(100, 100, 4, (2, 2)) == (2, 2)
    for bad in ((2, 3), (0, 4), "rows", 4):
        with pytest.raises(ValueError):
            shard_grid(100, 100, 4, bad)


def _worker(rank, world, port, M, N, K, profile, out_name, local, q, grid=None, local2=False, splitk="auto"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from mmaemu_b200.sharding import shard_grid, shard_rows, sharded_scaled_mm
    from oracle import oracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(3)
        a = (torch.randn(M, K, generator=g) * 8).to(F8["e5m2"])
        bt = (torch.randn(N, K, generator=g) * 8).to(F8["e4m3"])
        od = getattr(torch, out_name)
        seen = []
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            gm, gn = shard_grid(M, N, world, grid)
            m0, m1 = shard_rows(M, gm, rank // gn)
            n0, n1 = shard_rows(N, gn, rank % gn) if gn > 1 else (0, N)
            extra = dict(input_is_local=True, full_rows=M) if local else {}      # only this rank's rows are passed
            if local2:                                                           # ... and only its columns of mat2
                extra.update(mat2_is_local=True, full_cols=N)
            y = sharded_scaled_mm(a[m0:m1] if local else a, bt[n0:n1].t() if local2 else bt.t(), torch.tensor(0.25),
                                  torch.tensor(3.0), out_dtype=od, use_fast_accum=True, profile=profile,
                                  compute=_oracle_compute(seen), grid=grid, splitk=splitk, **extra)
            from mmaemu_b200.splitk import resolve_splitk
            d = resolve_splitk(M, N, K, a_dtype=a.dtype, b_dtype=bt.dtype, out_dtype=od, use_fast_accum=True,
                               profile=profile, splitk=splitk)
        want = oracle.scaled_mm(a.view(torch.uint8).numpy(), bt.view(torch.uint8).numpy(), 0.25, 3.0, out=out_name,
                                fmt_a="e5m2", fmt_b="e4m3", preset=profile, fast=True, S=d.S, scheme=d.scheme)
        it = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[y.element_size()]
        got = y.contiguous().view(it).numpy().view(want.dtype)
        called = [] if (m1 == m0 or n1 == n0) else [1 if d.S == 1 else (d.S, d.scheme)]   # no rectangle: no compute
        ok = y.shape == (M, N) and np.array_equal(got, want) and seen == called
        q.put((rank, bool(ok), d.S))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _oracle_compute(seen):
    from oracle import oracle

    def compute(a, mat2, sa, sb, bias, sr, out_dtype, fast, *, profile, splitk, backend):
        seen.append(splitk)
        S, scheme = (1, "none") if splitk == 1 else splitk
        name = str(out_dtype).replace("torch.", "")
        bits = oracle.scaled_mm(a.view(torch.uint8).numpy(), mat2.t().contiguous().view(torch.uint8).numpy(),
                                float(sa), float(sb), out=name, fmt_a="e5m2", fmt_b="e4m3", preset=profile, fast=fast,
                                S=S, scheme=scheme, threads=2)
        it = {1: np.uint8, 2: np.int16, 4: np.int32}[bits.itemsize]
        return torch.from_numpy(bits.view(it).copy()).view(out_dtype)
    return compute


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("M,N,K,profile,out,local", [
    (256, 64, 8192, "hopper", "float32", False),        # equal slabs; the H100 table splits K for the full shape
    (192, 64, 2048, "ada", "bfloat16", False),          # ragged: rank 0 owns 128 rows, rank 1 owns 64; S = 3 by the table
    (100, 192, 1024, "hopper", "float8_e5m2", False),   # rank 1 owns nothing
    (256, 64, 8192, "hopper", "bfloat16", True),        # every rank passes only its own slab (input_is_local)
    (192, 64, 2048, "ada", "float32", True),
])
def test_two_ranks_assemble_the_oracle_result(M, N, K, profile, out, local):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, M, N, K, profile, out, local, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(2))
    assert [r[1] for r in results] == [True, True], results


@pytest.mark.parametrize("world,grid,M,N,K,profile,out,local,local2,splitk", [
    (2, (1, 2), 256, 64, 8192, "hopper", "bfloat16", False, False, "auto"),        # columns only; S from the H100 table
    (4, (2, 2), 200, 320, 1024, "ada", "float16", False, False, (3, "pairwise")),  # ragged both ways (128 + 72, 256 + 64)
    (4, (2, 2), 200, 320, 1024, "hopper", "float8_e4m3fn", True, True, 1),         # only own rows and columns are passed
    (4, "auto", 16, 1024, 512, "hopper", "float32", False, True, (2, "contiguous")),   # a decode shape: auto = (1, 4)
    (4, (1, 4), 128, 304, 256, "ada", "bfloat16", False, False, 1),                # the last rank owns no columns
])
def test_a_grid_of_ranks_assembles_the_oracle_result(world, grid, M, N, K, profile, out, local, local2, splitk):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, M, N, K, profile, out, local, q, grid, local2, splitk))
             for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(world))
    assert [r[1] for r in results] == [True] * world, results


def _worker_reject(rank, world, port, case, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import datetime
    import torch.distributed as dist
    import mmaemu_b200 as mm
    from mmaemu_b200.sharding import shard_rows, sharded_scaled_mm
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    try:
        M, N, K = 100, 64, 256                              # rank 1 owns no rows
        g = torch.Generator().manual_seed(5)
        a = (torch.randn(M, K, generator=g) * 4).to(F8["e4m3"])
        bt = (torch.randn(N, K, generator=g) * 4).to(F8["e4m3"])
        sa, sb = torch.tensor(0.5), torch.tensor(2.0)
        kw = dict(out_dtype=torch.bfloat16, profile="ada", compute=_oracle_compute([]))
        want = None
        if case == "bias":
            kw["bias"] = torch.zeros(N, dtype=torch.bfloat16)
            want = mm.UnsupportedFeatureError
        elif case == "rowwise":
            sa, sb = torch.full((M, 1), 0.5), torch.full((1, N), 2.0)
            want = mm.UnsupportedFeatureError
        elif case == "grad":
            sa = sa.clone().requires_grad_(True)
            want = mm.UnsupportedFeatureError
        elif case == "e5m2_out":
            kw["out_dtype"] = torch.float8_e5m2           # e4m3 x e4m3 -> e5m2: the profile rejects it
            want = mm.ReferenceRejectsError
        elif case == "layout":
            bt = bt.t().contiguous().t()                    # mat2 = bt.t() is then row-major: cuBLASLt rejects
            want = mm.ReferenceRejectsError
        m0, m1 = shard_rows(M, world, rank)
        local = case != "bias"                              # both ways of passing the operand
        try:
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                if local:
                    sharded_scaled_mm(a[m0:m1], bt.t(), sa, sb, input_is_local=True, full_rows=M, **kw)
                else:
                    sharded_scaled_mm(a, bt.t(), sa, sb, **kw)
            raised = None
        except Exception as e:  # noqa: BLE001
            raised = type(e)
        q.put((rank, raised is want, str(raised)))
        dist.barrier()                                      # reached by every rank: nobody is stuck in a collective
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("case", ["bias", "rowwise", "grad", "e5m2_out", "layout"])
def test_a_rejected_call_is_rejected_on_every_rank(case):
    """The whole call is validated from metadata before any rank computes, so a rank that owns no rows raises the same
    exception as the others instead of walking into the collective alone."""
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_reject, args=(r, 2, port, case, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    results = sorted(q.get(timeout=5) for _ in range(2))
    assert [r[1] for r in results] == [True, True], results


def _worker_gather(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    import torch.distributed as dist
    from mmaemu_b200.sharding import gather_rows, shard_rows
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = True
        for rows, dtype in ((300, torch.float8_e4m3fn), (100, torch.float8_e5m2), (256, torch.bfloat16)):
            g = torch.Generator().manual_seed(rows)
            full = torch.randn(rows, 48, generator=g).to(dtype)
            m0, m1 = shard_rows(rows, world, rank)                 # 100 rows on two ranks: rank 1 owns nothing
            got = gather_rows(full[m0:m1].clone(), rows)
            ok = ok and got.dtype == dtype and got.shape == full.shape and bool(
                torch.equal(got.view(torch.uint8), full.view(torch.uint8)))
        try:
            gather_rows(full[:1], 256)
            ok = False
        except ValueError:
            pass
        q.put((rank, ok))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_gather_rows_assembles_a_row_sharded_operand():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker_gather, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert sorted(q.get(timeout=5) for _ in range(2)) == [(0, True), (1, True)]
