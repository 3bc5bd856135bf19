"""sharded_scaled_mm on two B200s (-m gpu; skipped on a machine with one GPU): one process per GPU, NCCL for the
plumbing. Both ways of assembling the result are run -- the kernel's epilogue storing into every GPU's copy through
peer pointers ("peer"), and row slabs followed by an all-gather ("nccl") -- and every rank's assembled result must
equal the single-GPU result of the whole call and, on sampled rows of every rank's slab, the oracle. Ragged row counts
(a last slab that is shorter, a rank without rows), column groups (grid 1 x 2, with a rank without columns) and
split-K plans (decided on the whole shape) are covered.
NVLS is switched off for NCCL: these child processes come and go."""
import os
import socket
import warnings

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

import datagen

pytestmark = pytest.mark.gpu
WORLD = 2
CASES = [
    # M, N, K, profile, out, fast, splitk
    (1024, 512, 2048, "hopper", "float16", True, 1),
    (640, 256, 1024, "hopper", "bfloat16", False, 1),                  # ragged: 384 + 256 rows
    (100, 192, 1024, "ada", "float8_e4m3fn", False, 1),                # rank 1 owns no rows
    (256, 128, 8192, "hopper", "float32", True, (4, "contiguous")),    # split-K plan, decided on the whole call
]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _operands(M, N, K, seed):
    rng = np.random.default_rng(seed)
    a = datagen.codes(rng, M, K, "e4m3", "gauss40")
    b = datagen.codes(rng, N, K, "e4m3", "all_codes")
    a[M // 3, 5], a[M - 1, K - 1], b[7, 0] = 0x7F, 0xFF, 0x7F          # NaN codes: rows M/3 and M-1, column 7
    return a, b


def _worker(rank, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import datetime
    import torch.distributed as dist
    import mmaemu_b200 as mm
    from mmaemu_b200.sharding import shard_rows, sharded_scaled_mm
    from oracle import oracle
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=WORLD, device_id=dev, timeout=datetime.timedelta(seconds=120))
    results = []
    try:
        for i, (M, N, K, profile, out, fast, splitk) in enumerate(CASES):
            a, b = _operands(M, N, K, i)
            od = getattr(torch, out)
            ad, bd = torch.from_numpy(a).to(dev).view(torch.float8_e4m3fn), torch.from_numpy(b).to(dev).view(torch.float8_e4m3fn)
            sa, sb = torch.tensor(0.75, device=dev), torch.tensor(1.5, device=dev)
            kw = dict(out_dtype=od, use_fast_accum=fast, profile=profile, splitk=splitk)
            with warnings.catch_warnings():
                warnings.simplefilter("ignore")
                whole = mm.scaled_mm(ad, bd.t(), sa, sb, **kw)                     # the whole call on this GPU
                m0, m1 = shard_rows(M, WORLD, rank)
                for mode in ("peer", "nccl"):
                    for local in (False, True):
                        extra = dict(input_is_local=True, full_rows=M) if local else {}
                        y = sharded_scaled_mm(ad[m0:m1] if local else ad, bd.t(), sa, sb, assemble=mode, **kw, **extra)
                        torch.cuda.synchronize(dev)
                        it = {1: torch.uint8, 2: torch.int16, 4: torch.int32}[y.element_size()]
                        same = y.shape == (M, N) and bool(torch.equal(y.view(it), whole.view(it)))
                        results.append((i, mode, local, same))
                    # column groups (grid 1 x 2): whole operands, then only this rank's columns of mat2
                    n0, n1 = shard_rows(N, WORLD, rank)
                    for local2 in (False, True):
                        extra = dict(mat2_is_local=True, full_cols=N) if local2 else {}
                        y = sharded_scaled_mm(ad, bd[n0:n1].t() if local2 else bd.t(), sa, sb, assemble=mode,
                                              grid=(1, WORLD), **kw, **extra)
                        torch.cuda.synchronize(dev)
                        same = y.shape == (M, N) and bool(torch.equal(y.view(it), whole.view(it)))
                        results.append((i, mode, "columns" + ("-local" if local2 else ""), same))
                    # twice in a row with the same shape: the symmetric buffer is reused, the first result stays intact
                    y1 = sharded_scaled_mm(ad, bd.t(), sa, sb, assemble=mode, **kw)
                    y2 = sharded_scaled_mm(ad, bd.t(), sb, sa, assemble=mode, **kw)
                    torch.cuda.synchronize(dev)
                    results.append((i, mode, "reuse", bool(torch.equal(y1.view(it), whole.view(it)))
                                    and bool(torch.equal(y2.view(it), whole.view(it)))))
            # sampled rows of both slabs against the oracle
            S, scheme = (1, "none") if splitk == 1 else splitk
            rows = np.unique(np.array([0, M // 3, M // 2, M - 1]))
            want = oracle.scaled_mm(a[rows], b, 0.75, 1.5, out=out, preset=profile, fast=fast, S=S, scheme=scheme)
            got = whole[torch.as_tensor(rows, device=dev)].cpu().view(it).numpy().view(want.dtype)
            results.append((i, "oracle", "-", bool(np.array_equal(got, want))))
        q.put((rank, results))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_gpus_assemble_the_whole_result():
    if torch.cuda.device_count() < WORLD:
        pytest.skip(f"needs {WORLD} GPUs, this machine has {torch.cuda.device_count()}")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, q)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(600)
        assert p.exitcode == 0
    for _ in range(WORLD):
        rank, results = q.get(timeout=10)
        bad = [r for r in results if not r[3]]
        assert not bad, f"rank {rank}: {bad}"
        assert len(results) == len(CASES) * 11
