"""Host logic of the multi-GPU layer: partitioner properties, and a world_size-2 gloo run in
which CPU "ranks" compute their shards with the oracle and the assembled result equals the
oracle on the whole problem."""
import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from kuiper_b200 import sharding, synth

REPO = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("m,world,align", [(65536, 8, 256), (8192, 2, 256), (1000, 4, 128), (100, 8, 256), (0, 3, 64),
                                            (4096, 3, 256), (64, 1, 256)])
def test_row_blocks_cover_disjoint_aligned(m, world, align):
    r = sharding.row_blocks(m, world, align)
    assert len(r) == world
    sharding.check_partition(r, m)
    for a, b in r:
        if b > a:
            assert a % align == 0 and (b % align == 0 or b == m)
    sizes = [b - a for a, b in r]
    assert max(sizes) - min(sizes) <= align or m < world * align
    if m == 65536 and world == 8:
        assert sizes == [8192] * 8


def test_batch_ranges():
    assert sharding.batch_ranges(64, 8) == [(8 * i, 8 * i + 8) for i in range(8)]
    assert [b - a for a, b in sharding.batch_ranges(10, 4)] == [3, 3, 2, 2]


def test_csr_ranges_balance():
    csr = synth.csr_poisson(4, 4096, 8192, 16.0)
    # make the matrix lopsided: rows 0..511 carry many more nonzeros
    heavy = synth.csr_poisson(5, 512, 8192, 200.0)
    ro = torch.cat([heavy.row_off.long(), heavy.row_off.long()[-1] + csr.row_off.long()[1:]])
    by_rows = sharding.csr_row_ranges(ro, 4, "rows")
    by_nnz = sharding.csr_row_ranges(ro, 4, "nnz")
    for r in (by_rows, by_nnz):
        sharding.check_partition(r, ro.numel() - 1)
    nnz = lambda rs: [int(ro[b] - ro[a]) for a, b in rs]
    assert max(nnz(by_nnz)) - min(nnz(by_nnz)) <= 2 * 200 + 64
    assert max(nnz(by_rows)) > 2 * max(nnz(by_nnz)) - min(nnz(by_nnz))
    with pytest.raises(ValueError):
        sharding.check_partition([(0, 3), (4, 8)], 8)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank),
                      MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    for p in (REPO, REPO / "oracle", REPO / "tests"):
        sys.path.insert(0, str(p))
    from oracle_api import Oracle, bf16_bits
    orc = Oracle()
    ranks = sharding.init_from_env(backend="gloo")
    assert ranks.world == world and ranks.device.type == "cpu"

    # ---- bf16 GEMM, ragged row blocks (M = 3 tiles of 64 over 2 ranks), B replicated from rank 0
    m, n, k = 160, 48, 96
    ranges = sharding.row_blocks(m, world, align=64)
    a_full, b_full = synth.gemm_bf16(1, m, n, k, b_col_major=False)
    lo, hi = ranges[rank]
    a_blk, _ = synth.gemm_bf16(1, m, n, k, row0=lo, rows=hi - lo, b_col_major=False)   # generated on its own rank
    assert torch.equal(a_blk, a_full[lo:hi])
    b_rep = sharding.replicate(b_full if rank == 0 else None, (k, n), torch.bfloat16, ranks)
    assert torch.equal(b_rep, b_full)

    def cpu_gemm_tc(A, B, **kw):
        return torch.tensor(orc.gemm(bf16_bits(A), bf16_bits(B), kind="bf16"))

    local = sharding.gemm_tc_sharded(a_blk, b_rep, ranges, ranks, compute=cpu_gemm_tc)
    assert local.shape == (hi - lo, n)
    full = sharding.gemm_tc_sharded(a_blk, b_rep, ranges, ranks, gather=True, compute=cpu_gemm_tc)
    want = torch.tensor(orc.gemm(bf16_bits(a_full), bf16_bits(b_full), kind="bf16"))
    assert torch.equal(full, want)
    only_root = sharding.gemm_tc_sharded(a_blk, b_rep, ranges, ranks, gather=True, root=1, compute=cpu_gemm_tc)
    assert (only_root is None) == (rank != 1)

    # ---- u64 GEMM, equal row blocks: bit exact after the gather
    ua, ub = synth.gemm_u64(3, 64, 24, 40, full_range=True)
    ur = sharding.row_blocks(64, world, align=32)
    ulo, uhi = ur[rank]

    def cpu_u64(A, B, **kw):
        return torch.tensor(orc.gemm_int(A.numpy().view(np.uint64), B.numpy().view(np.uint64)).view(np.int64))

    ufull = sharding.gemm_sharded(ua[ulo:uhi].contiguous(), ub, ur, ranks, gather=True, compute=cpu_u64)
    assert torch.equal(ufull, cpu_u64(ua, ub))

    # ---- batched pages
    pa, pb = synth.gemm_f16_batched(2, 5, 16, 16, 16)
    pr = sharding.batch_ranges(5, world)
    plo, phi = pr[rank]

    def cpu_batched(A, B, **kw):
        return torch.stack([torch.tensor(orc.acc(bf16_bits(A[i]), bf16_bits(B[i]), kind="f16")) for i in range(A.shape[0])]) \
            if A.shape[0] else torch.empty((0, 16, 16), dtype=torch.float64)

    pfull = sharding.batched_gemm_tc_sharded(pa[plo:phi], pb[plo:phi], pr, ranks, gather=True, compute=cpu_batched)
    assert torch.equal(pfull, cpu_batched(pa, pb))

    # ---- SpMM by nnz-balanced CSR row ranges (unequal shards)
    csr = synth.csr_poisson(4, 96, 128, 9.0)
    bd = synth.spmm_dense_b(4, 128, 20)
    sr = sharding.csr_row_ranges(csr.row_off, world, "nnz")
    slo, shi = sr[rank]
    shard = synth.csr_poisson(4, 96, 128, 9.0, row0=slo, nrows=shi - slo)   # generated on its own rank
    sl = csr.row_slice(slo, shi)
    assert torch.equal(shard.col_ind, sl.col_ind) and torch.equal(shard.row_off, sl.row_off)

    def cpu_spmm(c, B, **kw):
        return torch.tensor(orc.spmm_f32(c.rows, B.shape[1], c.elems.numpy(), c.col_ind.numpy().view(np.uint32),
                                         c.row_off.numpy().view(np.uint32), B.numpy()))

    sfull = sharding.spmm_sharded(shard, bd, sr, ranks, gather=True, compute=cpu_spmm)
    assert torch.equal(sfull, cpu_spmm(csr, bd))

    # ---- a rank that holds the wrong number of rows is reported on that rank
    try:
        sharding.gather_rows(torch.zeros((hi - lo + 1, n)), ranges, ranks)
        raised = False
    except ValueError:
        raised = True
    assert raised
    torch.distributed.barrier()
    (Path(out_dir) / ("ok%d" % rank)).write_text("ok")
    torch.distributed.destroy_process_group()


def test_two_ranks_on_gloo(tmp_path, oracle):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert all((tmp_path / ("ok%d" % r)).exists() for r in range(world))


# --------------------------------------------------------------------------- the C partitioners
def test_c_partitioners_match_the_python_ones():
    """klas_b200_mg_row_blocks / klas_b200_mg_csr_row_ranges (host-only functions of the C ABI)
    against sharding.row_blocks / csr_row_ranges: cover, disjoint, tile-aligned, nnz-balanced."""
    import ctypes as C
    from kuiper_b200 import _lib
    lib = _lib.load()
    for m, world, align in [(8192, 8, 256), (65536, 8, 512), (1000, 3, 128), (5, 4, 1), (0, 2, 16), (700, 4, 256)]:
        out = (C.c_uint64 * (world + 1))()
        assert lib.klas_b200_mg_row_blocks(m, world, align, out) == 0
        want = sharding.row_blocks(m, world, align)
        assert [(out[i], out[i + 1]) for i in range(world)] == want
        assert all(out[i] % align == 0 for i in range(1, world) if out[i] < m)
    g = torch.Generator().manual_seed(5)
    lens = torch.randint(0, 50, (997,), generator=g)
    lens[100] = 5000                       # one heavy row
    row_off = torch.zeros(998, dtype=torch.int64)
    row_off[1:] = torch.cumsum(lens, 0)
    ro32 = row_off.to(torch.int32).numpy().astype("uint32")
    for world in (1, 2, 3, 8):
        for balance in ("rows", "nnz"):
            out = (C.c_uint32 * (world + 1))()
            assert lib.klas_b200_mg_csr_row_ranges(ro32.ctypes.data, 997, world, int(balance == "nnz"), out) == 0
            got = [(out[i], out[i + 1]) for i in range(world)]
            sharding.check_partition(got, 997)
            if balance == "nnz":
                assert got == sharding.csr_row_ranges(row_off, world, "nnz")
    assert lib.klas_b200_mg_row_blocks(10, 0, 1, None) == _lib.ERR_INVALID
