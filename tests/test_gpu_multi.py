"""Two ranks, one GPU each, NCCL: sharded products with and without the gather step.
Skipped on a box with fewer than two GPUs (the single-GPU logic is covered elsewhere and the
multi-rank host logic by the gloo tests)."""
import os
import socket
import sys
from pathlib import Path

import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu

REPO = Path(__file__).resolve().parent.parent


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    os.environ.update(RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1",
                      MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    sys.path.insert(0, str(REPO))
    from kuiper_b200 import klas, sharding, synth
    ranks = sharding.init_from_env()
    dev = ranks.device

    # bf16 GEMM: 2 x 1024 rows, B replicated by broadcast from rank 0
    m, n, k = 2048, 768, 512
    ranges = sharding.row_blocks(m, world, align=256)
    lo, hi = ranges[rank]
    a_blk, _ = synth.gemm_bf16(1, m, n, k, row0=lo, rows=hi - lo, b_col_major=True, device=dev)
    b_full = synth.gemm_bf16(1, 8, n, k, rows=8, b_col_major=True, device=dev)[1] if rank == 0 else None
    b_rep = sharding.replicate(b_full, (n, k), torch.bfloat16, ranks)
    local = sharding.gemm_tc_sharded(a_blk, b_rep, ranges, ranks, b_col_major=True)
    full = sharding.gemm_tc_sharded(a_blk, b_rep, ranges, ranks, gather=True, b_col_major=True)
    assert local.shape == (hi - lo, n) and full.shape == (m, n)
    a_all, bt = synth.gemm_bf16(1, m, n, k, b_col_major=True, device=dev)
    want = klas.gemm_tc(a_all, bt, b_col_major=True)          # the whole product on one GPU
    assert torch.equal(full, want)
    assert torch.equal(full[lo:hi], local)

    # u64 GEMM, bit exact after the gather; ragged blocks (3 tiles of 128 over 2 ranks)
    ua, ub = synth.gemm_u64(3, 384, 160, 96, full_range=True, device=dev)
    ur = sharding.row_blocks(384, world, align=128)
    ulo, uhi = ur[rank]
    ufull = sharding.gemm_sharded(ua[ulo:uhi].contiguous(), ub, ur, ranks, gather=True)
    assert torch.equal(ufull, klas.gemm(ua, ub))

    # SpMM by nnz-balanced CSR row ranges (unequal shards), root-only gather
    csr = synth.csr_poisson(4, 3000, 2048, 20.0, device=dev)
    bd = synth.spmm_dense_b(4, 2048, 128, device=dev)
    sr = sharding.csr_row_ranges(csr.row_off, world, "nnz")
    slo, shi = sr[rank]
    shard = csr.row_slice(slo, shi)
    got = sharding.spmm_sharded(shard, bd, sr, ranks, gather=True, root=0)
    if rank == 0:
        assert torch.equal(got, klas.spmm(csr, bd))
    else:
        assert got is None
    torch.cuda.synchronize()
    torch.distributed.barrier()
    (Path(out_dir) / ("ok%d" % rank)).write_text("ok")
    torch.distributed.destroy_process_group()


def test_two_ranks_nccl(tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert (tmp_path / "ok0").exists() and (tmp_path / "ok1").exists()
