"""Multi-GPU layer of the Klas hot path: one process per GPU, shards that need no exchange.

The reference is single-GPU.  Its three products shard without any data-path collective:

* dense GEMM      by contiguous row blocks of A and C (tile-aligned), B replicated;
* batched GEMM    by contiguous ranges of pages;
* CSR x dense     by contiguous CSR row ranges (equal rows, or equal nonzeros), B replicated.

Each rank computes its shard with the single-GPU kernels.  A collective (NCCL all-gather /
gather over NVLink through torch.distributed) runs only when the caller asks for C
assembled, and replicating B is a one-off broadcast outside any timed region.

Everything here is host logic over torch.distributed; it also runs on the gloo backend with
CPU tensors when a `compute` callable is injected (the multi-process CPU tests do that).
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Callable, List, Optional, Sequence, Tuple

import torch
import torch.distributed as dist

Range = Tuple[int, int]


# --------------------------------------------------------------------------- partitioners
def row_blocks(m: int, world: int, align: int = 256) -> List[Range]:
    """Splits rows [0, m) into `world` contiguous blocks whose boundaries are multiples of
    `align` (the tensor-core tile height), as even as that allows.  Blocks may be empty when
    m < world * align.  The blocks cover [0, m) exactly once, in rank order."""
    if m < 0 or world < 1 or align < 1:
        raise ValueError("row_blocks: bad arguments")
    units = -(-m // align)                      # tiles, the last one possibly ragged
    out, start = [], 0
    for r in range(world):
        n_units = units // world + (1 if r < units % world else 0)
        stop = min(m, start + n_units * align)
        out.append((start, stop))
        start = stop
    assert start == m
    return out


def batch_ranges(batch: int, world: int) -> List[Range]:
    """Contiguous page ranges, sizes differing by at most one."""
    return row_blocks(batch, world, align=1)


def csr_row_ranges(row_off: torch.Tensor, world: int, balance: str = "rows") -> List[Range]:
    """Contiguous CSR row ranges.  balance="rows": equal row counts; balance="nnz": boundaries
    chosen by binary search on row_off so that every range holds about nnz / world nonzeros."""
    rows = int(row_off.numel()) - 1
    if balance == "rows":
        return row_blocks(rows, world, align=1)
    if balance != "nnz":
        raise ValueError("balance must be 'rows' or 'nnz'")
    ro = row_off.to(torch.int64).cpu()
    nnz = int(ro[-1])
    cuts = [0]
    for r in range(1, world):
        target = (nnz * r) // world
        cut = int(torch.searchsorted(ro, torch.tensor([target]), right=False)[0])
        cuts.append(min(max(cut, cuts[-1]), rows))
    cuts.append(rows)
    return [(cuts[i], cuts[i + 1]) for i in range(world)]


def check_partition(ranges: Sequence[Range], total: int) -> None:
    """Raises unless `ranges` tile [0, total) in order without gaps or overlap."""
    pos = 0
    for a, b in ranges:
        if a != pos or b < a:
            raise ValueError("ranges do not tile [0, %d): %s" % (total, list(ranges)))
        pos = b
    if pos != total:
        raise ValueError("ranges end at %d, expected %d" % (pos, total))


# --------------------------------------------------------------------------- process group
@dataclass
class Ranks:
    rank: int
    world: int
    local_rank: int
    device: torch.device

    @property
    def is_root(self) -> bool:
        return self.rank == 0


def init_from_env(backend: Optional[str] = None) -> Ranks:
    """Joins the job described by RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT
    (as torchrun sets them).  With WORLD_SIZE == 1 no process group is created."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    use_cuda = torch.cuda.is_available() and backend != "gloo"
    device = torch.device("cuda", local) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        kwargs = {"device_id": device} if use_cuda else {}
        dist.init_process_group(backend or ("nccl" if use_cuda else "gloo"), rank=rank, world_size=world, **kwargs)
    return Ranks(rank, world, local, device)


def replicate(t: Optional[torch.Tensor], shape, dtype, ranks: Ranks, src: int = 0) -> torch.Tensor:
    """Broadcasts `t` (given on rank `src`) so that every rank holds a replica -- how B is
    distributed once, before any timed region."""
    if ranks.rank == src:
        out = t.to(ranks.device).contiguous()
    else:
        out = torch.empty(tuple(shape), dtype=dtype, device=ranks.device)
    if ranks.world > 1:
        dist.broadcast(out, src=src)
    return out


# --------------------------------------------------------------------------- gathering C
def gather_rows(local: torch.Tensor, ranges: Sequence[Range], ranks: Ranks,
                root: Optional[int] = None) -> Optional[torch.Tensor]:
    """Assembles the row-sharded result.  root=None: every rank receives all rows (all-gather);
    root=r: only rank r does.  Equal shards use one all_gather_into_tensor; unequal shards
    (ragged tiles, nnz-balanced CSR ranges) are padded to the longest shard and trimmed."""
    check_partition(ranges, ranges[-1][1])
    if ranks.world == 1:
        return local
    sizes = [b - a for a, b in ranges]
    if local.shape[0] != sizes[ranks.rank]:
        raise ValueError("rank %d holds %d rows, its range has %d" % (ranks.rank, local.shape[0], sizes[ranks.rank]))
    tail = tuple(local.shape[1:])
    longest = max(sizes)
    if longest == 0:
        return local.new_empty((0,) + tail)
    if all(s == longest for s in sizes):
        out = local.new_empty((longest * ranks.world,) + tail)
        dist.all_gather_into_tensor(out, local.contiguous())
    else:
        padded = local.new_zeros((longest,) + tail)
        padded[:local.shape[0]] = local
        buf = local.new_empty((longest * ranks.world,) + tail)
        dist.all_gather_into_tensor(buf, padded)
        out = torch.cat([buf[r * longest:r * longest + s] for r, s in enumerate(sizes)], dim=0)
    if root is not None and ranks.rank != root:
        return None
    return out


# --------------------------------------------------------------------------- sharded products
def _default_gemm_tc(A, B, **kw):
    from . import klas
    return klas.gemm_tc(A, B, **kw)


def _default_gemm(A, B, **kw):
    from . import klas
    return klas.gemm(A, B, **kw)


def _default_spmm(csr, B, **kw):
    from . import klas
    return klas.spmm(csr, B, **kw)


def gemm_tc_sharded(A_rows: torch.Tensor, B: torch.Tensor, ranges: Sequence[Range], ranks: Ranks, *,
                    gather: bool = False, root: Optional[int] = None,
                    compute: Callable = _default_gemm_tc, **kw) -> Optional[torch.Tensor]:
    """Tensor-core GEMM on this rank's row block `A_rows` (= rows ranges[rank] of A) against the
    replicated B.  Returns the local C block, or the assembled C when gather=True."""
    a, b = ranges[ranks.rank]
    if A_rows.shape[-2] != b - a:
        raise ValueError("A block has %d rows, range %s" % (A_rows.shape[-2], (a, b)))
    local = compute(A_rows, B, **kw)
    return gather_rows(local, ranges, ranks, root) if gather else local


def gemm_sharded(A_rows: torch.Tensor, B: torch.Tensor, ranges: Sequence[Range], ranks: Ranks, *,
                 gather: bool = False, root: Optional[int] = None,
                 compute: Callable = _default_gemm, **kw) -> Optional[torch.Tensor]:
    """CUDA-core GEMM (f32 / f64 / u32 / u64) on this rank's row block."""
    a, b = ranges[ranks.rank]
    if A_rows.shape[-2] != b - a:
        raise ValueError("A block has %d rows, range %s" % (A_rows.shape[-2], (a, b)))
    local = compute(A_rows, B, **kw)
    return gather_rows(local, ranges, ranks, root) if gather else local


def batched_gemm_tc_sharded(A_pages: torch.Tensor, B_pages: torch.Tensor, ranges: Sequence[Range],
                            ranks: Ranks, *, gather: bool = False, root: Optional[int] = None,
                            compute: Callable = _default_gemm_tc, **kw) -> Optional[torch.Tensor]:
    """Batched GEMM on this rank's pages (A, B and C pages are co-located; nothing is replicated)."""
    a, b = ranges[ranks.rank]
    if A_pages.shape[0] != b - a or B_pages.shape[0] != b - a:
        raise ValueError("page counts do not match range %s" % ((a, b),))
    local = compute(A_pages, B_pages, **kw)
    return gather_rows(local, ranges, ranks, root) if gather else local


def spmm_sharded(csr_rows, B: torch.Tensor, ranges: Sequence[Range], ranks: Ranks, *,
                 gather: bool = False, root: Optional[int] = None,
                 compute: Callable = _default_spmm, **kw) -> Optional[torch.Tensor]:
    """CSR x dense on this rank's CSR row range (`csr_rows` = Csr.row_slice(*ranges[rank]): offsets
    rebased to 0, its own longest-first order) against the replicated B."""
    a, b = ranges[ranks.rank]
    if csr_rows.rows != b - a:
        raise ValueError("CSR shard has %d rows, range %s" % (csr_rows.rows, (a, b)))
    local = compute(csr_rows, B, **kw)
    return gather_rows(local, ranges, ranks, root) if gather else local
