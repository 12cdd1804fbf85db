"""Seeded synthetic workloads for the Klas hot path.

Every value is a pure function of (seed, stream, index) through a counter-based
splitmix64, so any shard of a matrix can be generated on its own rank, on the
CPU or on the GPU, and equals the same slice of the whole matrix.  No
library-defined random stream is involved.

The five workloads generated here stand in for the configurations the
benchmarks are quoted on (uniform f32 GEMM, N(0,1) bf16 GEMM, uniform f16
batched GEMM, u64 GEMM with entries below 2^32, Poisson(64) CSR x dense SpMM).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

_MASK = (1 << 64) - 1
_GOLDEN = 0x9E3779B97F4A7C15
_M1 = 0xBF58476D1CE4E5B9
_M2 = 0x94D049BB133111EB


def _s64(v: int) -> int:
    """Two's-complement view of an unsigned 64-bit constant (torch has no uint64 math)."""
    v &= _MASK
    return v - (1 << 64) if v >= (1 << 63) else v


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    """Logical shift right of int64 lanes."""
    return (z >> s) & ((1 << (64 - s)) - 1)


def splitmix64(seed: int, index: torch.Tensor) -> torch.Tensor:
    """splitmix64 output number `index` (0-based) of the stream started at `seed`;
    int64 tensor holding the unsigned result bit pattern."""
    z = (index + 1) * _s64(_GOLDEN) + _s64(seed)
    z = (z ^ _lsr(z, 30)) * _s64(_M1)
    z = (z ^ _lsr(z, 27)) * _s64(_M2)
    return z ^ _lsr(z, 31)


def splitmix64_scalar(seed: int, index: int) -> int:
    """Pure-Python splitmix64, used by the tests to pin the tensor version."""
    z = (seed + (index + 1) * _GOLDEN) & _MASK
    z = ((z ^ (z >> 30)) * _M1) & _MASK
    z = ((z ^ (z >> 27)) * _M2) & _MASK
    return z ^ (z >> 31)


def _stream_seed(seed: int, stream: int) -> int:
    """Derives an independent stream seed (matrix A, matrix B, ...) from a config seed."""
    return splitmix64_scalar(seed ^ 0x5851F42D4C957F2D, stream)


def _index(start: int, count: int, device) -> torch.Tensor:
    return torch.arange(start, start + count, dtype=torch.int64, device=device)


def unit_uniform(seed: int, stream: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """float64 uniform in [0, 1) from the top 53 bits."""
    z = splitmix64(_stream_seed(seed, stream), _index(start, count, device))
    return _lsr(z, 11).to(torch.float64) * (1.0 / (1 << 53))


def uniform(seed: int, stream: int, start: int, count: int, lo: float, hi: float,
            dtype=torch.float32, device="cpu") -> torch.Tensor:
    """Uniform in [lo, hi), rounded to `dtype` (round-to-nearest-even)."""
    u = unit_uniform(seed, stream, start, count, device)
    return (lo + (hi - lo) * u).to(dtype)


def normal(seed: int, stream: int, start: int, count: int, dtype=torch.bfloat16,
           device="cpu") -> torch.Tensor:
    """N(0,1) by Box-Muller on two uniforms per value, rounded to `dtype`."""
    s = _stream_seed(seed, stream)
    idx = _index(start, count, device)
    z1 = splitmix64(s, 2 * idx)
    z2 = splitmix64(s, 2 * idx + 1)
    u1 = (_lsr(z1, 11).to(torch.float64) + 1.0) * (1.0 / (1 << 53))  # (0, 1]
    u2 = _lsr(z2, 11).to(torch.float64) * (1.0 / (1 << 53))
    n = torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(2.0 * math.pi * u2)
    return n.to(dtype)


def integers_below_2_32(seed: int, stream: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """Uniform integers in [0, 2^32), returned as int64 (bit pattern of the u64 value)."""
    z = splitmix64(_stream_seed(seed, stream), _index(start, count, device))
    return _lsr(z, 32)


def integers_u64(seed: int, stream: int, start: int, count: int, device="cpu") -> torch.Tensor:
    """Full-range 64-bit patterns (as int64): exercises wrap-around."""
    return splitmix64(_stream_seed(seed, stream), _index(start, count, device))


# --------------------------------------------------------------------------- GEMM workloads
def gemm_f32(seed: int, m: int, n: int, k: int, row0: int = 0, rows: int | None = None, device="cpu"):
    """A[rows x k], B[k x n] uniform [-1,1) f32; rows [row0, row0+rows) of the m x k matrix."""
    rows = m - row0 if rows is None else rows
    a = uniform(seed, 0, row0 * k, rows * k, -1.0, 1.0, torch.float32, device).view(rows, k)
    b = uniform(seed, 1, 0, k * n, -1.0, 1.0, torch.float32, device).view(k, n)
    return a, b


def gemm_bf16(seed: int, m: int, n: int, k: int, row0: int = 0, rows: int | None = None,
              b_col_major: bool = True, device="cpu", chunk_rows: int = 2048):
    """A[rows x k] row-major and B (n x k if b_col_major else k x n), N(0,1) rounded to bf16.
    B[kk][nn] is the same value in both storage orders."""
    rows = m - row0 if rows is None else rows
    a = torch.empty((rows, k), dtype=torch.bfloat16, device=device)
    for r in range(0, rows, chunk_rows):
        c = min(chunk_rows, rows - r)
        a[r:r + c] = normal(seed, 0, (row0 + r) * k, c * k, torch.bfloat16, device).view(c, k)
    # logical B[kk][nn] has stream index nn * k + kk (column-major enumeration)
    bt = torch.empty((n, k), dtype=torch.bfloat16, device=device)
    for r in range(0, n, chunk_rows):
        c = min(chunk_rows, n - r)
        bt[r:r + c] = normal(seed, 1, r * k, c * k, torch.bfloat16, device).view(c, k)
    return a, (bt if b_col_major else bt.t().contiguous())


def gemm_f16_batched(seed: int, batch: int, m: int, n: int, k: int, batch0: int = 0,
                     device="cpu"):
    """Pages [batch0, batch0+batch) of A[.][m][k], B[.][k][n], uniform [-0.5,0.5) f16."""
    a = uniform(seed, 0, batch0 * m * k, batch * m * k, -0.5, 0.5, torch.float16, device)
    b = uniform(seed, 1, batch0 * k * n, batch * k * n, -0.5, 0.5, torch.float16, device)
    return a.view(batch, m, k), b.view(batch, k, n)


def gemm_u64(seed: int, m: int, n: int, k: int, row0: int = 0, rows: int | None = None,
             full_range: bool = False, device="cpu"):
    """u64 matrices as int64 bit patterns; entries in [0, 2^32) unless full_range."""
    rows = m - row0 if rows is None else rows
    gen = integers_u64 if full_range else integers_below_2_32
    a = gen(seed, 0, row0 * k, rows * k, device).view(rows, k)
    b = gen(seed, 1, 0, k * n, device).view(k, n)
    return a, b


# --------------------------------------------------------------------------- SpMM workload
@dataclass
class Csr:
    rows: int
    shared: int
    elems: torch.Tensor     # [nnz] f32 (or int32 bit patterns of u32)
    col_ind: torch.Tensor   # [nnz] int32, sorted and distinct inside a row
    row_off: torch.Tensor   # [rows + 1] int32
    row_indices: torch.Tensor  # [rows] int32: rows by decreasing nnz (stable)

    @property
    def nnz(self) -> int:
        return int(self.elems.numel())

    def to(self, device) -> "Csr":
        return Csr(self.rows, self.shared, self.elems.to(device), self.col_ind.to(device),
                   self.row_off.to(device), self.row_indices.to(device))

    def row_slice(self, r0: int, r1: int) -> "Csr":
        """CSR of rows [r0, r1) with offsets rebased to 0 and its own longest-first order."""
        ro = self.row_off[r0:r1 + 1].to(torch.int64)
        lo, hi = int(ro[0]), int(ro[-1])
        off = (ro - lo).to(torch.int32)
        return Csr(r1 - r0, self.shared, self.elems[lo:hi].clone(), self.col_ind[lo:hi].clone(),
                   off, longest_first(off))


def longest_first(row_off: torch.Tensor) -> torch.Tensor:
    """Row order by decreasing nnz, ties by row index (the schedule the reference's
    drivers build on the host, test/spmm_common.c.inc:140-157)."""
    lens = (row_off[1:].to(torch.int64) - row_off[:-1].to(torch.int64))
    return torch.argsort(-lens, stable=True).to(torch.int32)


def _poisson_counts(seed: int, stream: int, row0: int, rows: int, mean: float, cap: int,
                    device) -> torch.Tensor:
    """Poisson(mean) by inversion of the CDF on one uniform per row, clamped to cap."""
    kmax = int(mean + 12 * math.sqrt(max(mean, 1.0)) + 16)
    logp = [-mean + i * math.log(mean) - math.lgamma(i + 1) for i in range(kmax)] if mean > 0 else [0.0]
    cdf = torch.cumsum(torch.tensor([math.exp(v) for v in logp], dtype=torch.float64), 0).to(device)
    u = unit_uniform(seed, stream, row0, rows, device)
    cnt = torch.searchsorted(cdf, u, right=False)
    return torch.clamp(cnt, max=cap).to(torch.int64)


def csr_poisson(seed: int, rows: int, shared: int, mean_nnz: float, row0: int = 0,
                nrows: int | None = None, device="cpu", value_kind: str = "f32") -> Csr:
    """Rows [row0, row0+nrows) of a rows x shared CSR matrix: per-row nnz ~ Poisson(mean_nnz),
    distinct sorted uniform columns, values uniform [-1,1) (f32) or [1, 100) (u32)."""
    nrows = rows - row0 if nrows is None else nrows
    cnt = _poisson_counts(seed, 2, row0, nrows, mean_nnz, shared, device)
    maxc = int(cnt.max()) if nrows > 0 else 0
    ridx = torch.arange(row0, row0 + nrows, dtype=torch.int64, device=device)
    if maxc == 0:
        cols_sorted = torch.zeros((nrows, 0), dtype=torch.int64, device=device)
    elif maxc * 8 >= shared or maxc * maxc * 2 >= shared:
        # rows where repeated draws would collide often: first cnt entries of a per-row random permutation
        keys = splitmix64(_stream_seed(seed, 3),
                          (ridx[:, None] * shared + torch.arange(shared, device=device)[None, :]).reshape(-1))
        perm = torch.argsort(keys.view(nrows, shared), dim=1, stable=True)[:, :maxc]
        j = torch.arange(maxc, device=device)[None, :]
        perm = torch.where(j < cnt[:, None], perm, shared + j)  # padding sorts last
        cols_sorted = torch.sort(perm, dim=1).values
    else:
        # sparse rows: draw with replacement, redraw the (rare) rows that collide
        j = torch.arange(maxc, dtype=torch.int64, device=device)[None, :]
        cols_sorted = torch.empty((nrows, maxc), dtype=torch.int64, device=device)
        todo = torch.arange(nrows, device=device)
        attempt = 0
        while todo.numel() > 0:
            r = ridx[todo]
            ctr = ((r[:, None] * 64 + attempt) * 4096 + j).reshape(-1)
            z = splitmix64(_stream_seed(seed, 3), ctr)
            c = (_lsr(z, 11).to(torch.float64) * (1.0 / (1 << 53)) * shared).to(torch.int64)
            c = torch.clamp(c, max=shared - 1).view(-1, maxc)
            c = torch.where(j < cnt[todo][:, None], c, shared + j)
            c = torch.sort(c, dim=1).values
            dup = ((c[:, 1:] == c[:, :-1]) & (c[:, 1:] < shared)).any(dim=1)
            cols_sorted[todo[~dup]] = c[~dup]
            todo = todo[dup]
            attempt += 1
            if attempt >= 64:
                raise RuntimeError("csr_poisson: could not draw distinct columns")
    valid = cols_sorted < shared
    row_off = torch.zeros(nrows + 1, dtype=torch.int64, device=device)
    row_off[1:] = torch.cumsum(cnt, 0)
    col_ind = cols_sorted[valid].to(torch.int32)
    nnz = int(row_off[-1])
    # value of nonzero number t of global row r: stream index r * 4096 + t
    t = (torch.arange(maxc, dtype=torch.int64, device=device)[None, :]).expand(nrows, maxc)
    vidx = (ridx[:, None] * 4096 + t)[valid]
    z = splitmix64(_stream_seed(seed, 4), vidx)
    u = _lsr(z, 11).to(torch.float64) * (1.0 / (1 << 53))
    if value_kind == "f32":
        elems = (-1.0 + 2.0 * u).to(torch.float32)
    else:
        elems = (1 + (u * 99).to(torch.int64)).to(torch.int32)
    assert elems.numel() == nnz
    row_off32 = row_off.to(torch.int32)
    return Csr(nrows, shared, elems, col_ind, row_off32, longest_first(row_off32))


def power_law_counts(rows: int, shared: int, mean_nnz: float, alpha: float = 0.8, device="cpu") -> torch.Tensor:
    """Row lengths proportional to 1 / rank^alpha, scaled to the given mean and capped at `shared`:
    a few very long rows and a long tail of short ones (the shape of the reference's non-uniform
    SpMM bench, bench/sputnik-bench/spmm_bench.cu:136-154, with row i of rank i + 1)."""
    w = torch.arange(1, rows + 1, dtype=torch.float64, device=device) ** (-alpha)
    cnt = torch.floor(w * (mean_nnz * rows / float(w.sum()))).to(torch.int64)
    return torch.clamp(cnt, min=0, max=shared)


def csr_from_counts(seed: int, cnt: torch.Tensor, shared: int, device="cpu", value_kind: str = "f32",
                    dense_from: int = 1024) -> Csr:
    """CSR matrix with the given number of nonzeros per row: distinct sorted columns, uniform over
    [0, shared), values uniform [-1,1) (f32) or [1, 100) (u32).  Short rows (up to `dense_from`
    nonzeros and few enough that repeated draws rarely collide) are drawn together, with redraws on
    collisions; each other row takes the `cnt` smallest of `shared` hashed keys, one row at a time."""
    cnt = cnt.to(torch.int64).to(device)
    nrows = int(cnt.numel())
    if int(cnt.max()) > shared:
        raise ValueError("a row cannot have more distinct columns than the matrix")
    row_off = torch.zeros(nrows + 1, dtype=torch.int64, device=device)
    row_off[1:] = torch.cumsum(cnt, 0)
    nnz = int(row_off[-1])
    col_ind = torch.empty(nnz, dtype=torch.int32, device=device)
    is_short = (cnt <= dense_from) & (cnt * cnt <= shared)   # few collisions expected per draw
    short = torch.nonzero(is_short).flatten()
    maxc = int(cnt[short].max()) if short.numel() else 0
    if maxc > 0:
        j = torch.arange(maxc, dtype=torch.int64, device=device)[None, :]
        todo = short
        attempt = 0
        while todo.numel() > 0:
            ctr = ((todo[:, None] * 64 + attempt) * 4096 + j).reshape(-1)
            z = splitmix64(_stream_seed(seed, 3), ctr)
            c = (_lsr(z, 11).to(torch.float64) * (1.0 / (1 << 53)) * shared).to(torch.int64)
            c = torch.clamp(c, max=shared - 1).view(-1, maxc)
            c = torch.where(j < cnt[todo][:, None], c, shared + j)
            c = torch.sort(c, dim=1).values
            dup = ((c[:, 1:] == c[:, :-1]) & (c[:, 1:] < shared)).any(dim=1)
            good = todo[~dup]
            cg = c[~dup]
            valid = cg < shared
            dest = (row_off[good][:, None] + j)[valid]
            col_ind[dest] = cg[valid].to(torch.int32)
            todo = todo[dup]
            attempt += 1
            if attempt >= 256:
                raise RuntimeError("csr_from_counts: could not draw distinct columns")
    allc = torch.arange(shared, dtype=torch.int64, device=device)
    for r in torch.nonzero(~is_short).flatten().tolist():
        keys = splitmix64(_stream_seed(seed, 3), r * shared + allc)
        pick = torch.argsort(keys, stable=True)[:int(cnt[r])]
        lo = int(row_off[r])
        col_ind[lo:lo + int(cnt[r])] = torch.sort(pick).values.to(torch.int32)
    z = splitmix64(_stream_seed(seed, 4), torch.arange(nnz, dtype=torch.int64, device=device))
    u = _lsr(z, 11).to(torch.float64) * (1.0 / (1 << 53))
    if value_kind == "f32":
        elems = (-1.0 + 2.0 * u).to(torch.float32)
    else:
        elems = (1 + (u * 99).to(torch.int64)).to(torch.int32)
    row_off32 = row_off.to(torch.int32)
    return Csr(nrows, shared, elems, col_ind, row_off32, longest_first(row_off32))


def spmm_dense_b(seed: int, shared: int, cols: int, device="cpu", value_kind: str = "f32"):
    """Dense right-hand side, uniform [-1,1) f32 (or u32 in [0, 100) as int32)."""
    if value_kind == "f32":
        return uniform(seed, 5, 0, shared * cols, -1.0, 1.0, torch.float32, device).view(shared, cols)
    u = unit_uniform(seed, 5, 0, shared * cols, device)
    return (u * 100).to(torch.int32).view(shared, cols)
