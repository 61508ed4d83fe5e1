"""Column-slab GEMM over the GPUs of one box: C = A * B with A replicated, rank r owning
columns slab(r) of B and C.  One process per GPU (`torch.distributed`, NCCL over NVLink);
the compute step has no collective — every rank runs the ordinary single-GPU GEMM on its slab
— and the only exchange is the optional all-gather of the C slabs.

The reference (adelj88/rocm_wmma_gemm) is single-GPU; this driver has no counterpart there.
No kernel reads a peer's memory and no TMA load uses cluster multicast.

Slab storage (what each rank holds):
  A       the whole M x K matrix, in layout_a                      (replicated)
  B slab  K x n_count, dense, in layout_b  (for column-major B this is the contiguous block of
          columns [n_begin, n_begin + n_count) of the full matrix)
  C slab  M x n_count, dense, in layout_c
`gather()` returns the full M x N matrix in layout_c on every rank: column-major slabs simply
concatenate; row-major slabs are interleaved row by row after the all-gather.
"""
from __future__ import annotations

from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import loader as _loader
from . import slab as _slab


def _interleave_row_major(gathered: torch.Tensor, M: int, widths) -> torch.Tensor:
    """[rank][M][width_r] (concatenated, each slab dense row-major) -> [M][sum(width)]."""
    parts, off = [], 0
    for w in widths:
        parts.append(gathered[off: off + M * w].view(M, w))
        off += M * w
    return torch.cat(parts, dim=1).contiguous().view(-1)


class ColumnSlabGemm:
    """Plans and runs one rank's share of C = A * B.

    gemm_fn(C_slab, A, B_slab, M, n_count, K, layout_c, layout_a, layout_b) runs the local GEMM;
    the default is the library's loader (a B200 is required — there is no CPU path).  Tests on
    CPU ranks pass their own checker here.
    """

    def __init__(self, M: int, N: int, K: int, layout_c: int = 0, layout_a: int = 0, layout_b: int = 1,
                 group=None, align: int = 256, gemm_fn: Optional[Callable] = None,
                 rank: Optional[int] = None, world: Optional[int] = None):
        self.M, self.N, self.K = M, N, K
        self.layout_c, self.layout_a, self.layout_b = int(layout_c), int(layout_a), int(layout_b)
        self.group = group
        if world is None:
            world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        self.rank, self.world = rank, world
        self.slabs = [_slab(N, world, r, align) for r in range(world)]
        self.n_begin, self.n_count = self.slabs[rank]
        self._gemm = gemm_fn
        self._loader = None

    # -- compute: no collective ------------------------------------------------------------------
    def _local(self, C, A, B, rows, stream=None) -> None:
        """The local GEMM on `rows` rows of A and of the C slab."""
        if self._gemm is not None:
            self._gemm(C, A, B, rows, self.n_count, self.K, self.layout_c, self.layout_a, self.layout_b)
            return
        if self._loader is None:
            self._loader = _loader()
        self._loader.gemm(C, A, B, rows, self.n_count, self.K, self.layout_c, self.layout_a, self.layout_b,
                          stream=stream)

    def run(self, C_slab, A, B_slab, stream=None) -> None:
        if self.n_count == 0:
            return
        self._local(C_slab, A, B_slab, self.M, stream)

    # -- compute overlapped with the exchange ----------------------------------------------------
    def run_and_gather(self, C_slab: torch.Tensor, A: torch.Tensor, B_slab: torch.Tensor, panels: int = 4) -> torch.Tensor:
        """run() + gather() with the all-gather of row panel p in flight while panel p + 1 is
        being computed (the GEMM of a panel and the collective of the previous one run on
        different streams).  Needs row-major A and C (row panels are then contiguous) and equal
        slabs; anything else takes the plain run() then gather() route.  Returns the full C."""
        widths = [c for _, c in self.slabs]
        even = len(set(widths)) == 1 and widths[0] * self.world == self.N
        if self.world == 1 or self.layout_a != 0 or self.layout_c != 0 or not even or panels < 2:
            self.run(C_slab, A, B_slab)
            return self.gather(C_slab)
        M, K, nl, G = self.M, self.K, self.n_count, self.world
        step = -(-M // panels)
        step = -(-step // 256) * 256
        on_gpu = C_slab.is_cuda
        if on_gpu and getattr(self, "_comm", None) is None:
            self._comm = torch.cuda.Stream()
        Cf, Af = C_slab.reshape(-1), A.reshape(-1)
        full = torch.empty(M * self.N, dtype=Cf.dtype, device=Cf.device)
        pending = []
        for r0 in range(0, M, step):
            r1 = min(M, r0 + step)
            Cp = Cf[r0 * nl: r1 * nl]
            self._local(Cp, Af[r0 * K: r1 * K], B_slab, r1 - r0)
            stage = torch.empty(G * (r1 - r0) * nl, dtype=Cf.dtype, device=Cf.device)
            if on_gpu:
                done = torch.cuda.Event()
                done.record()
                with torch.cuda.stream(self._comm):
                    self._comm.wait_event(done)
                    work = dist.all_gather_into_tensor(stage.view(torch.uint8), Cp.view(torch.uint8), group=self.group,
                                                       async_op=True)
            else:
                work = dist.all_gather_into_tensor(stage.view(torch.uint8), Cp.view(torch.uint8), group=self.group,
                                                   async_op=True)
            pending.append((work, stage, r0, r1))
        rows = full.view(M, G, nl)
        for work, stage, r0, r1 in pending:
            work.wait()
            # [rank][row][col] -> rows r0..r1 of the full matrix, slab by slab
            rows[r0:r1].copy_(stage.view(G, r1 - r0, nl).permute(1, 0, 2))
        return full

    # -- optional exchange -----------------------------------------------------------------------
    def gather(self, C_slab: torch.Tensor) -> torch.Tensor:
        """All-gather of the C slabs; returns the full C (flat, layout_c) on every rank."""
        M = self.M
        widths = [c for _, c in self.slabs]
        if self.world == 1:
            return C_slab.reshape(-1)[: M * self.N]
        wmax = max(widths)
        flat = C_slab.reshape(-1)
        if self.n_count < wmax:  # ragged last slabs: pad to a common size for the collective
            pad = torch.zeros(M * wmax, dtype=flat.dtype, device=flat.device)
            pad[: M * self.n_count] = flat[: M * self.n_count]
            flat = pad
        else:
            flat = flat[: M * wmax].contiguous()
        out = torch.empty(self.world * M * wmax, dtype=flat.dtype, device=flat.device)
        # the collective moves bytes: independent of which element types a backend knows
        dist.all_gather_into_tensor(out.view(torch.uint8), flat.view(torch.uint8), group=self.group)
        pieces = [out[r * M * wmax: r * M * wmax + M * widths[r]] for r in range(self.world)]
        packed = torch.cat(pieces)
        if self.layout_c == 1:
            return packed  # column-major: slab r is columns slab(r), already in place
        return _interleave_row_major(packed, M, widths)
