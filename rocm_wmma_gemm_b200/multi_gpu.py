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
    def run(self, C_slab, A, B_slab, stream=None) -> None:
        if self.n_count == 0:
            return
        if self._gemm is not None:
            self._gemm(C_slab, A, B_slab, self.M, self.n_count, self.K, self.layout_c, self.layout_a, self.layout_b)
            return
        if self._loader is None:
            self._loader = _loader()
        self._loader.gemm(C_slab, A, B_slab, self.M, self.n_count, self.K, self.layout_c, self.layout_a,
                          self.layout_b, stream=stream)

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
