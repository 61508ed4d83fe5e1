"""Column-slab GEMM over the GPUs of one box: C = A * B with A replicated, rank r owning
columns slab(r) of B and C.  One process per GPU; the compute step has no collective — every
rank runs the ordinary single-GPU GEMM on its slab — and the only exchange is the optional
gather of C (and, for host-resident inputs, the replication of A over NVLink).

The exchange itself lives behind the library's C ABI (include/b200_gemm.h, "multi-GPU
column-slab driver": NCCL communicator, peer-visible buffers, NCCL all-gather + re-layout,
copy-engine push, and the slab GEMM with the gather fused into its epilogue).  This module is
the ctypes view of it; `torch.distributed` is used only as the side channel that carries the
128-byte communicator id and the 64-byte memory handles between the processes.

The reference (adelj88/rocm_wmma_gemm) is single-GPU; this driver has no counterpart there.
No kernel reads a peer's memory and no TMA load uses cluster multicast.

Slab storage (what each rank holds):
  A       the whole M x K matrix, in layout_a                      (replicated)
  B slab  K x n_count, dense, in layout_b  (for column-major B this is the contiguous block of
          columns [n_begin, n_begin + n_count) of the full matrix)
  C slab  M x n_count, dense, in layout_c  (not needed by the fused gather)
  C full  M x N in layout_c on every rank, after any of the three gathers
"""
from __future__ import annotations

import ctypes
from typing import Callable, Optional

import torch
import torch.distributed as dist

from . import GemmConfig, _check, lib as _lib
from . import loader as _loader
from . import slab as _slab

COMM_ID_BYTES = 128
IPC_HANDLE_BYTES = 64


def _interleave_row_major(gathered: torch.Tensor, M: int, widths) -> torch.Tensor:
    """[rank][M][width_r] (concatenated, each slab dense row-major) -> [M][sum(width)]."""
    parts, off = [], 0
    for w in widths:
        parts.append(gathered[off: off + M * w].view(M, w))
        off += M * w
    return torch.cat(parts, dim=1).contiguous().view(-1)


class _RawDeviceMemory:
    """Lets torch view device memory the library allocated (no copy, no ownership)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


def _stream_cell(stream):
    """Pointer to a cell holding the stream handle, as the C ABI takes streams."""
    handle = int(getattr(stream, "cuda_stream", stream)) if stream is not None else torch.cuda.current_stream().cuda_stream
    box = ctypes.c_void_p(handle)
    return box, ctypes.cast(ctypes.pointer(box), ctypes.c_void_p)


class SlabDriver:
    """One rank's handle on the C-ABI multi-GPU driver for one problem shape.

    Owns the NCCL communicator (`b200_gemm_comm_*`) and one peer-visible copy of the full C per
    rank (`b200_gemm_peer_*`): `full_c` is this rank's copy as a torch tensor; the other ranks'
    copies are mapped so that `push` and `gemm_gather` can write into them.  `types` is the
    library's type-pair index (0 f16<-f16, 1 f32<-f16, 2 bf16<-bf16, 3 f32<-bf16).
    """

    _OUT = {0: torch.float16, 1: torch.float32, 2: torch.bfloat16, 3: torch.float32}

    def __init__(self, M: int, N: int, K: int, types: int, layout_c: int = 0, layout_a: int = 0, layout_b: int = 1,
                 group=None, align: int = 256, peer_buffers: bool = True):
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("SlabDriver needs an initialised torch.distributed process group (the side channel)")
        self.lib = _lib()
        self.M, self.N, self.K, self.types = M, N, K, int(types)
        self.layout_c, self.layout_a, self.layout_b = int(layout_c), int(layout_a), int(layout_b)
        self.group, self.align = group, align
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.device = torch.cuda.current_device()
        self.n_begin, self.n_count = _slab(N, self.world, self.rank, align)
        self.out_dtype = self._OUT[self.types]
        self.esz = 4 if self.types in (1, 3) else 2
        # communicator: rank 0's id travels over the process group
        ident = ctypes.create_string_buffer(COMM_ID_BYTES)
        if self.rank == 0:
            _check(self.lib.b200_gemm_comm_id(ident))
        box = [bytes(ident.raw)]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
        self._comm = ctypes.c_void_p()
        _check(self.lib.b200_gemm_comm_create(box[0], self.world, self.rank, ctypes.byref(self._comm)))
        # one full C per rank, mapped into every process
        self._own = ctypes.c_void_p()
        self._ptrs = (ctypes.c_void_p * self.world)()
        self._mapped = []
        self.full_c = None
        if peer_buffers:
            nbytes = M * N * self.esz
            handle = ctypes.create_string_buffer(IPC_HANDLE_BYTES)
            _check(self.lib.b200_gemm_peer_alloc(nbytes, ctypes.byref(self._own), handle))
            handles = [None] * self.world
            dist.all_gather_object(handles, bytes(handle.raw), group=group)
            for r in range(self.world):
                if r == self.rank:
                    self._ptrs[r] = self._own.value
                else:
                    p = ctypes.c_void_p()
                    _check(self.lib.b200_gemm_peer_open(handles[r], ctypes.byref(p)))
                    self._ptrs[r] = p.value
                    self._mapped.append(p.value)
            self.full_c = torch.as_tensor(_RawDeviceMemory(self._own.value, nbytes), device=f"cuda:{self.device}").view(self.out_dtype)

    # -- the three gathers -----------------------------------------------------------------------
    def gemm_gather(self, A, B_slab, stream=None, config: Optional[GemmConfig] = None) -> None:
        """`b200_gemm_slab_gather`: slab GEMM whose epilogue stores every tile into every rank's
        full C.  Complete after `barrier()`."""
        box, sp = _stream_cell(stream)
        _check(self.lib.b200_gemm_slab_gather(self.types, self._ptrs, A.data_ptr(), B_slab.data_ptr(), self.M, self.N, self.K,
                                              self.layout_c, self.layout_a, self.layout_b, self.world, self.rank, self.align,
                                              sp, ctypes.byref(config) if config is not None else None))

    def push(self, C_slab, stream=None) -> None:
        """`b200_gemm_slab_push`: copy-engine copies of this rank's slab into every rank's full C."""
        box, sp = _stream_cell(stream)
        _check(self.lib.b200_gemm_slab_push(self.types, self._ptrs, C_slab.data_ptr(), self.M, self.N, self.layout_c,
                                            self.world, self.rank, self.align, sp))

    def allgather(self, C_full, C_slab, staging=None, stream=None) -> None:
        """`b200_gemm_slab_allgather`: NCCL all-gather of the slabs into `C_full` (any device
        buffer of M x N elements); row-major C needs `staging` of the same size."""
        box, sp = _stream_cell(stream)
        _check(self.lib.b200_gemm_slab_allgather(self._comm, self.types, C_full.data_ptr(),
                                                 C_slab.data_ptr() if C_slab is not None else None,
                                                 staging.data_ptr() if staging is not None else None,
                                                 self.M, self.N, self.layout_c, self.align, sp))

    # -- around them -----------------------------------------------------------------------------
    def barrier(self, stream=None) -> None:
        """Work queued on `stream` after this starts once every rank's stream has come this far."""
        box, sp = _stream_cell(stream)
        _check(self.lib.b200_gemm_comm_barrier(self._comm, sp))

    def replicate(self, buf, bytes_per_rank: int, stream=None) -> None:
        """In-place all-gather inside `buf`: block r (bytes_per_rank bytes) comes from rank r."""
        box, sp = _stream_cell(stream)
        _check(self.lib.b200_gemm_comm_allgather_inplace(self._comm, buf.data_ptr(), bytes_per_rank, sp))

    def gemm_host(self, C_slab, A, B_slab) -> None:
        """`b200_gemm_slab_host`: host tensors in (whole A, this rank's B slab), this rank's C
        slab out; 1/world of A crosses PCIe per GPU, NVLink carries the rest."""
        _check(self.lib.b200_gemm_slab_host(self._comm, self.types, C_slab.data_ptr(), A.data_ptr(), B_slab.data_ptr(),
                                            self.M, self.N, self.K, self.layout_c, self.layout_a, self.layout_b, self.align))

    def close(self) -> None:
        """Unmaps the peers' buffers, then (after every rank has done so) frees this rank's."""
        if self._comm:
            torch.cuda.synchronize()
            self.full_c = None
            for p in self._mapped:
                self.lib.b200_gemm_peer_close(p)
            self._mapped = []
            dist.barrier(group=self.group)
            if self._own:
                self.lib.b200_gemm_peer_free(self._own)
                self._own = ctypes.c_void_p()
            self.lib.b200_gemm_comm_destroy(self._comm)
            self._comm = ctypes.c_void_p()


class ColumnSlabGemm:
    """Plans and runs one rank's share of C = A * B.

    gemm_fn(C_slab, A, B_slab, M, n_count, K, layout_c, layout_a, layout_b) runs the local GEMM;
    the default is the library's loader (a B200 is required — there is no CPU path).  Tests on
    CPU ranks pass their own checker here; with CPU tensors the exchange goes through
    `torch.distributed` (gloo), with CUDA tensors through the library's own driver
    (`SlabDriver`).
    """

    def __init__(self, M: int, N: int, K: int, layout_c: int = 0, layout_a: int = 0, layout_b: int = 1,
                 group=None, align: int = 256, gemm_fn: Optional[Callable] = None,
                 rank: Optional[int] = None, world: Optional[int] = None):
        self.M, self.N, self.K = M, N, K
        self.layout_c, self.layout_a, self.layout_b = int(layout_c), int(layout_a), int(layout_b)
        self.group, self.align = group, align
        if world is None:
            world = dist.get_world_size(group) if dist.is_available() and dist.is_initialized() else 1
        if rank is None:
            rank = dist.get_rank(group) if dist.is_available() and dist.is_initialized() else 0
        self.rank, self.world = rank, world
        self.slabs = [_slab(N, world, r, align) for r in range(world)]
        self.n_begin, self.n_count = self.slabs[rank]
        self._gemm = gemm_fn
        self._loader = None
        self._driver = None

    def driver(self, types: int) -> SlabDriver:
        """The C-ABI driver for this shape (created on first use; collective: every rank calls it)."""
        if self._driver is None or self._driver.types != types:
            if self._driver is not None:
                self._driver.close()
            self._driver = SlabDriver(self.M, self.N, self.K, types, self.layout_c, self.layout_a, self.layout_b,
                                      group=self.group, align=self.align)
        return self._driver

    def close(self) -> None:
        if self._driver is not None:
            self._driver.close()
            self._driver = None

    @staticmethod
    def _types_of(C, A) -> int:
        return _loader._type_index(C, A, None)

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

    # -- compute with the exchange fused in --------------------------------------------------------
    def run_and_gather(self, C_slab: torch.Tensor, A: torch.Tensor, B_slab: torch.Tensor, panels: int = 4) -> torch.Tensor:
        """run() + gather() in one step; returns the full C (flat, layout_c).

        CUDA tensors: the slab GEMM stores every tile straight into every rank's full C
        (`b200_gemm_slab_gather`), then a barrier; `C_slab` is not touched.  Where the fused
        kernel does not apply (a plan outside the CTA-pair tiles) the route is run() then
        gather().  CPU tensors (tests of the host logic): the all-gather of row panel p is in
        flight while panel p + 1 is computed."""
        if C_slab.is_cuda and self._gemm is None and self.world > 1:
            from . import GemmError
            drv = self.driver(self._types_of(C_slab, A))
            try:
                drv.gemm_gather(A, B_slab)
            except GemmError as err:
                if err.status != 7:  # B200_GEMM_ERR_BAD_CONFIG: not a gathering tile
                    raise
                self.run(C_slab, A, B_slab)
                return self.gather(C_slab)
            drv.barrier()
            return drv.full_c
        widths = [c for _, c in self.slabs]
        even = len(set(widths)) == 1 and widths[0] * self.world == self.N
        if self.world == 1 or self.layout_a != 0 or self.layout_c != 0 or not even or panels < 2:
            self.run(C_slab, A, B_slab)
            return self.gather(C_slab)
        M, K, nl, G = self.M, self.K, self.n_count, self.world
        step = -(-M // panels)
        step = -(-step // 256) * 256
        Cf, Af = C_slab.reshape(-1), A.reshape(-1)
        full = torch.empty(M * self.N, dtype=Cf.dtype, device=Cf.device)
        pending = []
        for r0 in range(0, M, step):
            r1 = min(M, r0 + step)
            Cp = Cf[r0 * nl: r1 * nl]
            self._local(Cp, Af[r0 * K: r1 * K], B_slab, r1 - r0)
            stage = torch.empty(G * (r1 - r0) * nl, dtype=Cf.dtype, device=Cf.device)
            work = dist.all_gather_into_tensor(stage.view(torch.uint8), Cp.view(torch.uint8), group=self.group, async_op=True)
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
        if C_slab.is_cuda and self._gemm is None:
            # the library's driver: NCCL all-gather (+ re-layout kernel for row-major C)
            types = {torch.float16: 0, torch.float32: 1, torch.bfloat16: 2}[C_slab.dtype]
            drv = self.driver(types)
            staging = torch.empty(M * self.N, dtype=C_slab.dtype, device=C_slab.device) if self.layout_c == 0 else None
            drv.allgather(drv.full_c, C_slab, staging)
            return drv.full_c
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
