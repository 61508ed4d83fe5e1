"""The column-slab driver's host logic on two CPU ranks over gloo.  The local GEMM of each
rank is the oracle (the product has no CPU path); what is under test is the partition, the
slab storage convention and the all-gather + re-layout of C."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import oracle


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _logical(bits, rows, cols, layout):
    return bits.reshape(rows, cols) if layout == 0 else bits.reshape(cols, rows).T


def _store(mat, layout):
    return np.ascontiguousarray(mat if layout == 0 else mat.T).ravel()


def _worker(rank, world, port, M, N, K, lc, la, lb, types, align, result_file):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from rocm_wmma_gemm_b200.multi_gpu import ColumnSlabGemm
    bf16 = types >= 2
    A = oracle.init_matrix(M, K, la, bf16)
    B_full = _logical(oracle.init_matrix(K, N, lb, bf16), K, N, lb)

    def cpu_gemm(C_slab, A_t, B_t, m, n, k, c_l, a_l, b_l):
        out = oracle.hgemm(types, A_t.numpy().view(np.uint16), B_t.numpy().view(np.uint16), m, n, k, c_l, a_l, b_l)
        C_slab.copy_(torch.from_numpy(out.view(np.int16) if out.dtype == np.uint16 else out))

    plan = ColumnSlabGemm(M, N, K, lc, la, lb, align=align, gemm_fn=cpu_gemm)
    n0, nl = plan.n_begin, plan.n_count
    B_slab = torch.from_numpy(_store(B_full[:, n0:n0 + nl], lb).view(np.int16))
    out_dt = torch.float32 if types in (1, 3) else torch.int16
    C_slab = torch.zeros(M * max(nl, 1), dtype=out_dt)
    A_t = torch.from_numpy(A.view(np.int16))
    plan.run(C_slab, A_t, B_slab)
    full = plan.gather(C_slab[: M * nl])
    # the overlapped route must give the same matrix (it falls back where it does not apply)
    C2 = torch.zeros_like(C_slab)
    full2 = plan.run_and_gather(C2, A_t, B_slab, panels=3)
    assert torch.equal(full2, full), "run_and_gather differs from run + gather"
    if rank == 1 % world:
        np.save(result_file, full.numpy())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("M,N,K,lc,la,lb,types,align", [
    (48, 512, 64, 0, 0, 1, 3, 256),   # the benchmark's layout: A row, B col, C row; even slabs
    (600, 512, 32, 0, 0, 1, 2, 256),  # several row panels through the overlapped route
    (40, 512, 32, 1, 1, 0, 0, 256),   # column-major C: slabs concatenate
    (24, 1000, 48, 0, 0, 0, 1, 256),  # ragged: slabs of 512 and 488 columns
    (16, 200, 32, 1, 0, 1, 2, 256),   # fewer column groups than ranks: rank 1 owns nothing
])
def test_column_slab_two_ranks(tmp_path, M, N, K, lc, la, lb, types, align):
    world = 2
    port = _free_port()
    result = str(tmp_path / "full.npy")
    mp.spawn(_worker, args=(world, port, M, N, K, lc, la, lb, types, align, result), nprocs=world, join=True)
    got = np.load(result)
    bf16 = types >= 2
    ref = oracle.hgemm(types, oracle.init_matrix(M, K, la, bf16), oracle.init_matrix(K, N, lb, bf16), M, N, K, lc, la, lb)
    ref = ref.view(np.int16) if ref.dtype == np.uint16 else ref
    assert got.shape == ref.shape
    assert np.array_equal(got, ref)


def test_single_rank_plan_needs_no_process_group():
    from rocm_wmma_gemm_b200.multi_gpu import ColumnSlabGemm
    plan = ColumnSlabGemm(128, 16384, 64, world=8, rank=3)
    assert (plan.n_begin, plan.n_count) == (6144, 2048)
    assert sum(c for _, c in plan.slabs) == 16384
