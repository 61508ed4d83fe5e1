"""The multi-GPU column-slab driver on real GPUs (needs at least two): one process per GPU, each
computes its slab through the C ABI and the three gathers of C — NCCL all-gather + re-layout,
copy-engine push, and the slab GEMM with the gather fused into its epilogue — must all leave
the reference's result (the CPU oracle on the same seeded inputs) on EVERY rank."""
import os
import socket

import numpy as np
import pytest
import torch

import oracle

pytestmark = pytest.mark.gpu


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


CASES = [
    # types, M, N, K, lc, la, lb, align
    (2, 512, 1024, 256, 0, 0, 1, 256),   # the benchmark's layouts (bf16 -> bf16), even slabs
    (3, 384, 1536, 192, 1, 1, 0, 256),   # f32 out, column-major C: slabs concatenate
    (0, 256, 1280, 128, 0, 0, 0, 256),   # f16, ragged slabs at 2 and 4 ranks (N is not a multiple of world x align)
    (1, 520, 2048, 320, 0, 1, 1, 64),    # f32 out, ragged M (edge tiles clipped inside the full matrix)
    (2, 4608, 1024, 128, 0, 0, 1, 256),  # tall enough for the host-buffer call to work in two row panels
]


def _worker(rank, world, port, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    import torch.distributed as dist
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import rocm_wmma_gemm_b200 as g
    from rocm_wmma_gemm_b200.multi_gpu import ColumnSlabGemm, SlabDriver
    L = g.loader()
    failures = []
    for ci, (types, M, N, K, lc, la, lb, align) in enumerate(CASES):
        bf16 = types >= 2
        A = oracle.init_matrix(M, K, la, bf16)
        B_full = _logical(oracle.init_matrix(K, N, lb, bf16), K, N, lb)
        drv = SlabDriver(M, N, K, types, lc, la, lb, align=align)
        n0, nl = drv.n_begin, drv.n_count
        dA = torch.from_numpy(A.view(np.int16)).cuda()
        dB = torch.from_numpy(_store(B_full[:, n0:n0 + nl], lb).view(np.int16)).cuda() if nl else torch.zeros(8, dtype=torch.int16, device="cuda")
        out_dt = torch.float32 if types in (1, 3) else torch.int16
        C_slab = torch.zeros(M * max(nl, 1), dtype=out_dt, device="cuda")
        if nl:
            L.gemm(C_slab, dA, dB, M, nl, K, lc, la, lb, types=types)
        full = drv.full_c.view(out_dt)
        results = {}
        # 1. NCCL all-gather (+ re-layout for row-major C)
        full.fill_(-1)
        staging = torch.empty(M * N, dtype=out_dt, device="cuda") if lc == 0 else None
        drv.allgather(full, C_slab, staging)
        torch.cuda.synchronize()
        results["allgather"] = full.cpu().numpy().copy()
        dist.barrier()
        # 2. copy-engine push into every rank's full C
        full.fill_(-1)
        torch.cuda.synchronize()
        dist.barrier()
        drv.push(C_slab)
        drv.barrier()
        torch.cuda.synchronize()
        results["push"] = full.cpu().numpy().copy()
        dist.barrier()
        # 3. the slab GEMM with the gather fused into its epilogue (twice: the second run finds
        #    the first one's output in place)
        for rep in range(2):
            full.fill_(-1)
            torch.cuda.synchronize()
            dist.barrier()
            drv.gemm_gather(dA, dB)
            drv.barrier()
            torch.cuda.synchronize()
        results["fused"] = full.cpu().numpy().copy()
        dist.barrier()
        g.device_status()
        ref = oracle.hgemm(types, A, oracle.init_matrix(K, N, lb, bf16), M, N, K, lc, la, lb)
        ref = ref.view(np.int16) if ref.dtype == np.uint16 else ref
        slab_ref = None
        for name, got in results.items():
            if types in (1, 3):
                ok = np.allclose(got, ref, rtol=0, atol=1e-4)
            else:
                gf = oracle.bits_to_f32(got.view(np.uint16), bf16)
                rf = oracle.bits_to_f32(ref.view(np.uint16), bf16)
                eps = 2.0 ** -8 if bf16 else 2.0 ** -11
                ok = bool((np.abs(gf - rf) <= 2 * eps * np.abs(rf) + eps * np.sqrt(K) / 3.0).all())
            if not ok:
                failures.append(f"case {ci} rank {rank}: {name} differs from the CPU reference")
        # 4. host buffers in, host slab out: 1 / world of A over PCIe, the rest over NVLink
        hA = torch.from_numpy(A.view(np.int16)).pin_memory()
        hB = torch.from_numpy(_store(B_full[:, n0:n0 + nl], lb).view(np.int16)) if nl else torch.zeros(8, dtype=torch.int16)
        hC = torch.full((M * max(nl, 1),), -1, dtype=out_dt)
        drv.gemm_host(hC, hA, hB)
        if nl and not torch.equal(hC[: M * nl], C_slab[: M * nl].cpu()):
            failures.append(f"case {ci} rank {rank}: the host-buffer slab call differs from the device-pointer call")
        # the three routes move the same numbers: bit-equal among themselves where the tile
        # shapes agree (all-gather and push both carry the slab the plain call produced)
        if not np.array_equal(results["allgather"], results["push"]):
            failures.append(f"case {ci} rank {rank}: push differs from allgather")
        drv.close()
    # the high-level wrapper: run_and_gather on CUDA tensors = fused route
    types, M, N, K, lc, la, lb, align = CASES[0]
    plan = ColumnSlabGemm(M, N, K, lc, la, lb, align=align)
    A = oracle.init_matrix(M, K, la, True)
    B_full = _logical(oracle.init_matrix(K, N, lb, True), K, N, lb)
    dA = torch.from_numpy(A.view(np.int16)).cuda().view(torch.bfloat16)
    dB = torch.from_numpy(_store(B_full[:, plan.n_begin:plan.n_begin + plan.n_count], lb).view(np.int16)).cuda().view(torch.bfloat16)
    C_slab = torch.zeros(M * plan.n_count, dtype=torch.bfloat16, device="cuda")
    full1 = plan.run_and_gather(C_slab, dA, dB).clone()
    plan.run(C_slab, dA, dB)
    full2 = plan.gather(C_slab).clone()
    torch.cuda.synchronize()
    ref = oracle.hgemm(types, A, oracle.init_matrix(K, N, lb, True), M, N, K, lc, la, lb)
    for name, t in (("run_and_gather", full1), ("gather", full2)):
        gf = oracle.bits_to_f32(t.view(torch.int16).cpu().numpy().view(np.uint16), True)
        rf = oracle.bits_to_f32(ref, True)
        if not (np.abs(gf - rf) <= 2 * 2.0 ** -8 * np.abs(rf) + 2.0 ** -8 * np.sqrt(K) / 3.0).all():
            failures.append(f"ColumnSlabGemm.{name} rank {rank} differs from the CPU reference")
    plan.close()
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as f:
        f.write("\n".join(failures))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_three_gathers_match_the_reference_on_every_rank(tmp_path, world):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        text = open(tmp_path / f"rank{r}.txt").read()
        assert text == "", text


def test_slab_driver_from_plain_cpp():
    """tests/cpp/test_slab_driver.cpp: host threads as ranks, plain peer pointers, no Python in
    the loop - the fused gather and the NCCL all-gather against the CPU reference on every rank."""
    import shutil
    import subprocess
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    if shutil.which("g++") is None or shutil.which("gcc") is None:
        pytest.skip("no host C++ compiler on this machine")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    built = subprocess.run(["sh", os.path.join(root, "tests", "cpp", "build_slab_test.sh")], capture_output=True, text=True, timeout=600)
    assert built.returncode == 0, built.stdout + built.stderr
    proc = subprocess.run([os.path.join(root, "tests", "cpp", "test_slab_driver")], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-3000:] + proc.stderr[-3000:]
    assert "0 failed" in proc.stdout
