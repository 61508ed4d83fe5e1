"""Launch rules for sizes without a table entry and for skinny problems, checked through
`b200_gemm_plan` (pure host code, no GPU): each case is a choice that was measured on a B200
against the alternatives, so a change of the cost models that flips one of them shows up here."""
import pytest

import rocm_wmma_gemm_b200 as g

KERNEL = {"generic": 1, "staged": 2, "transposed": 3}


def plan(M, N, K, types=2, layouts=(0, 1, 0)):
    la, lb, lc = layouts
    return g.plan(M, N, K, lc, la, lb, types=types, sm_count=148)


@pytest.mark.parametrize("shape,split,cluster_k,slab", [
    ((16, 8192, 8192), 1, 0, 56),     # 147 one-CTA slabs: K partitions gain nothing (the model sees 3 %)
    ((64, 8192, 8192), 2, 1, 112),    # 74 slabs x 2: halves the L2 re-reads of the 64-row operand
    ((16, 4096, 14336), 2, 1, 56),    # few rows, long K: the MMA thread, not HBM, bounded 32-row slabs
    ((64, 28672, 8192), 1, 0, 104),   # two waves of slabs: persistent one-CTA slabs
    ((16, 28672, 8192), 1, 0, 104),
])
def test_skinny_problems_choose_slabs_and_k_partitions(shape, split, cluster_k, slab):
    p = plan(*shape, types=1)
    assert p.kernel == KERNEL["transposed"]
    assert (p.split_k, p.cluster_k, p.tile_m) == (split, cluster_k, slab)


def test_clusters_of_four_count_on_seven_eighths_of_the_sms():
    # 64 x 4096 x 4096: four K partitions, and 32 slabs of 128 rows (128 CTAs), not 37 of 112 (148):
    # 37 clusters of four do not fit at once and took two waves
    p = plan(64, 4096, 4096, types=1)
    assert (p.kernel, p.split_k, p.cluster_k, p.tile_m, p.ctas) == (KERNEL["transposed"], 4, 1, 128, 128)


@pytest.mark.parametrize("shape,tile,cluster,split,cluster_k", [
    ((128, 4096, 4096), (128, 128), 1, 4, 1),     # K partitions inside clusters instead of a second kernel
    ((256, 4096, 4096), (128, 128), 1, 2, 1),
    ((100, 5000, 5000), (128, 128), 1, 3, 1),     # a cluster of three
    ((8192, 128, 8192), (128, 128), 1, 2, 1),
    ((8192, 8192, 128), (128, 256), 1, 1, 0),     # short K: the output drain decides, one-CTA tiles drain faster
    ((4096, 4096, 64), (128, 256), 1, 1, 0),      # not 2048 narrow tiles (per-tile overhead)
    ((1536, 1536, 1536), (128, 128), 1, 1, 0),    # one wave of small tiles beats one wave of pair tiles
    ((2304, 2304, 2304), (256, 192), 2, 1, 0),    # 81 pair tiles of 256 columns would need two waves
    ((3000, 3000, 3000), (256, 256), 2, 1, 0),    # two waves: pairs, not one-CTA tiles
    ((512, 512, 4096), (128, 128), 1, 8, 0),      # more partitions than a cluster takes: workspace + reduction pass
])
def test_sizes_without_a_table_entry(shape, tile, cluster, split, cluster_k):
    p = plan(*shape)
    assert p.kernel == KERNEL["staged"]
    assert ((p.tile_m, p.tile_n), p.cluster, p.split_k, p.cluster_k) == (tile, cluster, split, cluster_k)


def test_run_time_widths_need_a_k_major_operand_and_whole_output_chunks():
    # B row-major (an N-major B' in the kernel view) cannot use the in-between pair widths
    assert plan(2304, 2304, 2304, layouts=(0, 0, 0)).tile_n in (128, 256, 512)
    # f32 output: chunks of 32 columns, so 160 is allowed where 16-bit outputs (64) take 192
    assert plan(2304, 2304, 2304, types=3).tile_n == 160
    assert plan(2304, 2304, 2304, types=2).tile_n == 192
