"""CPU tests of the tuned-config machinery: the compiled lookup agrees with a Python
restatement of the reference's selection order over the committed JSON tables, the generator
is deterministic, the GOMEA search finds optima of synthetic landscapes, and the tuner's
constraint checker matches what the library accepts."""
import json
import os
import random

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CFG_DIR = os.path.join(ROOT, "rocm_wmma_gemm_b200", "config")

from rocm_wmma_gemm_b200.config import generate_config, tune  # noqa: E402
from rocm_wmma_gemm_b200.config.gomea import Gomea, learn_models, mutual_information, upgma_subsets  # noqa: E402


def load_entries():
    f16 = os.path.join(CFG_DIR, "gemm_config_sm100_f16.json")
    f32 = os.path.join(CFG_DIR, "gemm_config_sm100_f32.json")
    return generate_config.load(f16, 0) + generate_config.load(f32, 1)


def py_find_best(entries, m, n, k, tg, la, lb, lc):
    """The reference's order (config/generate_config.py:174-271): exact, exact in group 0,
    closest (nearest K, then nearest (M, N)) in the group, closest in group 0, default."""
    table = dict(entries)

    def exact(g):
        return table.get((m, n, k, g, la, lb, lc))

    def closest(g):
        cands = [(key, cfg) for key, cfg in entries if key[3] == g and key[4:] == (la, lb, lc)]
        if not cands:
            return None
        best_k = None
        for key, _ in cands:  # first strict minimum in table order (the table is sorted)
            d = abs(key[2] - k)
            if best_k is None or d < best_k[0]:
                best_k = (d, key[2])
        best = None
        for key, cfg in cands:
            if key[2] != best_k[1]:
                continue
            d = float(m - key[0]) ** 2 + float(n - key[1]) ** 2
            if best is None or d < best[0]:
                best = (d, cfg)
        return best[1]

    r = exact(tg)
    if r is None and tg != 0:
        r = exact(0)
    if r is None:
        r = closest(tg)
    if r is None and tg != 0:
        r = closest(0)
    return r if r is not None else generate_config.DEFAULT_CONFIG


def test_compiled_table_matches_json_and_selection_order(gemm_lib):
    entries = sorted(load_entries())
    assert entries, "the tuned JSON table is committed"
    rng = random.Random(0)
    queries = [key[:3] for key, _ in entries[::7]]
    queries += [(rng.choice([16, 100, 1024, 3000, 8192, 20000]), rng.choice([8, 512, 4096, 28672, 50000]),
                 rng.choice([16, 64, 1000, 4096, 8192, 30000])) for _ in range(200)]
    for (m, n, k) in queries:
        for tg in (0, 1):
            for la in (0, 1):
                for lb in (0, 1):
                    for lc in (0, 1):
                        cfg, idx = gemm_lib.get_gemm_params(m, n, k, lc, la, lb, tg)
                        want = py_find_best(entries, m, n, k, tg, la, lb, lc)
                        got = (cfg.tile_m, cfg.tile_n, cfg.stages, cfg.cluster, cfg.split_k, cfg.raster)
                        assert got == want, (m, n, k, tg, la, lb, lc)


def test_every_table_config_is_a_compiled_variant():
    for _, cfg in load_entries():
        tile_m, tile_n, stages, cluster, split_k, raster = cfg
        assert tile_m == 128 * cluster and cluster in (1, 2)
        assert tune.check_constraints((tile_m, tile_n, stages, split_k, raster))


def test_generator_is_deterministic_and_sorted(tmp_path):
    configs, rows, default_idx = generate_config.build_table(os.path.join(CFG_DIR, "gemm_config_sm100_f16.json"),
                                                             os.path.join(CFG_DIR, "gemm_config_sm100_f32.json"))
    assert configs == sorted(set(configs)) and configs[default_idx] == generate_config.DEFAULT_CONFIG
    assert [r[0] for r in rows] == sorted(r[0] for r in rows)
    text = generate_config.render(configs, rows, default_idx, ["x.json"])
    committed = open(os.path.join(ROOT, "rocm_wmma_gemm_b200", "csrc", "config_table.inc")).read()
    strip = lambda s: "\n".join(s.splitlines()[1:])
    assert strip(text) == strip(committed), "config_table.inc is stale: run config/generate_config.py"


def test_json_schema_is_the_references():
    with open(os.path.join(CFG_DIR, "gemm_config_sm100_f16.json")) as f:
        data = json.load(f)
    e = data["configurations"][0]
    assert set(e["range"]) == {"M", "N", "K"} and set(e["layout"]) == {"A", "B", "C"}
    assert set(e["config"]) == {"tile_m", "tile_n", "stages", "cluster", "split_k", "raster"}


def test_constraints():
    ok = tune.check_constraints
    assert ok((256, 512, 4, 1, 16)) and not ok((256, 512, 5, 1, 16))      # 5 x 48 KiB does not fit
    assert ok((128, 256, 4, 1, 8)) and not ok((128, 512, 2, 1, 8))        # 512 columns need a CTA pair
    assert not ok((256, 64, 4, 1, 8))                                      # a pair stages >= 64 B rows per CTA
    assert ok((128, 64, 8, 1, 8)) and ok((256, 128, 8, 1, 8))
    assert ok((256, 192, 6, 1, 8)) and not ok((128, 192, 4, 1, 8))         # in-between widths: CTA pairs only
    assert not ok((128, 128, 4, 32, 0), 128, 128, 1024)                    # more partitions than k-blocks
    assert not ok((128, 128, 4, 3, 0), 128, 128, 256)                      # 4 k-blocks in 3 parts is really 2
    assert len(tune.enumerate_valid(8192, 8192, 8192, 0)) > 500


def test_linkage_learning_finds_coupled_parameters():
    rng = random.Random(3)
    configs = []
    for _ in range(200):
        a = rng.choice([1, 2, 4, 8])
        configs.append((a, a * 2, rng.choice([0, 1, 2, 3]), rng.choice([5, 6, 7])))
    mi = mutual_information(configs)
    assert mi[0][1] > 10 * max(mi[0][2], mi[0][3], mi[2][3])
    fos = upgma_subsets(mi)
    assert (0, 1) in fos or (1, 0) in fos
    assert all((i,) in fos for i in range(4))
    models = learn_models({c: float(i) for i, c in enumerate(set(configs))})
    assert models and all(len(m) == 2 for m in models)


@pytest.mark.parametrize("seed", [0, 1, 2])
def test_gomea_finds_the_optimum_of_a_deceptive_landscape(seed):
    space = [(a, b, c, d, e) for a in range(4) for b in range(4) for c in range(4) for d in range(3) for e in range(3)]

    def cost(x):
        a, b, c, d, e = x
        block = 0.0 if (a, b) == (3, 3) else 1.0 + 0.1 * (a + b)   # a and b only pay off together
        return block + 0.3 * abs(c - 2) + 0.2 * d + 0.1 * abs(e - 1)

    search = Gomea(space, cost, budget=220, rng=random.Random(seed), strata=lambda x: x[0] * x[1])
    res = search.run()
    assert res.evaluations <= 220
    assert res.best_cost <= 0.1 + 1e-9, (res.best, res.best_cost)
    assert cost(res.best) == res.best_cost and res.elites[0][1] == res.best


def test_gomea_respects_budget_seeds_and_validity():
    valid = tune.enumerate_valid(8192, 8192, 8192, 0)
    seen = []

    def cost(c):
        seen.append(c)
        return 1.0 / (c[0] * c[1]) + 0.01 * c[3]

    seed_cfg = (256, 512, 4, 1, 16)
    res = Gomea(valid, cost, budget=40, seeds=[seed_cfg, (1, 2, 3, 4, 5)], rng=random.Random(1)).run()
    assert len(seen) == len(set(seen)) <= 40 and seen[0] == seed_cfg
    assert set(seen) <= set(valid)
    assert res.best[:2] == (256, 512)
