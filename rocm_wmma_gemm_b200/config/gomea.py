"""Parameter-less GOMEA over a small constrained discrete space.

The search method the reference's tuner uses (rocm_wmma_gemm/config/tune.py:55-765 of
adelj88/rocm_wmma_gemm): the Gene-pool Optimal Mixing Evolutionary Algorithm run under the
interleaved multistart scheme (populations of 4 * 2^c individuals, stepped in the order
0, 1, 0, 2, 0, 1, 0, 3, ...), with a linkage model re-learned every generation from the
better half of everything evaluated so far (rank-based mutual information between
parameters, UPGMA-clustered into a family of subsets), neutral moves accepted, forced
improvement towards the nearest elite of a small niched hall of fame, and a random restart
of individuals that still do not improve.  It is hardware-agnostic: the caller supplies the
parameter space, a validity predicate and a cost function (lower is better, `inf` = failed).

The implementation is written for this repository; only the algorithm is shared.
"""
from __future__ import annotations

import math
import random
from collections import Counter
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple

Config = Tuple[int, ...]
INF = float("inf")


def hamming(a: Config, b: Config) -> int:
    return sum(1 for x, y in zip(a, b) if x != y)


# ---------------------------------------------------------------------------------------------
# Linkage learning
# ---------------------------------------------------------------------------------------------
def _binned_ranks(column: Sequence[int], bins: int) -> List[int]:
    """Ordinal transform of one parameter column: distinct values -> fractional rank in [0, 1]
    -> one of `bins` equal-width bins."""
    levels = sorted(set(column))
    span = max(len(levels) - 1, 1)
    where = {v: i / span for i, v in enumerate(levels)}
    return [min(int(where[v] * bins), bins - 1) for v in column]


def mutual_information(configs: Sequence[Config], bins: int = 4) -> List[List[float]]:
    """Pairwise mutual information between parameters over a set of configurations."""
    n = len(configs)
    d = len(configs[0])
    cols = [_binned_ranks([c[k] for c in configs], bins) for k in range(d)]
    mi = [[0.0] * d for _ in range(d)]
    for i in range(d):
        pi = Counter(cols[i])
        for j in range(i + 1, d):
            pj = Counter(cols[j])
            pij = Counter(zip(cols[i], cols[j]))
            total = 0.0
            for (a, b), c in pij.items():
                total += (c / n) * math.log((c * n) / (pi[a] * pj[b]))
            mi[i][j] = mi[j][i] = total
    return mi


def upgma_subsets(mi: List[List[float]], floor: float = 1e-6) -> List[Tuple[int, ...]]:
    """Family of subsets from average-linkage clustering of the MI matrix: all singletons plus
    every merged group short of the full set; merging stops once the strongest remaining
    average MI is not above `floor` (no linkage left worth modelling)."""
    d = len(mi)
    clusters: List[Tuple[int, ...]] = [(i,) for i in range(d)]
    fos: List[Tuple[int, ...]] = list(clusters)
    while len(clusters) > 1:
        best, pair = -INF, None
        for x in range(len(clusters)):
            for y in range(x + 1, len(clusters)):
                a, b = clusters[x], clusters[y]
                avg = sum(mi[p][q] for p in a for q in b) / (len(a) * len(b))
                if avg > best:
                    best, pair = avg, (x, y)
        if best <= floor:
            break
        x, y = pair
        merged = clusters[x] + clusters[y]
        clusters = [c for k, c in enumerate(clusters) if k not in (x, y)] + [merged]
        if len(merged) < d:
            fos.append(merged)
    return fos


def learn_models(history: Dict[Config, float], tau: float = 0.5, min_sample: int = 8):
    """[(leader, fos)] — one linkage model per structural cluster of the better `tau` fraction
    of everything evaluated so far.  With too few survivors: a single univariate model."""
    scored = sorted(((t, c) for c, t in history.items() if t != INF), key=lambda x: x[0])
    if not scored:
        return []
    d = len(scored[0][1])
    univariate = [(i,) for i in range(d)]
    keep = [c for _, c in scored[: int(len(scored) * tau)]]
    if len(keep) < min_sample:
        return [(scored[0][1], univariate)]
    radius = max(2, int(d * 0.3))
    groups: Dict[Config, List[Config]] = {}
    for c in keep:  # leader clustering, best first
        for leader in groups:
            if hamming(c, leader) <= radius:
                groups[leader].append(c)
                break
        else:
            groups[c] = [c]
    models = []
    for leader, members in groups.items():
        models.append((leader, upgma_subsets(mutual_information(members)) if len(members) > 1 else univariate))
    return models


# ---------------------------------------------------------------------------------------------
# Search
# ---------------------------------------------------------------------------------------------
@dataclass
class Result:
    best: Optional[Config]
    best_cost: float
    evaluations: int
    history: Dict[Config, float] = field(default_factory=dict)
    elites: List[Tuple[float, Config]] = field(default_factory=list)


class Gomea:
    """minimise(cost) over `valid` (the enumerated feasible configurations)."""

    MAX_ELITES = 4
    STAGNATION_LIMIT = 4

    def __init__(self, valid: Sequence[Config], cost: Callable[[Config], float], budget: int,
                 seeds: Sequence[Config] = (), strata: Optional[Callable[[Config], float]] = None,
                 rng: Optional[random.Random] = None, log: Callable[[str], None] = lambda s: None):
        self.valid = list(valid)
        self.valid_set = set(self.valid)
        self.cost_fn = cost
        self.budget = budget
        self.seeds = [s for s in seeds if s in self.valid_set]
        self.strata = strata
        self.rng = rng or random.Random(0)
        self.log = log
        self.history: Dict[Config, float] = {}
        self.evals = 0
        self.elites: List[Tuple[float, Config]] = []

    # -- evaluation with memo; every distinct configuration costs one unit of budget ----------
    def cost(self, c: Config) -> float:
        if c in self.history:
            return self.history[c]
        t = self.cost_fn(c)
        self.history[c] = t
        self.evals += 1
        return t

    def exhausted(self) -> bool:
        return self.evals >= self.budget or len(self.history) >= len(self.valid)

    # -- initial populations: unseen configurations, largest stratum first, round-robin -------
    def _fresh(self, count: int) -> List[Config]:
        unseen = [c for c in self.valid if c not in self.history]
        self.rng.shuffle(unseen)
        if self.strata is None:
            return unseen[:count]
        buckets: Dict[float, List[Config]] = {}
        for c in unseen:
            buckets.setdefault(self.strata(c), []).append(c)
        order = sorted(buckets, reverse=True)
        picked: List[Config] = []
        depth = 0
        while len(picked) < count:
            took = False
            for key in order:
                if depth < len(buckets[key]) and len(picked) < count:
                    picked.append(buckets[key][depth])
                    took = True
            if not took:
                break
            depth += 1
        return picked

    def _merge_elites(self, population: List[Tuple[float, Config]]):
        local: List[Tuple[float, Config]] = []
        for t, c in sorted(population, key=lambda x: x[0]):
            if t != INF and all(hamming(c, e) >= 2 for _, e in local):
                local.append((t, c))
            if len(local) == self.MAX_ELITES:
                break
        for t, c in local:
            for k, (gt, gc) in enumerate(self.elites):
                if hamming(c, gc) < 2:  # same niche: keep the faster
                    if t < gt:
                        self.elites[k] = (t, c)
                    break
            else:
                self.elites.append((t, c))
        self.elites = sorted(self.elites, key=lambda x: x[0])[: self.MAX_ELITES]
        return local

    # -- optimal mixing ------------------------------------------------------------------------
    def _mix(self, current: Config, cur_cost: float, donors: Callable[[], Config], fos, accept_neutral=True):
        improved = False
        cur = list(current)
        groups = list(fos)
        self.rng.shuffle(groups)
        for group in groups:
            if self.exhausted():
                break
            donor = donors()
            if all(cur[i] == donor[i] for i in group):
                continue
            trial = list(cur)
            for i in group:
                trial[i] = donor[i]
            trial_t = tuple(trial)
            if trial_t not in self.valid_set:
                continue
            t = self.cost(trial_t)
            if t < cur_cost or (accept_neutral and t == cur_cost):
                improved = improved or t < cur_cost
                cur, cur_cost = trial, t
        return tuple(cur), cur_cost, improved

    def _generation(self, population: List[Tuple[float, Config]]):
        models = learn_models(self.history)
        local_elites = self._merge_elites(population)
        nxt: List[Tuple[float, Config]] = []
        for idx, (t, c) in enumerate(population):
            if self.exhausted():
                nxt.append((t, c))
                continue
            fos = min(models, key=lambda m: hamming(c, m[0]))[1] if models else [(i,) for i in range(len(c))]
            others = [p[1] for k, p in enumerate(population) if k != idx] or [c]
            c2, t2, improved = self._mix(c, t, lambda: self.rng.choice(others), fos)
            if not improved and len(others) > 0 and not self.exhausted():
                donor = self.rng.choice(others)  # whole-configuration swap as a last partial move
                if donor != c2 and self.cost(donor) < t2:
                    c2, t2, improved = donor, self.history[donor], True
            if not improved and local_elites:
                et, ec = min(local_elites, key=lambda e: hamming(c2, e[1]))
                if t2 > et:  # forced improvement: pull towards the nearest elite, strict gains only
                    c2, t2, improved = self._mix(c2, t2, lambda: ec, fos, accept_neutral=False)
                    if not improved and not self.exhausted():
                        fresh = self._fresh(1)
                        if fresh:
                            c2, t2 = fresh[0], self.cost(fresh[0])
            nxt.append((t2, c2))
        return nxt

    def run(self) -> Result:
        populations: List[List[Tuple[float, Config]]] = []
        best_seen: List[float] = []
        stagnant: List[int] = []
        step = 0
        idle_steps = 0
        while not self.exhausted() and idle_steps < 64:
            step += 1
            level = (step & -step).bit_length() - 1  # 0,1,0,2,0,1,0,3,...
            if level > len(populations):
                continue
            if level == len(populations):
                size = 4 * (2 ** level)
                members: List[Tuple[float, Config]] = []
                if level == 0:
                    for s in self.seeds:
                        members.append((self.cost(s), s))
                else:
                    members.extend(self.elites[:size])
                for c in self._fresh(max(0, size - len(members))):
                    if self.exhausted():
                        break
                    members.append((self.cost(c), c))
                if not members:
                    break
                populations.append(members)
                best_seen.append(INF)
                stagnant.append(0)
                self.log(f"population {level}: {len(members)} individuals")
            pop = populations[level]
            if stagnant[level] >= self.STAGNATION_LIMIT or len({c for _, c in pop}) <= 1 or len(pop) < 2:
                idle_steps += 1
                continue
            idle_steps = 0
            pop = self._generation(pop)
            populations[level] = pop
            top = min(t for t, _ in pop)
            if top < best_seen[level]:
                best_seen[level], stagnant[level] = top, 0
            else:
                stagnant[level] += 1
        for pop in populations:
            self._merge_elites(pop)
        scored = [(t, c) for c, t in self.history.items() if t != INF]
        if not scored:
            return Result(None, INF, self.evals, self.history, [])
        t, c = min(scored, key=lambda x: x[0])
        return Result(c, t, self.evals, self.history, list(self.elites))
