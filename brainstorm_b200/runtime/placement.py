"""Expert placement for expert-parallel routing: which rank hosts which expert of every MoE
layer, chosen from captured routing statistics so that a token's consecutive experts tend to
sit on the same rank and the all-to-all has less to move.

Counterpart of python/brt/runtime/placement.py:25-357 and of the search the reference runs
offline on top of it (benchmark/swin_moe/placement_cvxpy.py:14-76): the fabrics capture, per
scatter router, the cells every path received (``cell_decision_history``,
python/brt/router/fabric/base.py:150-201); consecutive routers give a transition matrix
``trace[i][p, q]`` = cells that took path p in layer i and path q in layer i + 1; the search
minimises the cells that change rank between layers,

    cost = sum_i sum_{p, q} trace[i][p, q] * [rank_i(p) != rank_{i+1}(q)],

with every rank hosting the same number of experts of every layer (what the sharded expert
weights of the fabrics require).  The reference hands this 0/1 program to cvxpy or Gurobi;
neither is a dependency here, so the search is a layer-by-layer assignment followed by
pairwise-swap descent (exhaustive for tiny problems), all in numpy.

The Swin-MoE checkpoint resharding of the reference's file (``adaptive_load_checkpoint``) is
model code and is not reproduced; ``reorder_gate_rows`` is the part of it that touches the
routing path (the gate's output rows follow the experts to their new ranks).
"""
import itertools
from typing import Dict, Iterator, List, Sequence, Tuple

import numpy as np
import torch
import torch.nn as nn

__all__ = [
    "sorted_k_even_partitions", "possible_placement_generator",
    "deterministic_rand_placement_generator", "placement_permute_generator",
    "permute_placement", "transition_trace", "placement_cost", "PlacementSolver",
    "search_placement", "placement_to_indices", "generate_rank_placement", "reorder_gate_rows",
    "adaptive_set_locality", "dump_trace", "dump_decision",
]


# ----------------------------------------------------------------------------- enumeration
def sorted_k_even_partitions(seq: Sequence[int], k: int, length: int) -> List[List[Tuple]]:
    """All ordered ways to split ``seq`` into ``k`` parts of at most ``length`` items, parts in
    shortlex order inside a partition, then every ordering of the parts (the reference's
    enumeration, placement.py:25-80)."""
    n = len(seq)
    groups: List[List[int]] = []

    def generate(i):
        if i >= n:
            yield [tuple(g) for g in groups]
            return
        if n - i > (k - len(groups)) * length:
            for g in groups:
                if len(g) < length:
                    g.append(seq[i])
                    yield from generate(i + 1)
                    g.pop()
        if len(groups) < k:
            groups.append([seq[i]])
            yield from generate(i + 1)
            groups.pop()

    parts = [sorted(ps, key=lambda p: (len(p), p)) for ps in generate(0)]
    parts.sort(key=lambda ps: (*map(len, ps), ps))
    ordered = []
    for partition in parts:
        ordered.extend([list(p) for p in itertools.permutations(partition)])
    return ordered


def possible_placement_generator(expert_num: int, world_size: int):
    assert expert_num % world_size == 0
    return sorted_k_even_partitions(list(range(expert_num)), world_size,
                                    expert_num // world_size)


def deterministic_rand_placement_generator(expert_num: int, world_size: int,
                                           seed: int = 0) -> Iterator[List[List[int]]]:
    """Distinct random balanced placements, the same sequence for the same seed."""
    assert expert_num % world_size == 0
    rng = np.random.RandomState(seed)
    used = set()
    while True:
        parts = np.split(rng.permutation(expert_num), world_size)
        placement = [sorted(int(e) for e in p) for p in parts]
        key = tuple(tuple(p) for p in placement)
        if key in used:
            continue
        used.add(key)
        yield placement


def placement_permute_generator(placement: List[List[int]]) -> Iterator[np.ndarray]:
    """Distinct orderings of the ranks of one placement."""
    rng = np.random.RandomState(0)
    used = set()
    limit = 1
    for i in range(2, len(placement) + 1):
        limit *= i
    while len(used) < limit:
        permuted = rng.permutation(np.asarray(placement))
        key = tuple(tuple(p) for p in permuted)
        if key in used:
            continue
        used.add(key)
        yield permuted


def permute_placement(placement: List[List[int]], seed: int = 0) -> np.ndarray:
    return np.random.RandomState(seed).permutation(np.asarray(placement))


# ----------------------------------------------------------------------------- statistics
def transition_trace(decision_histories: Sequence[Sequence[np.ndarray]]) -> List[np.ndarray]:
    """``decision_histories[i][p]`` holds the tags of the cells that router i sent down its path
    p (a fabric's ``cell_decision_history``).  Returns, for every pair of consecutive routers,
    the matrix of cells they share: trace[i][p, q] = |cells(i, p) & cells(i + 1, q)|."""
    trace = []
    for cur, nxt in zip(decision_histories[:-1], decision_histories[1:]):
        top = 1 + max([int(np.max(c)) for c in list(cur) + list(nxt) if len(c)] + [0])
        owner = np.zeros((len(nxt), top), dtype=np.int64)
        for q, cells in enumerate(nxt):
            np.add.at(owner[q], np.asarray(cells, dtype=np.int64), 1)
        m = np.zeros((len(cur), len(nxt)), dtype=np.int64)
        for p, cells in enumerate(cur):
            if len(cells):
                m[p] = owner[:, np.asarray(cells, dtype=np.int64)].sum(axis=1)
        trace.append(m)
    return trace


def _rank_of(placement: Sequence[Sequence[int]], expert_num: int) -> np.ndarray:
    rank = np.full(expert_num, -1, dtype=np.int64)
    for r, experts in enumerate(placement):
        rank[list(experts)] = r
    assert (rank >= 0).all(), "every expert needs a rank"
    return rank


def placement_cost(placements: Sequence[Sequence[Sequence[int]]],
                   trace: Sequence[np.ndarray]) -> int:
    """Cells that change rank between consecutive layers under ``placements`` (one placement
    = list of expert lists per rank, per layer)."""
    total = 0
    for i, m in enumerate(trace):
        a = _rank_of(placements[i], m.shape[0])
        b = _rank_of(placements[i + 1], m.shape[1])
        total += int(m[a[:, None] != b[None, :]].sum())
    return total


# ----------------------------------------------------------------------------- search
class PlacementSolver:
    """Balanced placement of every layer's experts on ``nodes`` ranks that keeps consecutive
    experts of a cell on one rank (objective and constraints of
    benchmark/swin_moe/placement_cvxpy.py:45-76; ``least_path_per_node`` is implied by the
    balance).  ``solve`` returns the placements and keeps the cost in ``self.cost``."""

    def __init__(self, nodes: int, scatter_trace: Sequence[np.ndarray], restarts: int = 8,
                 seed: int = 0, fix_first_layer: bool = False):
        self.nodes = nodes
        self.trace = [np.asarray(m, dtype=np.int64) for m in scatter_trace]
        self.path_nums = [self.trace[0].shape[0]] + [m.shape[1] for m in self.trace]
        for i, m in enumerate(self.trace):
            assert m.shape[0] == self.path_nums[i], "trace matrices do not chain"
        for n in self.path_nums:
            assert n % nodes == 0, "every layer's experts must split evenly over the ranks"
        self.restarts = restarts
        self.seed = seed
        self.fix_first_layer = fix_first_layer
        self.cost = None
        self.placements = None

    # rank vectors <-> placements
    def _to_placements(self, ranks):
        return [[sorted(int(e) for e in np.nonzero(r == node)[0]) for node in range(self.nodes)]
                for r in ranks]

    def _cost(self, ranks) -> int:
        return sum(int(m[ranks[i][:, None] != ranks[i + 1][None, :]].sum())
                   for i, m in enumerate(self.trace))

    def _affinity(self, ranks, layer) -> np.ndarray:
        """aff[e, node] = cells of expert e of ``layer`` whose neighbour-layer expert sits on
        ``node`` (both neighbours)."""
        n = self.path_nums[layer]
        aff = np.zeros((n, self.nodes), dtype=np.int64)
        if layer > 0:
            m = self.trace[layer - 1]  # [prev, this]
            for node in range(self.nodes):
                aff[:, node] += m[ranks[layer - 1] == node].sum(axis=0)
        if layer + 1 < len(self.path_nums):
            m = self.trace[layer]  # [this, next]
            for node in range(self.nodes):
                aff[:, node] += m[:, ranks[layer + 1] == node].sum(axis=1)
        return aff

    def _assign_layer(self, aff: np.ndarray) -> np.ndarray:
        """Balanced assignment that greedily takes the largest affinities first."""
        n = aff.shape[0]
        room = np.full(self.nodes, n // self.nodes)
        rank = np.full(n, -1, dtype=np.int64)
        order = np.dstack(np.unravel_index(np.argsort(-aff, axis=None, kind="stable"),
                                           aff.shape))[0]
        for e, node in order:
            if rank[e] < 0 and room[node] > 0:
                rank[e] = node
                room[node] -= 1
        return rank

    def _descend(self, ranks) -> None:
        """Pairwise swaps inside a layer while any of them lowers the cost."""
        first = 1 if self.fix_first_layer else 0
        improved = True
        while improved:
            improved = False
            for layer in range(first, len(ranks)):
                aff = self._affinity(ranks, layer)
                r = ranks[layer]
                n = len(r)
                # gain of swapping e and f (different ranks): both move to the other's rank
                stay = aff[np.arange(n), r]
                gain = (aff[:, r].T - stay[None, :]) + (aff[:, r] - stay[:, None])
                gain[r[:, None] == r[None, :]] = 0
                e, f = np.unravel_index(int(np.argmax(gain)), gain.shape)
                if gain[e, f] > 0:
                    r[e], r[f] = r[f], r[e]
                    improved = True

    def _solve_exhaustive(self):
        choices = []
        for layer, n in enumerate(self.path_nums):
            if layer == 0 and self.fix_first_layer:
                options = [np.repeat(np.arange(self.nodes), n // self.nodes)]
            else:
                options = [_rank_of(p, n) for p in possible_placement_generator(n, self.nodes)]
            choices.append(options)
        best, best_cost = None, None
        for combo in itertools.product(*choices):
            c = self._cost(combo)
            if best_cost is None or c < best_cost:
                best, best_cost = [x.copy() for x in combo], c
        return best, best_cost

    def solve(self, exhaustive_below: int = 20000):
        space = 1
        for n in self.path_nums:
            per = n // self.nodes
            ways = 1
            left = n
            for _ in range(self.nodes):
                ways *= _binom(left, per)
                left -= per
            space *= ways
            if space > exhaustive_below:
                break
        if space <= exhaustive_below:
            ranks, cost = self._solve_exhaustive()
        else:
            rng = np.random.RandomState(self.seed)
            ranks, cost = None, None
            for attempt in range(self.restarts):
                trial = []
                for layer, n in enumerate(self.path_nums):
                    if layer == 0:
                        r0 = np.repeat(np.arange(self.nodes), n // self.nodes)
                        trial.append(r0 if (attempt == 0 or self.fix_first_layer)
                                     else rng.permutation(r0))
                    else:
                        trial.append(np.zeros(n, dtype=np.int64))
                        only_prev = np.zeros((n, self.nodes), dtype=np.int64)
                        m = self.trace[layer - 1]
                        for node in range(self.nodes):
                            only_prev[:, node] = m[trial[layer - 1] == node].sum(axis=0)
                        trial[layer] = self._assign_layer(only_prev)
                self._descend(trial)
                c = self._cost(trial)
                if cost is None or c < cost:
                    ranks, cost = [t.copy() for t in trial], c
        self.cost = cost
        self.placements = self._to_placements(ranks)
        return self.placements


def _binom(n: int, k: int) -> int:
    out = 1
    for i in range(k):
        out = out * (n - i) // (i + 1)
    return out


def search_placement(decision_histories: Sequence[Sequence[np.ndarray]], world_size: int,
                     **solver_kwargs):
    """From the captured decisions of consecutive scatter routers to (placements, cost, cost of
    the default block placement)."""
    trace = transition_trace(decision_histories)
    solver = PlacementSolver(world_size, trace, **solver_kwargs)
    placements = solver.solve()
    default = [[list(range(r * (n // world_size), (r + 1) * (n // world_size)))
                for r in range(world_size)] for n in solver.path_nums]
    return placements, solver.cost, placement_cost(default, trace)


# ----------------------------------------------------------------------------- applying it
def load_balanced_placement(expert_loads: Sequence[float], world_size: int) -> List[List[int]]:
    """Experts dealt to ranks so that every rank hosts about the same load: most loaded expert
    first, each to the rank with the smallest load so far that still has room (every rank
    takes ``E / world_size`` experts); experts of a rank in ascending order.  Not in the
    reference, whose search (python/brt/runtime/placement.py:139-357) minimises the cells that
    change ranks between two layers; this one evens out what the ranks RECEIVE in one layer,
    which is what bounds the expert-parallel exchange when some experts are popular.  The
    result has the form the other helpers take (``placement_to_indices``,
    ``reorder_gate_rows``)."""
    E = len(expert_loads)
    if world_size < 1 or E % world_size != 0:
        raise ValueError("the experts must divide evenly over the ranks")
    per_rank = E // world_size
    bins: List[List[int]] = [[] for _ in range(world_size)]
    sums = [0.0] * world_size
    for e in sorted(range(E), key=lambda i: (-float(expert_loads[i]), i)):
        r = min((i for i in range(world_size) if len(bins[i]) < per_rank),
                key=lambda i: (sums[i], i))
        bins[r].append(e)
        sums[r] += float(expert_loads[e])
    return [sorted(b) for b in bins]


def placement_to_indices(placement: Sequence[Sequence[int]]) -> torch.Tensor:
    """Expert ids in the order the ranks host them (rank 0's experts, then rank 1's, ...): row
    i of a gate reordered with it scores the expert that now has global index i."""
    return torch.tensor(list(itertools.chain.from_iterable(placement)), dtype=torch.int64)


def generate_rank_placement(world_rank: int, world_size: int,
                            placements: Dict[Tuple, Sequence[Sequence[int]]] = None,
                            expert_keys: Sequence[Tuple] = (), global_expert_num: int = None):
    """Per expert key: the experts this rank hosts and the gate-row permutation.  Without
    ``placements`` every key gets the default block placement of ``global_expert_num`` experts
    (placement.py:200-236 of the reference, with the layer keys supplied by the caller instead
    of the Swin-MoE table)."""
    rank_placement, indices = {}, {}
    if placements is None:
        assert global_expert_num is not None and global_expert_num % world_size == 0
        per = global_expert_num // world_size
        block = [list(range(r * per, (r + 1) * per)) for r in range(world_size)]
        placements = {k: block for k in expert_keys}
    for key, placement in placements.items():
        rank_placement[key] = [int(e) for e in placement[world_rank]]
        indices[key] = placement_to_indices(placement)
    return list(placements.keys()), rank_placement, indices


def reorder_gate_rows(gate_weight: torch.Tensor, placement: Sequence[Sequence[int]]):
    """The gate's [experts, features] weight with its rows moved along with the experts."""
    return torch.index_select(gate_weight, 0, placement_to_indices(placement).to(
        gate_weight.device))


def adaptive_set_locality(model: nn.Module, locality_enabled_router: Dict[str, List[str]]):
    """Switch ``fabric.locality_aware`` on for the named scatter / gather routers
    (placement.py:326-345 of the reference; routers are named by module path here)."""
    from ..router import is_router

    for name, m in model.named_modules():
        if not is_router(m):
            continue
        kind = getattr(m, "_router_type", "")
        for side in ("scatter", "gather"):
            if side in kind and name in locality_enabled_router.get(side, []):
                m.fabric.locality_aware = True


def _scatter_fabrics(mod: nn.Module):
    from ..router import is_router

    return [m.fabric for _n, m in mod.named_modules()
            if is_router(m) and "scatter" in getattr(m, "_router_type", "")]


def dump_trace(mod: nn.Module, path: str = "scatter_results.npy"):
    """Captured load history of every scatter router (placement.py:83-88)."""
    np.save(path, np.array([np.array(f.load_history, dtype=object)
                            for f in _scatter_fabrics(mod)], dtype=object), allow_pickle=True)


def dump_decision(mod: nn.Module, path: str = "scatter_results.npy"):
    """Captured cell decisions of every scatter router (placement.py:91-99)."""
    np.save(path, np.array([np.array(f.cell_decision_history, dtype=object)
                            for f in _scatter_fabrics(mod)], dtype=object), allow_pickle=True)
