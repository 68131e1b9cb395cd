"""Expert placement search (CPU): enumeration helpers, the transition statistics and the
search itself against exhaustive enumeration on small problems."""
import itertools

import numpy as np
import pytest
import torch

from brainstorm_b200.runtime import placement as P


def test_enumeration_matches_the_counting_argument():
    # 4 experts on 2 ranks, 2 each: 3 unordered splits x 2 orderings
    got = P.possible_placement_generator(4, 2)
    assert len(got) == 6
    assert all(sorted(e for part in p for e in part) == [0, 1, 2, 3] for p in got)
    assert all(len(part) == 2 for p in got for part in p)
    assert len({tuple(map(tuple, p)) for p in got}) == 6
    # 6 experts on 3 ranks: 15 unordered splits x 3! orderings
    assert len(P.possible_placement_generator(6, 3)) == 90


def test_random_generators_are_deterministic_and_distinct():
    a = list(itertools.islice(P.deterministic_rand_placement_generator(8, 4, seed=3), 20))
    b = list(itertools.islice(P.deterministic_rand_placement_generator(8, 4, seed=3), 20))
    assert a == b
    assert len({tuple(map(tuple, p)) for p in a}) == 20
    for p in a:
        assert sorted(e for part in p for e in part) == list(range(8))
        assert all(part == sorted(part) and len(part) == 2 for part in p)
    perms = list(P.placement_permute_generator([[0, 1], [2, 3], [4, 5]]))
    assert len(perms) == 6 and len({tuple(map(tuple, p)) for p in perms}) == 6
    assert np.array_equal(P.permute_placement([[0, 1], [2, 3]], 1),
                          P.permute_placement([[0, 1], [2, 3]], 1))


def _histories(rng, layers, experts, cells, sticky):
    """Cells walk through the layers; with probability ``sticky`` a cell's next expert is tied
    to its current one by a hidden pairing, else it is random."""
    pair = [rng.permutation(experts) for _ in range(layers - 1)]
    choice = np.zeros((layers, cells), dtype=np.int64)
    choice[0] = rng.integers(0, experts, size=cells)
    for i in range(1, layers):
        tied = pair[i - 1][choice[i - 1]]
        free = rng.integers(0, experts, size=cells)
        choice[i] = np.where(rng.random(cells) < sticky, tied, free)
    tags = np.arange(1, cells + 1)
    return [[tags[choice[i] == e] for e in range(experts)] for i in range(layers)], choice


def test_transition_trace_counts_shared_cells():
    rng = np.random.default_rng(0)
    hist, choice = _histories(rng, 3, 4, 500, 0.5)
    trace = P.transition_trace(hist)
    assert len(trace) == 2
    for i, m in enumerate(trace):
        want = np.zeros((4, 4), dtype=np.int64)
        np.add.at(want, (choice[i], choice[i + 1]), 1)
        assert np.array_equal(m, want)
        assert m.sum() == 500


def test_search_is_optimal_on_small_problems():
    rng = np.random.default_rng(1)
    for layers, experts, world in ((2, 4, 2), (3, 4, 2), (2, 6, 3), (2, 6, 2)):
        hist, _ = _histories(rng, layers, experts, 400, 0.7)
        trace = P.transition_trace(hist)
        best = None
        options = P.possible_placement_generator(experts, world)
        for combo in itertools.product(options, repeat=layers):
            c = P.placement_cost(combo, trace)
            best = c if best is None else min(best, c)
        solver = P.PlacementSolver(world, trace)
        found = solver.solve()
        assert solver.cost == P.placement_cost(found, trace) == best
        # the descent (forced) may not beat the optimum and must stay balanced
        heur = P.PlacementSolver(world, trace, restarts=6)
        placements = heur.solve(exhaustive_below=0)
        assert heur.cost == P.placement_cost(placements, trace) >= best
        assert heur.cost <= 1.15 * best + 5
        for layer in placements:
            assert sorted(e for part in layer for e in part) == list(range(experts))
            assert all(len(part) == experts // world for part in layer)


def test_search_recovers_a_hidden_pairing_at_scale():
    """32 experts, 8 ranks, 4 layers: cells follow a hidden expert pairing 90 % of the time, so
    a good placement keeps most cells on their rank; the block placement keeps ~1/8."""
    rng = np.random.default_rng(2)
    hist, _ = _histories(rng, 4, 32, 20000, 0.9)
    placements, cost, default_cost = P.search_placement(hist, 8, restarts=4)
    moves = 3 * 20000
    assert default_cost > 0.8 * moves
    assert cost < 0.25 * moves
    assert cost == P.placement_cost(placements, P.transition_trace(hist))


def test_gate_rows_follow_the_experts():
    placement = [[2, 5], [0, 3], [1, 4]]
    idx = P.placement_to_indices(placement)
    assert idx.tolist() == [2, 5, 0, 3, 1, 4]
    w = torch.arange(6, dtype=torch.float32)[:, None] * torch.ones(1, 3)
    assert P.reorder_gate_rows(w, placement)[:, 0].tolist() == [2, 5, 0, 3, 1, 4]
    keys, mine, indices = P.generate_rank_placement(1, 3, {("l", 0): placement})
    assert keys == [("l", 0)] and mine[("l", 0)] == [0, 3]
    assert indices[("l", 0)].tolist() == idx.tolist()
    keys, mine, indices = P.generate_rank_placement(2, 4, expert_keys=[(2, 1), (2, 3)],
                                                    global_expert_num=8)
    assert mine[(2, 3)] == [4, 5] and indices[(2, 1)].tolist() == list(range(8))


def test_load_balanced_placement_evens_out_the_ranks():
    from brainstorm_b200.runtime.placement import load_balanced_placement

    rng = np.random.default_rng(5)
    for world, per_rank in ((2, 16), (4, 8), (8, 4), (8, 16)):
        loads = np.exp(rng.standard_normal(world * per_rank))      # a few popular experts
        placement = load_balanced_placement(loads.tolist(), world)
        assert sorted(e for hosted in placement for e in hosted) == list(range(world * per_rank))
        assert all(len(hosted) == per_rank and hosted == sorted(hosted) for hosted in placement)
        balanced = max(sum(loads[e] for e in hosted) for hosted in placement)
        block = max(loads[r * per_rank:(r + 1) * per_rank].sum() for r in range(world))
        mean = loads.sum() / world
        assert balanced <= block + 1e-9
        assert balanced <= 1.25 * mean, (world, per_rank, balanced / mean)
    with pytest.raises(ValueError):
        load_balanced_placement([1.0, 2.0, 3.0], 2)
    # ties are broken by index, so every rank computes the same placement
    assert load_balanced_placement([1.0] * 8, 4) == [[0, 4], [1, 5], [2, 6], [3, 7]]
