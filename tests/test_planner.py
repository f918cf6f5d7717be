"""Residency planner (b200moe_planner_*, host code only): the moves, tables and receipt of scripted traces equal the
reference's own Planner (include/strix/residency/expert_residency.hpp:102-147) - run here through oracle/_ref where the
reference checkout is present, through tests/golden/planner_golden.npz elsewhere - plus the properties the rule promises."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "planner_golden.npz")

# (layers, experts, top_k, slots, expert bytes per layer, decay, margin, budget, steps, ids per layer and step, seeded, zipf skew)
CASES = [
    (1, 16, 2, 6, [1000], 0.97, 1.5, 64 << 20, 40, 8, False, 1.1),
    (3, 32, 4, 8, [4096, 1000, 70000], 0.9, 0.5, 150000, 60, 16, True, 1.3),
    (2, 64, 8, 80, [100, 200], 0.97, 1.5, 250, 30, 32, False, 0.0),    # more slots than experts: everything fits in time, 250 bytes per step
    (2, 24, 2, 5, [5000, 9000], 0.5, 0.1, 6000, 50, 4, False, 2.0),     # one layer's expert is larger than the whole budget
]


def trace_of(case, seed):
    layers, experts, top_k, slots, eb, decay, margin, budget, steps, n, seeded, skew = case
    rng = np.random.default_rng(seed)
    p = 1.0 / np.arange(1, experts + 1) ** skew
    p /= p.sum()
    perm = [rng.permutation(experts) for _ in range(layers)]
    ids = np.zeros((steps, layers, n), np.uint32)
    for s in range(steps):
        drift = s // 15          # the popular experts change over time
        for l in range(layers):
            ids[s, l] = np.roll(perm[l], 3 * drift)[rng.choice(experts, size=n, p=p)]
    ids[steps // 2, 0, 0] = experts + 5   # an id out of range is ignored
    seed_counts = rng.integers(0, 50, size=(layers, experts)).astype(np.uint32) if seeded else None
    return ids, seed_counts


def run_library(case, ids, seed_counts):
    from b200moe.residency import Planner
    layers, experts, top_k, slots, eb, decay, margin, budget, steps, n, seeded, _ = case
    pl = Planner(layers, experts, top_k, slots, eb, decay, margin, budget)
    if seed_counts is not None:
        for l in range(layers):
            pl.seed(l, seed_counts[l])
        pl.fill_from_seed()
    per_step = []
    for s in range(steps):
        for l in range(layers):
            pl.observe(l, ids[s, l])
        pl.end_step()
        first, moves = pl.plan(), pl.plan()
        assert first == moves                      # plan() does not change the state
        for m in moves:
            pl.commit(m)
        per_step.append(moves)
    tables = np.stack([pl.table(l) for l in range(layers)])
    return per_step, tables, pl.receipt(), pl


@pytest.mark.parametrize("k", range(len(CASES)))
def test_planner_equals_the_reference(k):
    from oracle.loader import Ref
    case = CASES[k]
    ids, seed_counts = trace_of(case, 100 + k)
    got_moves, got_tables, got_receipt, pl = run_library(case, ids, seed_counts)
    layers, experts, top_k, slots, eb, decay, margin, budget, steps, n, seeded, _ = case
    if Ref.available():
        want_moves, want_tables, want_receipt = Ref().planner_trace(layers, experts, top_k, slots, eb, decay, margin, budget, ids, seed_counts, fill=seeded)
        assert got_moves == want_moves
        assert np.array_equal(got_tables, want_tables) and got_receipt == want_receipt
    g = np.load(GOLDEN)
    flat = np.array([m for step in got_moves for m in step], np.uint32).reshape(-1, 4)
    assert np.array_equal(flat, g[f"moves_{k}"]) and np.array_equal(np.array([len(s) for s in got_moves]), g[f"counts_{k}"])
    assert np.array_equal(got_tables, g[f"tables_{k}"]) and np.array_equal(np.array(list(got_receipt.values()), np.uint64), g[f"receipt_{k}"])
    assert sum(len(s) for s in got_moves) > 0      # the trace exercises the rule
    # the rule's promises, checked on the library's own trace
    slots_eff = min(slots, experts)
    for s, moves in enumerate(got_moves):
        spent = sum(eb[m[0]] for m in moves)
        assert spent <= budget or (len(moves) == 1 and eb[moves[0][0]] > budget)
        used = [set(int(v) for v in ids[s, l] if v < experts) for l in range(layers)]
        for layer, slot, evict, expert in moves:
            assert slot < slots_eff and expert < experts
            assert evict == 0xFFFFFFFF or evict not in used[layer]   # an expert the step used is never evicted
    for l in range(layers):
        t = got_tables[l]
        res = t[t >= 0]
        assert len(res) == len(set(res.tolist())) and len(res) <= slots_eff


def test_planner_argument_errors():
    import ctypes as C
    import b200moe
    from b200moe.residency import Planner
    with pytest.raises(b200moe.B200MoeError):
        Planner(0, 8, 2, 4, [])
    with pytest.raises(b200moe.B200MoeError):
        Planner(1, 8, 2, 4, [100], decay=1.0)
    pl = Planner(1, 8, 2, 4, [100])
    with pytest.raises(b200moe.B200MoeError):
        pl.seed(1, np.zeros(8, np.uint32))
    with pytest.raises(b200moe.B200MoeError):
        pl.commit((0, 9, 0xFFFFFFFF, 1))
    pl.seed(0, np.zeros(8, np.uint32))           # an all-zero prior changes nothing
    assert not pl.scores(0).any() and pl.plan() == []
    # a caller's array that is too small still learns the count
    pl.observe(0, [0, 1, 2, 3, 4, 5])
    pl.end_step()
    n = C.c_uint32()
    b200moe.check(b200moe.lib().b200moe_planner_plan(pl.handle, None, 0, C.byref(n)))
    assert n.value == 4 and len(pl.plan()) == 4   # four free slots, six candidates
