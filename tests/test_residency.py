"""Expert residency (include/b200moe.h, "Expert residency"): the eviction rule as a pure host function (CPU), and on the
GPU a layer with fewer slots than experts against the all-resident run, bit for bit."""
import numpy as np
import pytest

import b200moe
from b200moe import residency


@pytest.fixture(scope="module")
def gpu():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    b200moe.lib()  # fails loudly when the extension is missing
    return torch.device("cuda:0")


def test_choose_victims_policy():
    """Free slots ascending first; then slots whose expert the window does not use by (score, expert) ascending; an
    expert the window uses is never evicted (include/strix/residency/expert_residency.hpp:121-127)."""
    E = 8
    score = np.array([5.0, 1.0, 3.0, 1.0, 9.0, 0.5, 2.0, 7.0])
    slot_expert = np.array([4, -1, 1, 3, -1, 0], np.int32)     # slots 1 and 4 free
    used = np.zeros(E, np.uint8)
    used[[4, 6, 7, 2, 5]] = 1                                   # expert 4 is resident and in use
    v = residency.choose_victims(slot_expert, score, used, [2, 5, 6, 7])
    # free 1, 4; then experts 1 (score 1, slot 2) and 3 (score 1, slot 3): tie by expert id; expert 0 (score 5) is next
    assert v.tolist() == [1, 4, 2, 3]
    v = residency.choose_victims(slot_expert, score, used, [2, 5, 6, 7, 2])[:5]
    assert v.tolist() == [1, 4, 2, 3, 5]
    # expert 4 is in use: only five slots may be refilled
    with pytest.raises(b200moe.B200MoeError) as err:
        residency.choose_victims(slot_expert, score, used, [2, 5, 6, 7, 2, 5])
    assert err.value.code == 3
    assert residency.choose_victims(slot_expert, score, used, []).tolist() == []


def test_choose_victims_rejects_bad_table():
    with pytest.raises(b200moe.InvalidArgument):
        residency.choose_victims(np.array([9], np.int32), np.zeros(4), np.zeros(4, np.uint8), [1])


@pytest.mark.gpu
def test_residency_equals_all_resident(gpu, oracle):
    """16 experts, 6 slots: every window's output equals the CPU oracle's (experts + slot-order merge on the full tensors)
    and the all-resident layer's, bit for bit (FMA_SLOTS form), across misses, hits and evictions; an oversubscribed window
    is refused with the state unchanged; an id out of range stays invalid."""
    import torch
    from oracle import loader as O
    from b200moe import ops, synth
    rng = np.random.default_rng(61)
    E, S, H, I, K, rows = 16, 6, 512, 256, 2, 2
    for gt, dt in ((12, 12), (13, 7)):
        gate, up, down = synth.expert_tensors(rng, E, H, I, gt, dt)
        shape = ops.make_shape(H, I, E, K, gt, dt)
        hosts = [torch.from_numpy(a).pin_memory() for a in (gate, up, down)]
        res = residency.ExpertResidency(shape, *hosts, slots=S, device=gpu)
        full = ops.MoeLayer(shape, *(torch.from_numpy(a).to(gpu) for a in (gate, up, down)), rows, b200moe.COMBINE_FMA_SLOTS)
        part = ops.MoeLayer(res.slot_shape, res.gate, res.up, res.down, rows, b200moe.COMBINE_FMA_SLOTS)
        for step in range(14):
            pool = E if step % 3 else 5                     # some windows stay inside a hot set: hits
            ids = np.stack([rng.permutation(pool)[:K] for _ in range(rows)]).astype(np.int32)
            x = rng.standard_normal((rows, H), dtype=np.float32)
            w = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
            xa = ops.enqueue_quantize_a8(torch.from_numpy(x).to(gpu))
            ids_d, w_d = torch.from_numpy(ids).to(gpu), torch.from_numpy(w).to(gpu)
            slot_ids = res.map(ids_d)
            table = res.table()
            assert np.array_equal(slot_ids.cpu().numpy(), table[ids])
            y_full = full(xa, ids_d, w_d)
            y_part = part(xa, slot_ids, w_d)
            assert np.array_equal(y_full.cpu().numpy().view(np.uint32), y_part.cpu().numpy().view(np.uint32)), (gt, dt, step)
            codes, deltas, sums = oracle.quantize_a8(x)
            osh = O.Shape(H, I, E, K, gt, dt, float("inf"))
            raw = oracle.experts(osh, gate, up, down, ids.astype(np.uint32), codes, deltas, sums)["raw"]
            want = oracle.combine(O.COMBINE_FMA_SLOTS, raw, w, ids.astype(np.uint32))
            assert np.array_equal(y_part.cpu().numpy().view(np.uint32), want.view(np.uint32)), (gt, dt, step)
        st = res.stats()
        assert st["windows"] == 14 and st["misses"] > S and st["evictions"] > 0 and st["hits"] > 0
        assert (res.table() >= 0).sum() == S
        # more distinct experts than slots: refused, nothing changes
        before, stats_before = res.table().copy(), res.stats()
        with pytest.raises(b200moe.B200MoeError) as err:
            res.map(torch.arange(S + 1, dtype=torch.int32, device=gpu))
        assert err.value.code == 3 and np.array_equal(res.table(), before) and res.stats() == stats_before
        # an id out of range keeps an invalid slot id
        bad = torch.tensor([int(before.argmax()), E + 3], dtype=torch.int32, device=gpu)
        out = res.map(bad).cpu().numpy().view(np.uint32)
        assert out[1] == 0xFFFFFFFF and out[0] == before.max()
        res.close()


@pytest.mark.gpu
def test_planned_promotions_ahead_of_need(gpu, oracle):
    """The planner's moves applied by b200moe_residency_promote on a side stream: the initial residency comes from a seed,
    every step's moves stay inside the upload budget, the window after them equals the CPU oracle bit for bit, and windows
    inside the hot set stop missing once the promotions are in. Moves that contradict the table are refused unchanged."""
    import torch
    from oracle import loader as O
    from b200moe import ops, synth
    rng = np.random.default_rng(62)
    E, S, H, I, K, rows = 16, 6, 512, 256, 2, 2
    gate, up, down = synth.expert_tensors(rng, E, H, I, 12, 12)
    shape = ops.make_shape(H, I, E, K, 12, 12)
    expert_bytes = int(b200moe.lib().b200moe_expert_bytes(shape))
    hosts = [torch.from_numpy(a).pin_memory() for a in (gate, up, down)]
    res = residency.ExpertResidency(shape, *hosts, slots=S, device=gpu)
    part = ops.MoeLayer(res.slot_shape, res.gate, res.up, res.down, rows, b200moe.COMBINE_FMA_SLOTS)
    pl = residency.Planner(1, E, K, S, [expert_bytes], decay=0.5, margin_reuses=0.5, upload_bytes_per_step=2 * expert_bytes)
    prior = np.zeros(E, np.uint32)
    prior[[1, 2, 3, 4]] = (40, 30, 20, 10)
    pl.seed(0, prior)
    pl.fill_from_seed()
    side = torch.cuda.Stream(device=gpu)
    first = [(0, int(s), b200moe.MOVE_NO_EVICTION, int(e)) for e, s in enumerate(pl.table(0)) if s >= 0]
    res.promote(first, stream=side.cuda_stream)
    torch.cuda.current_stream().wait_stream(side)
    assert np.array_equal(res.table(), pl.table(0))
    late_misses, promoted = 0, 0
    for step in range(20):
        hot = np.array([1, 2, 3, 4, 5]) if step < 8 else np.array([8, 9, 10, 11, 12])   # the popular experts change
        ids = np.stack([rng.permutation(hot)[:K] for _ in range(rows)]).astype(np.int32)
        x = rng.standard_normal((rows, H), dtype=np.float32)
        w = rng.uniform(0.05, 0.6, size=(rows, K)).astype(np.float32)
        before = res.stats()["misses"]
        xa = ops.enqueue_quantize_a8(torch.from_numpy(x).to(gpu))
        ids_d, w_d = torch.from_numpy(ids).to(gpu), torch.from_numpy(w).to(gpu)
        y = part(xa, res.map(ids_d), w_d)
        if step >= 15:
            late_misses += res.stats()["misses"] - before
        codes, deltas, sums = oracle.quantize_a8(x)
        raw = oracle.experts(O.Shape(H, I, E, K, 12, 12, float("inf")), gate, up, down, ids.astype(np.uint32), codes, deltas, sums)["raw"]
        want = oracle.combine(O.COMBINE_FMA_SLOTS, raw, w, ids.astype(np.uint32))
        assert np.array_equal(y.cpu().numpy().view(np.uint32), want.view(np.uint32)), step
        # the planner sees the step, plans inside its budget; the copies run on the side stream, ordered before the next window.
        # Experts that the demand path loaded meanwhile are resident in the residency object but not in the planner's table:
        # the planner's table is brought in line first (its commit is the record of a copy that is in).
        pl.observe(0, ids)
        pl.end_step()
        table, mine = res.table(), pl.table(0)
        for e in range(E):
            if table[e] >= 0 and mine[e] != table[e]:
                holder = int(np.where(mine == table[e])[0][0]) if (mine == table[e]).any() else b200moe.MOVE_NO_EVICTION
                pl.commit((0, int(table[e]), holder, e))
                mine = pl.table(0)
        moves = pl.plan()
        assert len(moves) <= 2
        promoted += len(moves)
        side.wait_stream(torch.cuda.current_stream())
        res.promote(moves, stream=side.cuda_stream)
        for m in moves:
            pl.commit(m)
        torch.cuda.current_stream().wait_stream(side)
        assert np.array_equal(res.table(), pl.table(0))
    assert late_misses == 0 and promoted > 0      # the new hot set is resident by then, partly through planned promotions
    # contradicting moves: refused, nothing changes
    table = res.table().copy()
    resident, absent = int(np.argmax(table >= 0)), int(np.argmax(table < 0))
    for bad in ((0, int(table[resident]), b200moe.MOVE_NO_EVICTION, absent),       # the slot is not free
                (0, 0, int(np.where(table == 0)[0][0]), resident),                   # the expert is already resident
                (0, S, b200moe.MOVE_NO_EVICTION, absent)):                           # no such slot
        with pytest.raises(b200moe.InvalidArgument):
            res.promote([bad])
        assert np.array_equal(res.table(), table)
    res.close()
    pl.close()
