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
