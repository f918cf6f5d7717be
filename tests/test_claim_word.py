"""The claim word of the segment-streaming kernels (csrc/wide_common.cuh: claim_item, retire_claims, and the first-item
rule of the producers in gemv_q4k_wide.cu / gemv_q8_wide.cu), replayed as state machines under random interleavings:
every item is taken exactly once, a launch with fewer items than groups keeps one group per CTA busy before any CTA
runs two, and the word is back at zero when the last CTA has retired - whatever the order of the atomic operations."""
import random

CLAIM_BITS = 22
MASK = (1 << CLAIM_BITS) - 1
GROUPS = 2


class Word:
    def __init__(self):
        self.v = 0

    def add(self, x):          # atomicAdd: returns the old value
        old = self.v
        self.v = (self.v + x) & 0xFFFFFFFF
        return old


def run(n_items, grid, rng):
    word = Word()
    taken = []
    retired_in_cta = [0] * grid
    # one state machine per producer warp: ("first" | "claim" | "retire" | "done")
    producers = [{"cta": b, "g": g, "state": "first"} for b in range(grid) for g in range(GROUPS)]
    live = list(producers)
    while live:
        p = rng.choice(live)
        if p["state"] == "first":                       # the group's own number: no atomic
            k = p["g"] * grid + p["cta"]
            if k < n_items:
                taken.append((k, p["cta"], p["g"]))
                p["state"] = "claim"
            else:
                p["state"] = "retire"
        elif p["state"] == "claim":
            k = grid * GROUPS + (word.add(1) & MASK)
            if k < n_items:
                taken.append((k, p["cta"], p["g"]))
            else:
                p["state"] = "retire"
        elif p["state"] == "retire":
            retired_in_cta[p["cta"]] += 1
            if retired_in_cta[p["cta"]] == GROUPS:      # the CTA's last producer publishes the CTA's retirement
                before = word.add(1 << CLAIM_BITS)
                if (before >> CLAIM_BITS) == grid - 1:
                    word.v = 0                          # atomicExch by the grid's last CTA
            p["state"] = "done"
            live.remove(p)
    return word.v, taken


def test_every_item_once_and_the_word_returns_to_zero():
    rng = random.Random(7)
    for n_items, grid in ((0, 5), (1, 148), (80, 148), (147, 148), (148, 148), (296, 148), (297, 148), (3520, 148), (17, 3), (1000, 7)):
        for _ in range(3):
            left, taken = run(n_items, grid, rng)
            assert left == 0, (n_items, grid)
            assert sorted(k for k, _, _ in taken) == list(range(n_items)), (n_items, grid)
            if n_items <= grid:                         # fewer items than CTAs: one group per CTA, group 0
                assert all(g == 0 for _, _, g in taken) and len({c for _, c, _ in taken}) == n_items
