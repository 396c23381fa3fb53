"""A model of the barrier protocol of the tcgen05 prompt attention (csrc/attn_prompt_tc.cu),
run on the host with mbarrier semantics: a barrier completes a phase when its arrivals and
its bytes are in, and a wait names the PARITY of the phase it waits for, so a barrier that is
two phases on cannot be told from one that has not moved.  This is reasoning kept runnable, not
a test of the kernel: the kernel itself is held against the plain attention in
tests/test_gpu_kernels.py."""
import random

import pytest


class Barrier:
    def __init__(self, count):
        self.count, self.pending, self.tx, self.phase = count, count, 0, 0

    def arrive(self, tx=0):
        self.tx += tx
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects"
        self._check()

    def complete_tx(self, n):
        self.tx -= n
        self._check()

    def _check(self):
        if self.pending == 0 and self.tx == 0:
            self.phase ^= 1
            self.pending = self.count

    def done(self, parity):                 # mbarrier.try_wait.parity
        return self.phase != parity


# ---------------------------------------------------------------------------
# The ring of the tcgen05 prompt attention (csrc/attn_prompt_tc.cu): a producer (keys and
# values of block j into one of six tiles), an issuing thread (scores of up to three blocks
# ahead, then P V block by block) and the softmax warps.  The producer may fetch the values of
# block j only when the product of block j - 3 has read its tile.  If it learns that from the
# barrier that alternate blocks share (pv_done[j & 1]), the barrier can be two phases on by
# the time a late producer looks, once the last scores are issued and nothing holds the last
# products back; with a barrier per tile (v_free[j % 3]) the next phase always needs the tile
# that the producer fetches after its wait.
def simulate_prompt_ring(n_blk, seed, per_tile, producer_lag):
    rnd = random.Random(seed)
    NBUF = 3
    full = [Barrier(1) for _ in range(6)]
    s_full, p_full = [Barrier(1) for _ in range(NBUF)], [Barrier(1) for _ in range(NBUF)]
    pv_done, v_free = [Barrier(1) for _ in range(2)], [Barrier(1) for _ in range(NBUF)]
    tiles = [None] * 6
    inflight = []                                             # tensor-core work and copies complete later, in order

    def producer():
        for i in range(2 * n_blk):
            slot, j, is_v = i % 6, i >> 1, i & 1
            for _ in range(producer_lag if i == 2 * n_blk - 1 else 0):
                yield                                         # the producer is late for the last tile
            if j >= NBUF:
                jp = j - NBUF
                if is_v:
                    bar, par = (v_free[jp % NBUF], (jp // NBUF) & 1) if per_tile else (pv_done[jp & 1], (jp >> 1) & 1)
                else:
                    bar, par = s_full[jp % NBUF], (jp // NBUF) & 1
                while not bar.done(par):
                    yield
            full[slot].arrive(tx=1)
            inflight.append(("copy", slot, (j, is_v)))
            yield

    def issuer():
        def issue_s(j):
            i = 2 * j
            while not full[i % 6].done((i // 6) & 1):
                yield
            assert tiles[i % 6] == (j, 0), f"scores of block {j} read tile {tiles[i % 6]}"
            inflight.append(("mma", [s_full[j % NBUF]], None))
        for j in range(min(NBUF, n_blk)):
            yield from issue_s(j)
        for j in range(n_blk):
            i = 2 * j + 1
            while not (p_full[j % NBUF].done((j // NBUF) & 1) and full[i % 6].done((i // 6) & 1)):
                yield
            assert tiles[i % 6] == (j, 1), f"product of block {j} read tile {tiles[i % 6]}"
            inflight.append(("mma", [pv_done[j & 1], v_free[j % NBUF]], None))
            if j + NBUF < n_blk:
                while not pv_done[j & 1].done((j >> 1) & 1):
                    yield
                yield from issue_s(j + NBUF)
            yield

    def softmax():
        for j in range(n_blk):
            while not s_full[j % NBUF].done((j // NBUF) & 1):
                yield
            yield
            p_full[j % NBUF].arrive()
        for j in (n_blk - 2, n_blk - 1):
            if j >= 0:
                while not pv_done[j & 1].done((j >> 1) & 1):
                    yield

    threads = [producer(), issuer(), softmax()]
    alive, idle = [0, 1, 2], 0
    while alive:
        if inflight and rnd.random() < 0.4:
            kind, a, b = inflight.pop(0)
            if kind == "copy":
                tiles[a] = b
                full[a].complete_tx(1)
            else:
                for bar in a:
                    bar.arrive()
            idle = 0
            continue
        t = rnd.choice(alive)
        try:
            next(threads[t])
        except StopIteration:
            alive.remove(t)
            idle = 0
            continue
        idle += 1
        assert idle < 20000 or inflight, "nothing moves"


@pytest.mark.parametrize("n_blk", [1, 2, 3, 4, 5, 6, 7, 16, 33])
def test_prompt_attention_ring_with_a_barrier_per_value_tile_always_finishes(n_blk):
    for seed in range(30):
        for lag in (0, 50, 3000):
            simulate_prompt_ring(n_blk, seed, per_tile=True, producer_lag=lag)


def test_prompt_attention_ring_on_the_shared_product_barrier_can_stall_a_late_producer():
    stalled = 0
    for seed in range(30):
        try:
            simulate_prompt_ring(9, seed, per_tile=False, producer_lag=3000)
        except AssertionError:
            stalled += 1
    assert stalled > 0
