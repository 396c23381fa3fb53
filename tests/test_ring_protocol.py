"""The barrier protocol of the persistent decode attention kernels
(csrc/attn_decode_mma.cu, csrc/attn_decode_stream.cu), simulated on the host with
mbarrier semantics: a barrier completes a phase when its arrivals and its bytes
are in, and a wait names the PARITY of the phase it waits for.

Three stages, two pairs of warps; item n goes to stage n % 3 and to pair n % 2,
so a pair meets a stage every sixth item.  With one set of barriers per stage a
pair's wait lies two phases after its last one on that barrier, which a parity
cannot tell from none: the protocol then holds only while copies complete in the
order of their issue.  With barriers per (stage, pair) it holds under any order.
The simulation runs the producer and the four compute warps under random
interleavings and lets copies complete within a window of the oldest ones."""
import random

import pytest

STAGES, GROUPS, PAGES = 3, 2, 2


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


def simulate(chunks, seed, window, per_pair):
    """chunks[g]: how many chunks pair g consumes.  Raises AssertionError when a warp
    reads a tile that is not its own, a barrier gets too many arrivals, or nothing moves."""
    rnd = random.Random(seed)
    dims = GROUPS if per_pair else 1
    mk = lambda c: [[Barrier(c) for _ in range(dims)] for _ in range(STAGES)]
    full_k, full_v, empty = mk(1), mk(1), mk(PAGES)
    col = (lambda g: g) if per_pair else (lambda g: 0)
    content = [dict() for _ in range(STAGES)]
    inflight = []

    def producer():
        left, k, last = list(chunks), [0, 0], [None] * STAGES
        n = 0
        while left[0] > 0 or left[1] > 0:
            g, s = n % GROUPS, n % STAGES
            if per_pair:
                if left[g] > 0:
                    if last[s] is not None:
                        lg, lm = last[s]
                        while not empty[s][lg].done(lm & 1):
                            yield
                    last[s] = (g, n // (STAGES * GROUPS))
            else:
                rd = n // STAGES
                while not empty[s][0].done((rd & 1) ^ 1):
                    yield
                if left[g] == 0:            # the pair has run out: the item passes through empty
                    full_k[s][0].arrive()
                    full_v[s][0].arrive()
                    for _ in range(PAGES):
                        empty[s][0].arrive()
            if left[g] > 0:
                full_k[s][col(g)].arrive(tx=1)
                inflight.append((full_k[s][col(g)], s, "k", (g, k[g])))
                full_v[s][col(g)].arrive(tx=1)
                inflight.append((full_v[s][col(g)], s, "v", (g, k[g])))
                k[g] += 1
                left[g] -= 1
            n += 1
            yield

    def warp(g, sync):
        for k in range(chunks[g]):
            n = GROUPS * k + g
            s = n % STAGES
            parity = ((n // (STAGES * GROUPS)) if per_pair else (n // STAGES)) & 1
            while not full_k[s][col(g)].done(parity):
                yield
            assert content[s].get("k") == (g, k), f"pair {g} chunk {k} finds keys {content[s].get('k')}"
            yield
            while not full_v[s][col(g)].done(parity):
                yield
            assert content[s].get("v") == (g, k), f"pair {g} chunk {k} finds values {content[s].get('v')}"
            yield
            empty[s][col(g)].arrive()
            sync[0] += 1                    # the pair's named barrier
            while sync[0] < (k + 1) * PAGES:
                yield

    syncs = [[0], [0]]
    threads = [producer()] + [warp(g, syncs[g]) for g in range(GROUPS) for _ in range(PAGES)]
    alive, idle = list(range(len(threads))), 0
    while alive:
        if inflight and rnd.random() < 0.3:
            bar, s, what, tag = inflight.pop(rnd.randrange(min(len(inflight), window)))
            content[s] = dict(content[s])
            content[s][what] = tag
            bar.complete_tx(1)
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
        assert idle < 100000 or inflight, "nothing moves"


CASES = [(26, 26), (26, 13), (13, 0), (10, 5), (5, 0), (1, 1), (3, 40), (0, 7)]


@pytest.mark.parametrize("chunks", CASES)
def test_barriers_per_stage_and_pair_hold_under_any_order_of_copies(chunks):
    for seed in range(40):
        simulate(chunks, seed, window=1000, per_pair=True)


@pytest.mark.parametrize("chunks", CASES)
def test_shared_barriers_hold_while_copies_complete_in_order(chunks):
    for seed in range(25):
        simulate(chunks, seed, window=1, per_pair=False)


def test_shared_barriers_break_when_copies_may_overtake_each_other():
    bad = 0
    for seed in range(150):
        try:
            simulate((26, 26), seed, window=4, per_pair=False)
        except AssertionError:
            bad += 1
    assert bad > 0, "a wait two phases after the last one cannot be told from none"


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
