"""An executable model of the streamed compaction kernel's protocol (dcb::compact_stream_body), run under random
schedules. Every role of a block - the loader thread, the offsets warp, each worker warp - is a coroutine that stops
wherever the kernel would wait; a scheduler picks any runnable one at random. The model keeps the kernel's barriers
exactly (arrival counts and phase parity per slot), so it catches what cannot be provoked on purpose on a GPU:

  * a wait that could never be satisfied (the schedule stops with work left) - for any number of resident blocks, down
    to one, because an id is drawn only by a running block and a tile waits only for tiles with smaller ids;
  * a barrier that runs a whole phase ahead of a waiter (parity would then read as "not complete" for ever);
  * a slot reused before its previous tile was written out;
  * offsets that differ from those of a sequential compaction.
"""
import random

import pytest


class MBar:
    """mbarrier: `count` arrivals complete the current phase; wait(parity) is true once the phase of that parity is over."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def test(self, parity):
        return (self.phase & 1) != parity


class Sim:
    def __init__(self, num_tiles, grid, resident, warps, lag, nbuf, seed, copy_warps=0):
        self.rng = random.Random(seed)
        self.num_tiles, self.grid, self.resident, self.W, self.lag, self.nbuf = num_tiles, grid, resident, warps, lag, nbuf
        self.CW = copy_warps                    # 0: every worker writes its own run; else that many warps only write
        self.counts = [[self.rng.randrange(0, 9) for _ in range(warps)] for _ in range(num_tiles)]
        self.desc = [None] * num_tiles          # published tile totals
        self.counter = 0
        self.copies = []                        # bulk copies in flight: (block, slot)
        self.written = {}                       # (tile, worker) -> output offset it was written at
        self.result = None

    # ---- one block
    def make_block(self, b):
        nb, W = self.nbuf, self.W
        blk = type("Blk", (), {})()
        blk.full = [MBar(1) for _ in range(nb)]
        blk.ranked = [MBar(W) for _ in range(nb)]
        blk.offs = [MBar(1) for _ in range(nb)]
        blk.empty = [MBar(self.CW or W) for _ in range(nb)]
        blk.tile = [None] * nb
        blk.cnt = [[None] * W for _ in range(nb)]
        blk.off = [[None] * W for _ in range(nb)]
        blk.busy = [False] * nb                 # slot holds a tile that has not been written out by every worker
        blk.agents = [self.loader(blk), self.offsets(blk)] + [self.worker(blk, w) for w in range(W)]
        blk.agents += [self.copier(blk, c) for c in range(self.CW)]
        return blk

    def loader(self, blk):
        st, ph, r = 0, 0, 0
        while True:
            t = min(self.counter, self.num_tiles)
            self.counter += 1
            if r >= self.nbuf:
                while not blk.empty[st].test(ph ^ 1):
                    yield
            assert not blk.busy[st], "slot reused before its tile was written out"
            blk.tile[st] = t
            if t < self.num_tiles:
                blk.busy[st] = True
                self.copies.append((blk, st))   # lands later, at a random moment
            else:
                blk.full[st].arrive()
                return
            r += 1
            st += 1
            if st == self.nbuf:
                st, ph = 0, ph ^ 1
            yield

    def offsets(self, blk):
        st, ph = 0, 0
        last_tile, run_incl, pending = -1, 0, None
        while True:
            while not blk.ranked[st].test(ph):
                yield
            tile = blk.tile[st]
            valid = tile < self.num_tiles
            if valid:
                cnt = list(blk.cnt[st])
                self.desc[tile] = sum(cnt)
            if pending is not None:
                p_tile, p_st, p_cnt = pending
                for i in range(last_tile + 1, p_tile):
                    while self.desc[i] is None:
                        yield
                exclusive = run_incl + sum(self.desc[last_tile + 1:p_tile])
                acc = exclusive
                for w in range(self.W):
                    blk.off[p_st][w] = acc
                    acc += p_cnt[w]
                if p_tile == self.num_tiles - 1:
                    self.result = acc
                blk.offs[p_st].arrive()
                run_incl, last_tile, pending = acc, p_tile, None
            if not valid:
                return
            pending = (tile, st, cnt)
            st += 1
            if st == self.nbuf:
                st, ph = 0, ph ^ 1
            yield

    def worker(self, blk, w):
        st = sj = ph = pj = 0
        nvalid = 1 << 62
        k = 0
        while k < nvalid + (0 if self.CW else self.lag):
            if k < nvalid:
                while not blk.full[st].test(ph):
                    yield
                tile = blk.tile[st]
                if tile >= self.num_tiles:
                    nvalid = k
                else:
                    blk.cnt[st][w] = self.counts[tile][w]
                blk.ranked[st].arrive()
                st += 1
                if st == self.nbuf:
                    st, ph = 0, ph ^ 1
                yield
            if not self.CW and k >= self.lag:
                if k - self.lag < nvalid:
                    while not blk.offs[sj].test(pj):
                        yield
                    tile = blk.tile[sj]
                    assert (tile, w) not in self.written
                    self.written[(tile, w)] = blk.off[sj][w]
                    blk.empty[sj].arrive()
                    if all(bar.pending == bar.count for bar in [blk.empty[sj]]):
                        blk.busy[sj] = False      # the last worker's arrival completed the phase
                sj += 1
                if sj == self.nbuf:
                    sj, pj = 0, pj ^ 1
            k += 1
            yield

    def copier(self, blk, c):
        """A warp that only writes: the round's tile id comes from the slot's `full` phase (long complete), then the
        offsets; it writes the runs of workers c, c + CW, ... and gives the slot back."""
        sj = pj = 0
        while True:
            while not blk.full[sj].test(pj):
                yield
            tile = blk.tile[sj]
            if tile >= self.num_tiles:
                return
            while not blk.offs[sj].test(pj):
                yield
            assert blk.tile[sj] == tile, "the slot was reloaded while a copy warp still had to write it"
            for w in range(c, self.W, self.CW):
                assert (tile, w) not in self.written
                self.written[(tile, w)] = blk.off[sj][w]
            blk.empty[sj].arrive()
            if blk.empty[sj].pending == blk.empty[sj].count:
                blk.busy[sj] = False
            sj += 1
            if sj == self.nbuf:
                sj, pj = 0, pj ^ 1
            yield

    # ---- scheduler
    def run(self, max_steps=400_000):
        """Random interleaving of copy completions and role steps. A role that is waiting just looks again when picked, so
        a wait that can never be satisfied shows up as the step budget running out."""
        waiting = list(range(self.grid))
        running = []
        for _ in range(max_steps):
            while waiting and len(running) < self.resident:
                running.append(self.make_block(waiting.pop(0)))
            if not running:
                return not self.copies
            if self.copies and self.rng.random() < 0.25:
                blk, st = self.copies.pop(self.rng.randrange(len(self.copies)))
                blk.full[st].arrive()
                continue
            blk = self.rng.choice(running)
            i = self.rng.randrange(len(blk.agents))
            try:
                next(blk.agents[i])
            except StopIteration:
                blk.agents.pop(i)
                if not blk.agents:
                    running.remove(blk)
        return False

    def check(self):
        acc = 0
        for t in range(self.num_tiles):
            for w in range(self.W):
                assert self.written[(t, w)] == acc, (t, w, self.written[(t, w)], acc)
                acc += self.counts[t][w]
        assert self.result == acc


@pytest.mark.parametrize("lag,nbuf", [(1, 3), (2, 4), (2, 5), (3, 5), (2, 8)])
@pytest.mark.parametrize("grid,resident", [(1, 1), (4, 4), (6, 2), (7, 1), (12, 5)])
def test_stream_protocol_finishes_with_sequential_offsets(lag, nbuf, grid, resident):
    for seed in range(6):
        num_tiles = [0 + 1, 3, 17, 64][seed % 4] + seed
        sim = Sim(num_tiles, grid, resident, warps=3, lag=lag, nbuf=nbuf, seed=seed * 7919 + lag * 31 + nbuf)
        assert sim.run(), "the schedule stopped with work left"
        sim.check()
        assert sim.counter >= num_tiles + 1     # every block that ran drew one id past the end and stopped there


def test_stream_protocol_many_random_shapes():
    r = random.Random(5)
    for _ in range(40):
        lag = r.randrange(1, 4)
        nbuf = lag + 2 + r.randrange(0, 3)
        grid = r.randrange(1, 10)
        sim = Sim(r.randrange(1, 90), grid, r.randrange(1, grid + 1), warps=r.randrange(1, 5), lag=lag, nbuf=nbuf, seed=r.randrange(1 << 30))
        assert sim.run()
        sim.check()


@pytest.mark.parametrize("warps,copy_warps", [(4, 2), (4, 1), (3, 3), (5, 2)])
@pytest.mark.parametrize("grid,resident", [(1, 1), (6, 2), (7, 1), (12, 5)])
def test_stream_protocol_with_copy_warps(warps, copy_warps, grid, resident):
    """The same with the writing done by warps of their own (the kernel's default shape: 4 workers, 2 copy warps)."""
    for seed in range(6):
        num_tiles = [1, 3, 17, 64][seed % 4] + seed
        for lag, nbuf in ((2, 4), (3, 5), (3, 7)):
            sim = Sim(num_tiles, grid, resident, warps=warps, lag=lag, nbuf=nbuf, seed=seed * 104729 + warps, copy_warps=copy_warps)
            assert sim.run(), "the schedule stopped with work left"
            sim.check()
