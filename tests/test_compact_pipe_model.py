"""A small executable model of the pipelined compaction kernel's protocol (dcb::compact_pipe_body), run under random
schedules. It checks what the kernel's comments claim and what cannot be provoked on purpose on a GPU:

  * progress without co-residency: with fewer resident blocks than launched blocks the launch still finishes, because a
    tile waits only for tiles with smaller ids and ids are drawn in increasing order by blocks that are running;
  * the same protocol with ids fixed in advance (tile = block + k * grid) can stop for ever when not all blocks are
    resident, which is why ids are drawn from a counter;
  * every tile gets the offset of a sequential compaction, whatever the interleaving, for every legal (LAG, PRE).

The model follows the kernel round by round: rank tile k; after the round's barrier draw the id for round k+PRE, publish
the count of tile k, work out the offset of tile k-LAG+1 (which needs the counts of all tiles between the block's
previous tile and that one), write tile k-LAG. A block that needs a count that is not published yet cannot advance.
"""
import random

import pytest


class Block:
    def __init__(self, sim, bid):
        self.sim, self.bid = sim, bid
        self.tiles = []            # tile id per round (None = no tile left)
        self.k = 0                 # current round
        self.phase = "start"
        self.last_tile, self.run_incl = -1, 0
        self.offset = {}           # round -> output offset
        self.done = False

    def draw(self):
        s = self.sim
        if s.static_ids:
            t = self.bid + len(self.tiles) * s.grid
            self.tiles.append(t if t < s.num_tiles else None)
            return
        if self.tiles and self.tiles[-1] is None:
            self.tiles.append(None)
            return
        t = s.counter
        s.counter += 1
        self.tiles.append(t if t < s.num_tiles else None)

    def nvalid(self):
        return next((i for i, t in enumerate(self.tiles) if t is None), None)

    def runnable(self):
        """False only while the offsets step waits for a count another block has not published."""
        if self.phase != "offset":
            return True
        j1 = self.k - self.sim.lag + 1
        nv = self.nvalid()
        if j1 < 0 or (nv is not None and j1 >= nv):
            return True
        return all(self.sim.count_published[t] for t in range(self.last_tile + 1, self.tiles[j1]))

    def step(self):
        s = self.sim
        if self.phase == "start":
            for _ in range(s.pre):
                self.draw()
            self.phase = "rank"
        elif self.phase == "rank":                       # (1) rank tile k (its count becomes known to the block)
            nv = self.nvalid()
            if nv is not None and self.k - s.lag >= nv:
                self.done = True
                return
            self.phase = "fetch"
        elif self.phase == "fetch":                      # after the barrier: (2) draw the id of round k+PRE
            self.draw()
            assert len(self.tiles) == self.k + s.pre + 1
            t = self.tiles[self.k]
            if t is not None:                            # (3) publish the count of tile k
                s.count_published[t] = True
            self.phase = "offset"
        elif self.phase == "offset":                     # (3) offset of tile k-LAG+1 = previous + counts in between
            j1 = self.k - s.lag + 1
            nv = self.nvalid()
            if j1 >= 0 and (nv is None or j1 < nv):
                t1 = self.tiles[j1]
                between = sum(s.counts[t] for t in range(self.last_tile + 1, t1))
                self.offset[j1] = self.run_incl + between
                self.run_incl += between + s.counts[t1]
                self.last_tile = t1
            self.phase = "write"
        elif self.phase == "write":                      # (4) write tile k-LAG at the offset found a round earlier
            j0 = self.k - s.lag
            nv = self.nvalid()
            if j0 >= 0 and (nv is None or j0 < nv):
                s.written[self.tiles[j0]] = self.offset[j0]
            self.k += 1
            self.phase = "rank"


class Sim:
    def __init__(self, num_tiles, grid, resident, lag, pre, seed, static_ids=False):
        self.num_tiles, self.grid, self.resident, self.lag, self.pre, self.static_ids = num_tiles, grid, resident, lag, pre, static_ids
        self.rng = random.Random(seed)
        self.counts = [self.rng.randrange(0, 4097) for _ in range(num_tiles)]
        self.count_published = [False] * num_tiles
        self.written = {}
        self.counter = 0

    def run(self, max_steps=2_000_000):
        """Blocks start in index order as slots free up (a 1-D grid is dispatched in index order). Returns True when all
        blocks finished, False when every resident block waits for a count that no resident block can publish."""
        waiting = [Block(self, b) for b in range(self.grid)]
        resident = []
        for _ in range(max_steps):
            while waiting and len(resident) < self.resident:
                resident.append(waiting.pop(0))
            if not resident:
                return True
            ready = [b for b in resident if b.runnable()]
            if not ready:
                return False
            b = self.rng.choice(ready)
            b.step()
            if b.done:
                resident.remove(b)
        raise AssertionError("model did not finish")


def expected_offsets(counts):
    out, acc = {}, 0
    for t, c in enumerate(counts):
        out[t] = acc
        acc += c
    return out


@pytest.mark.parametrize("lag,pre", [(2, 1), (3, 1), (3, 2), (4, 3)])
@pytest.mark.parametrize("grid,resident", [(12, 12), (12, 5), (12, 1), (40, 7)])
def test_drawn_ids_always_finish_with_sequential_offsets(lag, pre, grid, resident):
    for seed in range(6):
        sim = Sim(num_tiles=157, grid=grid, resident=resident, lag=lag, pre=pre, seed=seed)
        assert sim.run(), (lag, pre, grid, resident, seed)
        assert sim.written == expected_offsets(sim.counts)


def test_fewer_tiles_than_blocks_and_empty_input():
    for num_tiles in (0, 1, 3):
        sim = Sim(num_tiles=num_tiles, grid=9, resident=4, lag=2, pre=1, seed=1)
        assert sim.run()
        assert sim.written == expected_offsets(sim.counts)


def test_ids_fixed_in_advance_can_stop_without_co_residency():
    """With tile = block + k * grid and fewer slots than blocks, the resident blocks end up waiting for tiles of blocks
    that cannot start: the reason the kernel draws its ids from a counter."""
    stuck = 0
    for seed in range(6):
        sim = Sim(num_tiles=157, grid=12, resident=5, lag=2, pre=1, seed=seed, static_ids=True)
        stuck += 0 if sim.run() else 1
    assert stuck == 6
    # all blocks resident: the fixed assignment works too
    sim = Sim(num_tiles=157, grid=12, resident=12, lag=2, pre=1, seed=0, static_ids=True)
    assert sim.run() and sim.written == expected_offsets(sim.counts)
