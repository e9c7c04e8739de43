"""The barrier protocol of the two-tile tcgen05 attention kernel, replayed on the host under random schedules.

`csrc/attention_tcgen05.cu` (`attn_tc_pp_kernel`) synchronises a copy producer, three product-issuing threads, two
softmax warpgroups and a correction warpgroup through mbarriers that are waited for by PARITY: a wait tells "phase k
is over" from "phase k is running" only if the waiter is at most one phase away.  Roles run up to two key steps
apart, so this is easy to get wrong, and a mistake shows on the GPU as a wait that runs out (a second each) or as a
rare wrong row.  This model has the same roles, the same barriers with the same arrival counts and parities and the
same ring order, steps them in random interleavings and checks at every access that the data read is the data
meant.  It needs no GPU.  It knows nothing about arithmetic; `tests/test_gpu_kernels.py` covers that.
"""
import random

import pytest

NS = 8          # stages of the key/value ring (pp::NS)


class Barrier:
    """An mbarrier: `count` arrivals complete a phase; a parity wait passes when the phase of that parity is over."""

    def __init__(self, count):
        self.count, self.pending, self.phase = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0
        if self.pending == 0:
            self.phase += 1
            self.pending = self.count

    def passed(self, parity):
        return (self.phase & 1) != parity


class Deadlock(Exception):
    pass


def simulate(nsteps, ntq, seed, product_barriers_per_tile=2, softmax_threads=2, correction_threads=2):
    """One CTA walking `nsteps` key steps with `ntq` query tiles.  Raises AssertionError when a role touches data of
    the wrong step and Deadlock when nothing can move."""
    rnd = random.Random(seed)
    W, C, PB = softmax_threads, correction_threads, product_barriers_per_tile
    bars = {}
    for i in range(NS):
        bars["FULL", i] = Barrier(1)
        bars["EMPTY", i] = Barrier(ntq)                      # one commit per tile in use
    for t in range(2):
        bars["LF", t] = Barrier(W)
        for b in range(2):
            bars["SF", t, b] = Barrier(1)
            bars["PF", t, b] = Barrier(W)
            bars["SC", t, b] = Barrier(W)
            bars["OC", t, b] = Barrier(C)
            bars["OF", t, b] = Barrier(1)
    queues = [[], [], []]      # products issued and not yet executed, per issuing thread (each in order)
    copies = []                # [clocks left, stage, tile]
    ring = [None] * NS
    scores, probs, alpha, pv_issued, pv_done = {}, {}, {}, {}, {}

    def wait(name, parity):
        while not bars[name].passed(parity):
            yield

    def of_bar(t, j):          # the barrier product j of tile t signals, and the parity that means "it has landed"
        return (("OF", t, j % PB), ((j // PB) & 1))

    def k_index(j):
        return j if j < 2 else 2 * j - 1

    def v_index(j):
        return 2 * nsteps - 1 if j == nsteps - 1 else 2 * j + 2

    def producer():
        order = [("K", 0)] + ([("K", 1)] if nsteps > 1 else [])
        for j in range(nsteps):
            order.append(("V", j))
            if j + 2 < nsteps:
                order.append(("K", j + 2))
        for it, tile in enumerate(order):
            st = it % NS
            yield from wait(("EMPTY", st), ((it // NS) & 1) ^ 1)
            copies.append([rnd.randint(1, 6), st, tile])

    def score_issuer():
        for j in range(nsteps):
            b, idx = j & 1, k_index(j)
            st = idx % NS
            yield from wait(("FULL", st), (idx // NS) & 1)
            assert ring[st] == ("K", j), ("scores from the wrong tile", j, ring[st])
            for t in range(ntq):
                if j >= 2:
                    name, parity = of_bar(t, j - 2)
                    yield from wait(name, parity)
                    assert pv_done.get(t, -1) >= j - 2, ("scores over probabilities still in use", t, j)
                queues[2] += [("S", t, b, j, st), ("commit", ("SF", t, b)), ("commit", ("EMPTY", st))]

    def pv_issuer(t):
        for j in range(nsteps):
            b, par, idx = j & 1, (j >> 1) & 1, v_index(j)
            st = idx % NS
            yield from wait(("FULL", st), (idx // NS) & 1)
            assert ring[st] == ("V", j), ("values from the wrong tile", j, ring[st])
            yield from wait(("PF", t, b), par)
            yield from wait(("OC", t, b), par)
            for w in range(W):
                assert probs.get((t, b, w)) == j, ("probabilities of another step", t, j)
            pv_issued[t] = j
            queues[t] += [("PV", t, b, j, st), ("commit", of_bar(t, j)[0]), ("commit", ("EMPTY", st))]

    def softmax(t, w):
        for j in range(nsteps):
            b, par = j & 1, (j >> 1) & 1
            yield from wait(("SF", t, b), par)
            assert scores.get((t, b)) == j, ("scores of another step", t, j, scores.get((t, b)))
            yield
            alpha[b, t, w] = j
            bars["SC", t, b].arrive()
            for _ in range(rnd.randint(0, 3)):
                yield
            assert scores.get((t, b)) == j
            probs[t, b, w] = j
            bars["PF", t, b].arrive()
        bars["LF", t].arrive()

    def correction(c):
        for j in range(nsteps):
            b, par = j & 1, (j >> 1) & 1
            for t in range(ntq):
                yield from wait(("SC", t, b), par)
                for w in range(W):
                    assert alpha[b, t, w] == j, ("scale factors of another step", t, j)
                if j > 0 and rnd.random() < 0.5:             # this warp has a row to rescale
                    name, parity = of_bar(t, j - 1)
                    yield from wait(name, parity)
                    assert pv_done.get(t, -1) == j - 1, ("output rescaled while a product was in flight", t, j, pv_done.get(t, -1))
                    assert pv_issued.get(t, -1) == j - 1, ("output rescaled after the next product was issued", t, j)
                    for _ in range(rnd.randint(0, 3)):
                        yield
                bars["OC", t, b].arrive()
        for t in range(ntq):
            yield from wait(("LF", t), 0)
            name, parity = of_bar(t, nsteps - 1)
            yield from wait(name, parity)
            assert pv_done.get(t, -1) == nsteps - 1, ("output stored before the last product", t, pv_done.get(t, -1))

    agents = [producer(), score_issuer()] + [pv_issuer(t) for t in range(ntq)]
    agents += [softmax(t, w) for t in range(ntq) for w in range(W)] + [correction(c) for c in range(C)]

    def state():
        return (sum(b.phase * 1000 + b.pending for b in bars.values()), sum(map(len, queues)), len(copies))

    idle = 0
    while agents:
        before = state()
        queue = rnd.choice(queues)                           # the tensor core takes a thread's products in order
        if queue and rnd.random() < 0.5:
            op = queue.pop(0)
            if op[0] == "commit":
                bars[op[1]].arrive()
            elif op[0] == "S":
                _, t, b, j, st = op
                assert ring[st] == ("K", j), ("scores read a stage that was refilled", op, ring[st])
                scores[t, b] = j
            else:
                _, t, b, j, st = op
                assert ring[st] == ("V", j), ("product read a stage that was refilled", op, ring[st])
                pv_done[t] = j
        for c in list(copies):
            c[0] -= 1
            if c[0] <= 0:
                ring[c[1]] = c[2]
                bars["FULL", c[1]].arrive()
                copies.remove(c)
        agent = rnd.choice(agents)
        finished = False
        try:
            next(agent)
        except StopIteration:
            agents.remove(agent)
            finished = True
        idle = 0 if (finished or state() != before) else idle + 1
        if idle > 20000:
            raise Deadlock(f"nothing moves: {nsteps} steps, {ntq} tiles, seed {seed}")


@pytest.mark.parametrize("ntq", [1, 2])
@pytest.mark.parametrize("nsteps", [1, 2, 3, 4, 5, 7, 12, 33])
def test_protocol_holds_under_random_schedules(nsteps, ntq):
    for seed in range(25):
        simulate(nsteps, ntq, seed)


def test_one_product_barrier_per_tile_is_not_enough():
    """With a single barrier per tile for "product j has landed", the correction warps - up to two steps ahead of
    the products, and not looking at every product - take a parity for the wrong phase: the model must see a
    rescale in flight of a product, or a wait that never ends."""
    seen = False
    for seed in range(60):
        try:
            simulate(12, 2, seed, product_barriers_per_tile=1)
        except (AssertionError, Deadlock):
            seen = True
            break
    assert seen
