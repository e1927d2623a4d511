"""Model check of the handshake of the fused tensor-parallel all-reduce (csrc/elementwise.cu, `peer_row_handshake`,
and the slot alternation of tensor_parallel/peer_allreduce.py), on the CPU.

Each rank is a coroutine that yields between its memory operations; a random scheduler interleaves them.  The
property: whenever a rank reads a peer's slot for call k, the slot holds the peer's data of call k - i.e. two
alternating slots and monotonic per-row flags are enough, however far the ranks drift apart."""
import random

import pytest


def rank_program(rank, world, calls, slots, flags, log):
    """slots[r][s] = payload of rank r in slot s; flags[r][q] = last call number rank q announced to rank r."""
    for k in range(1, calls + 1):
        s = (k - 1) & 1                      # host side: slots alternate per call
        slots[rank][s] = (rank, k)           # the GEMM writes this rank's partial output
        yield
        for q in range(world):               # handshake: release-store the call number to every peer ...
            if q != rank:
                flags[q][rank] = k
                yield
        while any(flags[rank][q] < k for q in range(world) if q != rank):
            yield                            # ... and wait (bounded on the device) for theirs
        for q in range(world):               # sum the ranks' rows in rank order
            got = slots[q][s]
            assert got == (q, k), f"rank {rank} call {k}: slot of rank {q} holds {got}"
            log.append((rank, k, q))
            yield


@pytest.mark.parametrize("world", [2, 3, 4, 8])
def test_two_slots_and_monotonic_flags_suffice(world):
    rng = random.Random(world)
    for trial in range(200):
        calls = rng.randint(1, 7)
        slots = [[None, None] for _ in range(world)]
        flags = [[0] * world for _ in range(world)]
        log = []
        progs = [rank_program(r, world, calls, slots, flags, log) for r in range(world)]
        live = list(range(world))
        favourite = rng.randrange(world)     # one rank is scheduled much more often: it runs as far ahead as it can
        steps = 0
        while live:
            r = favourite if (favourite in live and rng.random() < 0.7) else rng.choice(live)
            try:
                next(progs[r])
            except StopIteration:
                live.remove(r)
            steps += 1
            assert steps < 200000, "deadlock"
        assert len(log) == world * world * calls


def test_a_single_slot_is_not_enough():
    # the same protocol with one slot: a rank that runs ahead overwrites what a slow peer has not read yet
    def program(rank, world, calls, slots, flags):
        for k in range(1, calls + 1):
            slots[rank] = (rank, k)
            yield
            for q in range(world):
                if q != rank:
                    flags[q][rank] = k
                    yield
            while any(flags[rank][q] < k for q in range(world) if q != rank):
                yield
            for q in range(world):
                if slots[q] != (q, k):
                    raise AssertionError("stale read")
                yield

    rng = random.Random(0)
    failures = 0
    for trial in range(300):
        slots, flags = [None, None], [[0, 0], [0, 0]]
        progs = [program(r, 2, 4, slots, flags) for r in range(2)]
        live = [0, 1]
        try:
            while live:
                r = 0 if (0 in live and rng.random() < 0.8) else rng.choice(live)
                try:
                    next(progs[r])
                except StopIteration:
                    live.remove(r)
        except AssertionError:
            failures += 1
    assert failures > 0


def test_same_slot_twice_in_a_row_can_read_stale_data():
    # What an odd number of calls per captured forward would do to the one-shot form: replays end and start on the
    # same slot, the handshake only fences the call after next, and a fast rank overwrites what a slow peer still reads.
    def program(rank, world, slot_of_call, slots, flags):
        for k, s in enumerate(slot_of_call, start=1):
            slots[rank][s] = (rank, k)
            yield
            for q in range(world):
                if q != rank:
                    flags[q][rank] = k
                    yield
            while any(flags[rank][q] < k for q in range(world) if q != rank):
                yield
            for q in range(world):
                if slots[q][s] != (q, k):
                    raise AssertionError("stale read")
                yield

    rng = random.Random(1)
    failures = 0
    for trial in range(300):
        slots, flags = [[None, None], [None, None]], [[0, 0], [0, 0]]
        progs = [program(r, 2, [0, 1, 0, 0, 1, 0], slots, flags) for r in range(2)]  # a 3-call forward replayed twice
        live = [0, 1]
        try:
            while live:
                r = 0 if (0 in live and rng.random() < 0.8) else rng.choice(live)
                try:
                    next(progs[r])
                except StopIteration:
                    live.remove(r)
        except AssertionError:
            failures += 1
    assert failures > 0


def two_shot_program(rank, world, calls, rows, inp, hidden, normed, flags_a, flags_b, log):
    """csrc/tp_exchange.cu: ONE input buffer and ONE output buffer per rank, two flag exchanges per call."""
    per = -(-rows // world)
    mine = range(rank * per, min(rows, (rank + 1) * per))
    for k in range(1, calls + 1):
        for r in range(rows):                      # the GEMM writes this rank's partial output
            inp[rank][r] = (rank, k, r)
            yield
        for q in range(world):                     # exchange A: announce, then wait
            if q != rank:
                flags_a[q][rank] = k
                yield
        while any(flags_a[rank][q] < k for q in range(world) if q != rank):
            yield
        for r in mine:                             # reduce my rows from every rank, add my residual, store everywhere
            for q in range(world):
                got = inp[q][r]
                assert got == (q, k, r), f"rank {rank} call {k}: input row {r} of rank {q} holds {got}"
                yield
            res = hidden[rank][r]                  # the residual: the previous call's hidden row (in place)
            assert res == (k - 1, r), f"rank {rank} call {k}: residual row {r} is {res}"
            for q in range(world):
                hidden[q][r] = (k, r)
                normed[q][r] = (k, r)
                yield
        for q in range(world):                     # exchange B
            if q != rank:
                flags_b[q][rank] = k
                yield
        while any(flags_b[rank][q] < k for q in range(world) if q != rank):
            yield
        for r in range(rows):                      # the next GEMM reads all normalised rows of this call
            assert normed[rank][r] == (k, r), f"rank {rank} after call {k}: normed row {r} is {normed[rank][r]}"
            log.append((rank, k, r))
            yield


@pytest.mark.parametrize("world,rows", [(2, 5), (3, 7), (4, 8), (8, 16), (8, 3)])
def test_two_shot_exchange_needs_one_buffer_only(world, rows):
    rng = random.Random(10 * world + rows)
    for trial in range(100):
        calls = rng.randint(1, 6)
        inp = [[None] * rows for _ in range(world)]
        hidden = [[(0, r) for r in range(rows)] for _ in range(world)]
        normed = [[None] * rows for _ in range(world)]
        fa = [[0] * world for _ in range(world)]
        fb = [[0] * world for _ in range(world)]
        log = []
        progs = [two_shot_program(r, world, calls, rows, inp, hidden, normed, fa, fb, log) for r in range(world)]
        live = list(range(world))
        favourite = rng.randrange(world)
        steps = 0
        while live:
            r = favourite if (favourite in live and rng.random() < 0.7) else rng.choice(live)
            try:
                next(progs[r])
            except StopIteration:
                live.remove(r)
            steps += 1
            assert steps < 2000000, "deadlock"
        assert len(log) == world * rows * calls


def two_shot_splitk_rank(rank, world, calls, rows, inp, flags_a, flags_b, counters, rng, log):
    """The split-K form of csrc/tp_exchange.cu at CTA granularity: a launch is `per` CTAs; each first writes a strided share
    of ALL rows of this rank's input buffer (the sums of its GEMM's partial products), the CTA that counts last on
    counters[2] sends exchange A, every CTA waits for the peers' A flags before it reads their rows, and the CTA that counts
    last on counters[1] runs exchange B.  A launch starts only when the previous one has ended (stream order)."""
    per = -(-rows // world)

    def cta(b, k):
        for r in range(b, rows, per):                       # split-K sums -> this rank's input rows
            inp[rank][r] = (rank, k, r)
            yield
        counters[rank][2] += 1                              # atomicAdd after the CTA's fence
        last = counters[rank][2] == per
        if last:
            counters[rank][2] = 0
        yield
        if last:
            for q in range(world):                          # exchange A, sent once all rows are written
                if q != rank:
                    flags_a[q][rank] = k
                    yield
        while any(flags_a[rank][q] < k for q in range(world) if q != rank):
            yield
        row = rank * per + b
        if row < rows:
            for q in range(world):
                got = inp[q][row]
                assert got == (q, k, row), f"rank {rank} call {k}: input row {row} of rank {q} holds {got}"
                log.append((rank, k, row, q))
                yield
        counters[rank][1] += 1
        if counters[rank][1] == per:                        # exchange B by the CTA that finishes last
            counters[rank][1] = 0
            for q in range(world):
                if q != rank:
                    flags_b[q][rank] = k
                    yield
            while any(flags_b[rank][q] < k for q in range(world) if q != rank):
                yield
            counters[rank][0] = k

    for k in range(1, calls + 1):
        ctas = [cta(b, k) for b in range(per)]
        while ctas:                                         # all CTAs of a launch are resident: any interleaving
            c = rng.choice(ctas)
            try:
                next(c)
            except StopIteration:
                ctas.remove(c)
            yield
        assert counters[rank][0] == k


@pytest.mark.parametrize("world,rows", [(2, 5), (3, 7), (4, 8), (8, 16), (8, 3)])
def test_two_shot_exchange_with_split_k_input(world, rows):
    rng = random.Random(100 * world + rows)
    for trial in range(60):
        calls = rng.randint(1, 5)
        inp = [[None] * rows for _ in range(world)]
        fa = [[0] * world for _ in range(world)]
        fb = [[0] * world for _ in range(world)]
        counters = [[0, 0, 0] for _ in range(world)]
        log = []
        progs = [two_shot_splitk_rank(r, world, calls, rows, inp, fa, fb, counters, rng, log) for r in range(world)]
        live = list(range(world))
        favourite = rng.randrange(world)
        steps = 0
        while live:
            r = favourite if (favourite in live and rng.random() < 0.7) else rng.choice(live)
            try:
                next(progs[r])
            except StopIteration:
                live.remove(r)
            steps += 1
            assert steps < 4000000, "deadlock"
        assert len(log) == world * rows * calls


def test_split_k_input_announced_by_the_first_cta_would_read_unfinished_rows():
    """Why the announcement waits for the arrival count: if CTA 0 announced as soon as ITS rows were written (as the
    plain form does, where the GEMM before the kernel has written everything), a peer could read a row that another CTA
    has not summed yet."""
    world, rows = 2, 6
    rng = random.Random(3)
    failures = 0
    for trial in range(200):
        inp = [[None] * rows for _ in range(world)]
        flag = [0] * world
        per = rows // world

        def cta(rank, b):
            for r in range(b, rows, per):
                inp[rank][r] = (rank, r)
                yield
            if b == 0:
                flag[rank] = 1
            yield
            while not flag[1 - rank]:
                yield
            row = rank * per + b
            assert inp[1 - rank][row] == (1 - rank, row)

        ctas = [cta(r, b) for r in range(world) for b in range(per)]
        try:
            while ctas:
                c = rng.choice(ctas)
                try:
                    next(c)
                except StopIteration:
                    ctas.remove(c)
        except AssertionError:
            failures += 1
    assert failures > 0


def test_choice_of_exchange_form_depends_on_sizes_every_rank_knows():
    """`use_one_shot` (tensor_parallel/peer_allreduce.py): one-shot while a rank pulls at most 8 MB per call."""
    from megatron_mixtera_b200.tensor_parallel import peer_allreduce as P

    assert P.use_one_shot(2, 128, 4096) and P.use_one_shot(4, 128, 4096) and P.use_one_shot(8, 128, 4096)
    assert P.use_one_shot(2, 256, 8192) and not P.use_one_shot(4, 256, 8192) and not P.use_one_shot(8, 256, 8192)
    assert not P.use_one_shot(4, 512, 4096)  # a large prefill step goes through the two-shot exchange
    old = P.ONE_SHOT_MAX_WORLD
    try:
        P.ONE_SHOT_MAX_WORLD = 1            # what the tests and the bench ablation use to force the two-shot form
        assert not P.use_one_shot(2, 8, 512)
    finally:
        P.ONE_SHOT_MAX_WORLD = old


def test_forward_guard_covers_every_communicator():
    """`begin_forward` / `end_forward` apply the one-shot form's even-number-of-calls rule to whichever communicators
    exist, including one that was created during the forward (it started on slot 0)."""
    from megatron_mixtera_b200.tensor_parallel import peer_allreduce as P

    class Fake:
        def __init__(self):
            self._next_slot = 0

        begin_forward = P.PeerAllReduce.begin_forward
        end_forward = P.PeerAllReduce.end_forward

        def call(self):
            self._next_slot ^= 1

    saved = dict(P._COMMS)
    try:
        P._COMMS.clear()
        at_entry = P.begin_forward()
        c = P._COMMS["one_shot"] = Fake()   # created by the first fused reduction of this forward
        c.call(); c.call()
        P.end_forward(at_entry)              # two calls: fine
        at_entry = P.begin_forward()
        c.call()
        with pytest.raises(RuntimeError):
            P.end_forward(at_entry)          # an odd number of calls would reuse a slot on replay
    finally:
        P._COMMS.clear()
        P._COMMS.update(saved)
