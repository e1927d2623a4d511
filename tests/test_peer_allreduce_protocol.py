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
