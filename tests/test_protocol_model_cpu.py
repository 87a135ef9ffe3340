"""Exhaustive interleaving check of the Lamport buffer-rotation protocol (a model, no GPU).

The one-shot kernel (csrc/include/tdx/ar_fusion_kernels.cuh, `oneshot_lamport_body`) has no barrier:
in call number e every rank pushes its rows into slot `rank` of each peer's buffer e % 3, re-fills
its own buffer (e + 2) % 3 with sentinels (the buffer of call e - 1), polls its own buffer e % 3
until no slot holds the sentinel, and finally advances its epoch. Blocks of one rank run
independently of each other, ranks drift apart by up to one call, and the buffers are reused every
third call. This test explores EVERY interleaving of those steps for small configurations and
checks three properties:

 * a poll that finds a slot written always reads the value of the CURRENT call (never a leftover
   of call e - 3 that a lost clear would expose, never the next call's data),
 * no reachable state is stuck before all calls are done (no deadlock),
 * every run ends with all ranks having completed all calls.

The same exploration with only two buffers in rotation must find a violation, which shows that the
third buffer is what makes the barrier-free reuse safe (and that the checker can see such a bug).
The reference rotates three buffers as well (src/common/all_reduce_fusion_impl.h:166-204) but also
needs a per-call flag exchange for its counters; here the proof obligation is discharged by search.
"""
from collections import deque

import pytest

SENTINEL = -1


def explore(nranks: int, nblocks: int, ncalls: int, nbuffers: int, clear_distance: int):
    """Breadth-first search over all interleavings.

    State: per rank the epoch, per (rank, block) a program counter, and the buffers
    buf[rank][buffer][src][block]. A block's program for call e is: push its row to every peer,
    clear its share of buffer (e + clear_distance) % nbuffers, poll its row from every peer. The
    last block to finish a call advances the rank's epoch (and with it starts the next call for
    all blocks of that rank), as `finish_launch` does with its arrival counter.
    Returns (violation or None, number of states)."""
    peers = [[p for p in range(nranks) if p != r] for r in range(nranks)]
    # program of one block for one call: list of (op, peer)
    prog = [[("push", p) for p in peers[r]] + [("clear", None)] + [("poll", p) for p in peers[r]] for r in range(nranks)]
    plen = len(prog[0])

    def initial():
        epochs = tuple(0 for _ in range(nranks))
        pcs = tuple(tuple(0 for _ in range(nblocks)) for _ in range(nranks))
        bufs = tuple(tuple(tuple(tuple(SENTINEL for _ in range(nblocks)) for _ in range(nranks)) for _ in range(nbuffers))
                     for _ in range(nranks))
        return epochs, pcs, bufs

    def set_buf(bufs, r, b, src, blk, val):
        rb = list(map(list, (list(map(list, x)) for x in bufs[r])))
        rb[b][src][blk] = val
        new_r = tuple(tuple(tuple(s) for s in bb) for bb in rb)
        return bufs[:r] + (new_r,) + bufs[r + 1:]

    start = initial()
    seen = {start}
    queue = deque([start])
    while queue:
        epochs, pcs, bufs = queue.popleft()
        if all(e == ncalls for e in epochs):
            continue
        moved = False
        for r in range(nranks):
            e = epochs[r]
            if e == ncalls:
                continue
            for blk in range(nblocks):
                pc = pcs[r][blk]
                if pc == plen:
                    continue            # this block has finished the call and waits for the launch to end
                op, peer = prog[r][pc]
                nb = bufs
                if op == "push":
                    nb = set_buf(bufs, peer, e % nbuffers, r, blk, e)
                elif op == "clear":
                    tgt = (e + clear_distance) % nbuffers
                    for src in range(nranks):
                        nb = set_buf(nb, r, tgt, src, blk, SENTINEL)
                else:
                    val = bufs[r][e % nbuffers][peer][blk]
                    if val == SENTINEL:
                        continue        # not enabled: keep polling
                    if val != e:
                        return (f"rank {r} block {blk} call {e}: read the data of call {val} from rank {peer}", len(seen))
                npc_r = pcs[r][:blk] + (pc + 1,) + pcs[r][blk + 1:]
                nepochs = epochs
                if all(x == plen for x in npc_r):          # last block of the launch: next call
                    nepochs = epochs[:r] + (e + 1,) + epochs[r + 1:]
                    npc_r = tuple(0 for _ in range(nblocks))
                state = (nepochs, pcs[:r] + (npc_r,) + pcs[r + 1:], nb)
                moved = True
                if state not in seen:
                    seen.add(state)
                    queue.append(state)
        if not moved:
            return (f"deadlock at epochs {epochs}, program counters {pcs}", len(seen))
    return (None, len(seen))


@pytest.mark.parametrize("nranks,nblocks,ncalls", [(2, 1, 7), (2, 2, 6), (3, 1, 6), (3, 2, 3), (4, 1, 3)])
def test_three_buffers_are_safe_in_every_interleaving(nranks, nblocks, ncalls):
    violation, states = explore(nranks, nblocks, ncalls, nbuffers=3, clear_distance=2)
    assert violation is None, violation
    assert states > 100          # the search really branched


def test_two_buffers_are_not():
    # rotate two buffers and clear "the other one": a fast rank's next push lands in a buffer
    # that the slow rank has not cleared / is still reading
    violation, _ = explore(2, 1, 5, nbuffers=2, clear_distance=1)
    assert violation is not None


def test_clearing_the_next_buffer_instead_of_the_previous_one_is_caught():
    # with three buffers, wiping (e + 1) % 3 can destroy what a rank that runs one call ahead already pushed
    violation, _ = explore(2, 1, 5, nbuffers=3, clear_distance=1)
    assert violation is not None
