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


# ---- flag-synchronised two-shot path ---------------------------------------------------------------
# One staging area and one result area per rank, reused by every call (no rotation); two flag
# barriers per call keep the reuse safe (`twoshot_flag_body`): ranks write their rows into the owners'
# staging slots and raise flag plane 0; after all plane-0 flags of the call the owner reduces its
# staging slots and writes the result into every rank's result area, then raises plane 1; after all
# plane-1 flags every rank reads its result area. Flags carry the call number and are compared with
# ">=", so a flag raised early by a rank that runs ahead is never lost.

CLOBBERED = -7


def explore_flags(nranks: int, ncalls: int, second_barrier: bool, stage_overwrites_results: bool = False):
    peers = [[p for p in range(nranks) if p != r] for r in range(nranks)]
    prog = []
    for r in range(nranks):
        steps = [("stage", p) for p in peers[r]] + [("signal", 0), ("wait", 0)]
        steps += [("reduce", p) for p in peers[r]] + [("publish", p) for p in peers[r]]
        if second_barrier:
            steps += [("signal", 1), ("wait", 1)]
        steps += [("epilogue", p) for p in peers[r]]
        prog.append(steps)
    plen = len(prog[0])
    none = tuple(SENTINEL for _ in range(nranks))
    start = (tuple(0 for _ in range(nranks)),                       # call number per rank
             tuple(0 for _ in range(nranks)),                       # program counter per rank
             tuple(none for _ in range(nranks)),                    # staging[rank][src]
             tuple(none for _ in range(nranks)),                    # result[rank][owner]
             tuple((none, none) for _ in range(nranks)))            # flags[rank][plane][src]
    seen = {start}
    queue = deque([start])

    def put(table, r, i, v):
        row = table[r][:i] + (v,) + table[r][i + 1:]
        return table[:r] + (row,) + table[r + 1:]

    while queue:
        calls, pcs, staging, result, flags = queue.popleft()
        if all(c == ncalls for c in calls):
            continue
        moved = False
        for r in range(nranks):
            e = calls[r]
            if e == ncalls:
                continue
            op, arg = prog[r][pcs[r]]
            st, rs, fl = staging, result, flags
            if op == "stage":
                st = put(staging, arg, r, e)
                if stage_overwrites_results:
                    # the result area starts where the gather area of the call ends: a LARGER next call's
                    # gather slots reach into the rows that the previous call's results occupy
                    for owner in range(nranks):
                        rs = put(rs, arg, owner, CLOBBERED)
            elif op == "signal":
                for p in peers[r]:
                    planes = list(fl[p])
                    planes[arg] = planes[arg][:r] + (e,) + planes[arg][r + 1:]
                    fl = fl[:p] + (tuple(planes),) + fl[p + 1:]
            elif op == "wait":
                if any(flags[r][arg][p] < e for p in peers[r]):
                    continue
            elif op == "reduce":
                if staging[r][arg] != e:
                    return (f"rank {r} call {e}: staging slot of rank {arg} holds call {staging[r][arg]}", len(seen))
            elif op == "publish":
                rs = put(result, arg, r, e)
            else:
                if result[r][arg] != e:
                    return (f"rank {r} call {e}: result of owner {arg} holds call {result[r][arg]}", len(seen))
            npc = pcs[r] + 1
            ncall = e
            if npc == plen:
                npc, ncall = 0, e + 1
            state = (calls[:r] + (ncall,) + calls[r + 1:], pcs[:r] + (npc,) + pcs[r + 1:], st, rs, fl)
            moved = True
            if state not in seen:
                seen.add(state)
                queue.append(state)
        if not moved:
            return (f"deadlock at calls {calls}, program counters {pcs}", len(seen))
    return (None, len(seen))


@pytest.mark.parametrize("nranks,ncalls", [(2, 6), (3, 4), (4, 2)])
def test_two_flag_barriers_make_the_shared_staging_safe(nranks, ncalls):
    violation, states = explore_flags(nranks, ncalls, second_barrier=True)
    assert violation is None, violation
    assert states > 100


def test_without_the_second_barrier_a_fast_rank_overwrites_what_a_slow_rank_still_reads():
    violation, _ = explore_flags(2, 3, second_barrier=False)
    assert violation is not None


def test_result_area_behind_a_size_dependent_gather_area_is_unsafe_when_messages_grow():
    """The epilogue of a call reads the result area after the last flag wait, and nothing follows that wait. If
    the result area started right behind the gather area, a rank that runs ahead into a larger call would push
    gather rows over result rows that a slow rank is still reading. The kernels therefore keep the result area
    at a fixed offset (second half of the staging region), which is the model without the overwrite."""
    violation, _ = explore_flags(2, 3, second_barrier=True, stage_overwrites_results=True)
    assert violation is not None and "result" in violation
    violation, _ = explore_flags(2, 3, second_barrier=True, stage_overwrites_results=False)
    assert violation is None
