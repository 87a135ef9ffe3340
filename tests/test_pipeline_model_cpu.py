"""Randomised interleaving checks of the mbarrier pipelines of the tcgen05 kernels (models, no GPU).

The kernels synchronise their roles (TMA producer, MMA thread, epilogue / softmax warps) with
mbarriers that are waited on by PHASE PARITY. The parity expressions - ``(it / stages) & 1``,
``((it / stages) - 1) & 1``, ``((n >> 1) - 1) & 1`` and friends - are the classic place for an
off-by-one that shows up on hardware as a hang or as a tile computed from the wrong data. These
models replay the role programs of

 * the persistent GEMM (csrc/gemm_persist.cu): operand ring that runs across tile boundaries,
   two accumulator buffers handed between the MMA thread and the epilogue warps;
 * the tensor-core decode attention kernel (csrc/attention_decode_tc.cu): K/V ring, double-buffered
   scores, one probability tile, one P*V buffer;
 * the prompt attention kernel (csrc/attention_prefill_tc.cu): separate K and V rings, two softmax groups on
   alternate chunks, each with its score buffer, probability tile and accumulator in tensor memory;
 * the CTA-pair GEMM (csrc/gemm_pair.cu): two producers crediting the leader's transaction-counting
   barriers, stages released in both CTAs by the leader's MMA thread, a persistent tile loop with two
   accumulator buffers that the epilogue warps of BOTH CTAs hand back to the leader

with the same parity expressions, under random schedules in which TMA completions and MMA
completions (tcgen05.commit arrivals) land late and at arbitrary moments, and check that every
consumer sees exactly the data it expects, that no buffer is overwritten before its reader is
done, and that nothing deadlocks. An mbarrier is modelled as the PTX ISA describes
mbarrier.try_wait.parity: the wait for parity p succeeds iff the barrier's current (incomplete) phase
has the other parity.
"""
import random

import pytest


class MBar:
    def __init__(self, count):
        self.count, self.pending, self.completed = count, count, 0

    def arrive(self):
        self.pending -= 1
        assert self.pending >= 0, "more arrivals than the barrier expects in one phase"
        if self.pending == 0:
            self.completed += 1
            self.pending = self.count

    def ready(self, parity):
        return parity != (self.completed & 1)


def run(actors, events, rng, max_steps=200000):
    """`actors`: generators that yield ("wait", bar, parity) until the wait can pass, or ("step",).
    `events`: list of pending asynchronous completions (callables), drained in random order per queue."""
    live = {i: a for i, a in enumerate(actors)}
    blocked = {}
    for _ in range(max_steps):
        if not live and not any(events.values()):
            return
        choices = []
        for i in live:
            w = blocked.get(i)
            if w is None or w[0].ready(w[1]):
                choices.append(("actor", i))
        for q, lst in events.items():
            if lst:
                choices.append(("event", q))
        assert choices, f"deadlock: actors {sorted(live)} blocked, no completion pending"
        kind, key = rng.choice(choices)
        if kind == "event":
            events[key].pop(0)()
            continue
        blocked.pop(key, None)
        try:
            req = next(live[key])
        except StopIteration:
            del live[key]
            continue
        if req[0] == "wait" and not req[1].ready(req[2]):
            blocked[key] = (req[1], req[2])
            # the generator re-yields the same wait when resumed: see wait() below
    raise AssertionError("did not finish")


def wait(bar, parity):
    while not bar.ready(parity):
        yield ("wait", bar, parity)


# ---- persistent GEMM ------------------------------------------------------------------------------

def persistent_gemm(ntiles_of_cta, nkb, stages, rng):
    full = [MBar(1) for _ in range(stages)]
    empty = [MBar(1) for _ in range(stages)]
    acc_full = [MBar(1) for _ in range(2)]
    n_epi = 2                                            # stands for the 128 epilogue threads
    acc_empty = [MBar(n_epi) for _ in range(2)]
    stage_data = [None] * stages
    stage_busy = [False] * stages                        # an MMA that read the stage has not completed yet
    acc = [None, None]                                   # (tile, list of k blocks) accumulated so far
    acc_readers = [0, 0]
    done_tiles = []
    events = {"tma": [], "mma": []}

    def producer():
        it = 0
        for t in range(ntiles_of_cta):
            for kb in range(nkb):
                s = it % stages
                if it >= stages:
                    yield from wait(empty[s], ((it // stages) - 1) & 1)
                assert not stage_busy[s], "stage overwritten while an MMA still reads it"

                def land(s=s, tag=(t, kb)):
                    stage_data[s] = tag
                    full[s].arrive()
                events["tma"].append(land)
                it += 1
                yield ("step",)

    def mma():
        it = 0
        for n in range(ntiles_of_cta):
            buf = n & 1
            if n >= 2:
                yield from wait(acc_empty[buf], ((n >> 1) - 1) & 1)
            assert acc_readers[buf] == 0, "accumulator overwritten while the epilogue reads it"
            for kb in range(nkb):
                s = it % stages
                yield from wait(full[s], (it // stages) & 1)
                assert stage_data[s] == (n, kb), f"MMA read {stage_data[s]} instead of {(n, kb)}"
                stage_busy[s] = True
                acc[buf] = (n, [kb]) if kb == 0 else (acc[buf][0], acc[buf][1] + [kb])

                def retire(s=s):
                    stage_busy[s] = False
                    empty[s].arrive()
                events["mma"].append(retire)
                it += 1
                yield ("step",)
            events["mma"].append(acc_full[buf].arrive)

    def epilogue(_who):
        for n in range(ntiles_of_cta):
            buf = n & 1
            yield from wait(acc_full[buf], (n >> 1) & 1)
            acc_readers[buf] += 1
            yield ("step",)
            assert acc[buf] == (n, list(range(nkb))), f"epilogue of tile {n} read {acc[buf]}"
            acc_readers[buf] -= 1
            if _who == 0:
                done_tiles.append(n)
            acc_empty[buf].arrive()

    run([producer(), mma()] + [epilogue(w) for w in range(n_epi)], events, rng)
    assert done_tiles == list(range(ntiles_of_cta))


@pytest.mark.parametrize("ntiles,nkb,stages", [(1, 1, 4), (1, 9, 4), (2, 3, 4), (5, 1, 4), (5, 6, 4), (7, 2, 3), (4, 13, 4)])
def test_persistent_gemm_pipeline(ntiles, nkb, stages):
    for seed in range(60):
        persistent_gemm(ntiles, nkb, stages, random.Random(seed))


# ---- tensor-core decode attention (csrc/attention_decode_tc.cu) ----------------------------------------
# K/V ring, double-buffered scores, TWO probability tiles and barrier pairs (p_full[c & 1], o_full[c & 1]) so that
# the softmax of chunk i runs while P*V of chunk i - 1 is still in flight; O accumulates in tensor memory and is
# only touched by the softmax threads at the (rare) rescale, behind a wait for P*V of chunk i - 1.

def attention(nchunks, stages, rng):
    kv_full = [MBar(1) for _ in range(stages)]
    kv_free = [MBar(1) for _ in range(stages)]
    s_full = [MBar(1) for _ in range(2)]
    n_sm = 2                                             # stands for the 128 softmax threads
    s_free = [MBar(n_sm) for _ in range(2)]
    p_full = [MBar(n_sm) for _ in range(2)]
    o_full = [MBar(1) for _ in range(2)]
    kv = [None] * stages
    kv_reads_pending = [0] * stages
    s_buf = [None, None]
    s_readers = [0, 0]
    p_tile = [{"chunk": None, "reads_pending": 0} for _ in range(2)]
    o_acc = {"chunks": [], "mma_pending": 0, "rescaling": 0}
    outputs = [[] for _ in range(n_sm)]
    events = {"tma": [], "mma_s": [], "mma_pv": []}      # each issuer's MMAs complete in its issue order

    def copy(c):
        s = c % stages
        assert kv_reads_pending[s] == 0, "K/V stage overwritten while an MMA still reads it"

        def land():
            kv[s] = c
            kv_full[s].arrive()
        events["tma"].append(land)

    def issue_scores(c):
        s = c % stages
        assert kv[s] == c, f"scores of chunk {c} read stage holding {kv[s]}"
        assert s_readers[c & 1] == 0, "score buffer overwritten while the softmax warps read it"
        kv_reads_pending[s] += 1

        def retire():
            s_buf[c & 1] = c
            kv_reads_pending[s] -= 1
            s_full[c & 1].arrive()
        events["mma_s"].append(retire)

    def issue_pv(c):
        s = c % stages
        assert kv[s] == c and p_tile[c & 1]["chunk"] == c, f"P*V of chunk {c}: P tile holds {p_tile[c & 1]['chunk']}"
        assert o_acc["rescaling"] == 0, "P*V issued while a softmax thread rescales O"
        kv_reads_pending[s] += 1
        p_tile[c & 1]["reads_pending"] += 1
        o_acc["mma_pending"] += 1

        def retire():
            o_acc["chunks"].append(c)
            o_acc["mma_pending"] -= 1
            kv_reads_pending[s] -= 1
            p_tile[c & 1]["reads_pending"] -= 1
            o_full[c & 1].arrive()
            kv_free[s].arrive()
        events["mma_pv"].append(retire)

    # three issuing threads: copies, score MMAs, P*V MMAs - each with its own chain of waits
    def loader():
        for c in range(min(nchunks, stages)):
            copy(c)
        for i in range(nchunks):
            if i + stages < nchunks:
                yield from wait(kv_free[i % stages], (i // stages) & 1)
                copy(i + stages)
            yield ("step",)

    def score_issuer():
        for c in range(nchunks):
            yield from wait(kv_full[c % stages], (c // stages) & 1)
            if c >= 2:
                yield from wait(s_free[c & 1], ((c >> 1) - 1) & 1)
            issue_scores(c)
            yield ("step",)

    def pv_issuer():
        for c in range(nchunks):
            yield from wait(p_full[c & 1], (c >> 1) & 1)
            yield from wait(kv_full[c % stages], (c // stages) & 1)
            issue_pv(c)
            yield ("step",)

    def softmax(who):
        for i in range(nchunks):
            buf = i & 1
            yield from wait(s_full[buf], (i >> 1) & 1)
            s_readers[buf] += 1
            yield ("step",)
            assert s_buf[buf] == i, f"softmax of chunk {i} read scores of {s_buf[buf]}"
            s_readers[buf] -= 1
            s_free[buf].arrive()
            if i >= 2:
                yield from wait(o_full[i & 1], ((i - 2) >> 1) & 1)
            if i >= 1 and rng.random() < 0.3:           # the rare rescale of O in tensor memory
                yield from wait(o_full[(i - 1) & 1], ((i - 1) >> 1) & 1)
                assert o_acc["chunks"] == list(range(i)) and o_acc["mma_pending"] == 0, "O not stable at the rescale point"
                o_acc["rescaling"] += 1
                yield ("step",)
                o_acc["rescaling"] -= 1
            assert p_tile[buf]["reads_pending"] == 0, "P tile overwritten while an MMA reads it"
            yield ("step",)
            p_tile[buf]["chunk"] = i
            outputs[who].append(i)
            p_full[buf].arrive()
        yield from wait(o_full[(nchunks - 1) & 1], ((nchunks - 1) >> 1) & 1)
        assert o_acc["chunks"] == list(range(nchunks)), f"final read saw {o_acc['chunks']}"

    run([loader(), score_issuer(), pv_issuer()] + [softmax(w) for w in range(n_sm)], events, rng)
    assert all(o == list(range(nchunks)) for o in outputs)


@pytest.mark.parametrize("nchunks,stages", [(1, 3), (2, 3), (3, 3), (4, 3), (9, 3), (16, 3), (5, 2)])
def test_attention_pipeline(nchunks, stages):
    for seed in range(60):
        attention(nchunks, stages, random.Random(seed))


def test_the_checker_sees_a_wrong_parity():
    # the same GEMM program with the classic slip in the producer's wait (parity of the current ring pass
    # instead of the previous one) must deadlock or corrupt data in at least one schedule
    def broken(rng):
        stages, nkb, ntiles = 2, 5, 2
        full = [MBar(1) for _ in range(stages)]
        empty = [MBar(1) for _ in range(stages)]
        data = [None] * stages
        events = {"tma": [], "mma": []}

        def producer():
            for it in range(ntiles * nkb):
                s = it % stages
                if it >= stages:
                    yield from wait(empty[s], (it // stages) & 1)      # wrong: should be ((it // stages) - 1) & 1

                def land(s=s, it=it):
                    data[s] = it
                    full[s].arrive()
                events["tma"].append(land)
                yield ("step",)

        def mma():
            for it in range(ntiles * nkb):
                s = it % stages
                yield from wait(full[s], (it // stages) & 1)
                assert data[s] == it
                events["mma"].append(empty[s].arrive)
                yield ("step",)

        run([producer(), mma()], events, rng)

    failures = 0
    for seed in range(40):
        try:
            broken(random.Random(seed))
        except AssertionError:
            failures += 1
    assert failures > 0


# ---- CTA-pair GEMM (csrc/gemm_pair.cu) ----------------------------------------------------------------
# Two CTAs, each with its own ring and producer. Only the LEADER's full[s] barriers are used: the leader's
# producer arms them for the bytes of both CTAs, and both CTAs' copies credit them - the peer's copy may land
# BEFORE the leader has armed the barrier for that ring pass (the transaction count goes negative for a while).
# The leader's MMA thread releases a stage in both CTAs and hands the accumulator to both epilogues.

class TxBar(MBar):
    """mbarrier with a transaction count: a phase completes when no arrival is pending and tx == 0."""

    def __init__(self, count):
        super().__init__(count)
        self.tx = 0

    def _maybe_complete(self):
        if self.pending == 0 and self.tx == 0:
            self.completed += 1
            self.pending = self.count

    def arrive_expect(self, nbytes):
        self.tx += nbytes
        self.pending -= 1
        assert self.pending >= 0
        self._maybe_complete()

    def complete_tx(self, nbytes):
        self.tx -= nbytes
        self._maybe_complete()


def pair_gemm(nkb, stages, rng):
    full = [TxBar(1) for _ in range(stages)]                       # leader's barriers
    empty = [[MBar(1) for _ in range(stages)] for _ in range(2)]   # per CTA
    acc_full = [MBar(1), MBar(1)]
    data = [[None] * stages for _ in range(2)]
    busy = [[False] * stages for _ in range(2)]
    got = []
    events = {"tma0": [], "tma1": [], "mma": []}

    def producer(rank):
        for i in range(nkb):
            s = i % stages
            if i >= stages:
                yield from wait(empty[rank][s], ((i // stages) - 1) & 1)
            assert not busy[rank][s], "stage overwritten while the MMA still reads it"
            if rank == 0:
                full[s].arrive_expect(2)                            # one unit per CTA

            def land(s=s, i=i):
                data[rank][s] = i
                full[s].complete_tx(1)
            events[f"tma{rank}"].append(land)
            yield ("step",)

    def mma():
        for i in range(nkb):
            s = i % stages
            yield from wait(full[s], (i // stages) & 1)
            assert data[0][s] == i and data[1][s] == i, f"K block {i}: stages hold {data[0][s]}, {data[1][s]}"
            busy[0][s] = busy[1][s] = True
            got.append(i)

            def retire(s=s):
                busy[0][s] = busy[1][s] = False
                empty[0][s].arrive()
                empty[1][s].arrive()
            events["mma"].append(retire)
            yield ("step",)

        def done():
            acc_full[0].arrive()
            acc_full[1].arrive()
        events["mma"].append(done)

    def epilogue(rank):
        yield from wait(acc_full[rank], 0)
        assert got == list(range(nkb))

    run([producer(0), producer(1), mma(), epilogue(0), epilogue(1)], events, rng)


@pytest.mark.parametrize("nkb,stages", [(1, 6), (6, 6), (7, 6), (25, 6), (9, 2)])
def test_cta_pair_gemm_pipeline(nkb, stages):
    for seed in range(80):
        pair_gemm(nkb, stages, random.Random(seed))


# ---- prompt attention (csrc/attention_prefill_tc.cu) ------------------------------------------------------
# K ring (freed when the scores of the chunk are complete) and V ring (freed when P*V is complete) run apart.
# Two softmax groups: group g takes the chunks g, g + 2, ... with score buffer g, its own accumulator O_g and TWO
# probability tiles (chunk i uses tile i % 4): before it overwrites the tile for chunk i it waits for the P*V product
# of chunk i - 4, and before the rare rescale of O_g for the product of chunk i - 2 (barriers pv_done[0..3], no phase
# skipped by any waiter). One more barrier, armed by both P*V issuers after their last product, tells both groups
# that both accumulators are final. Copies, the score MMAs of the even and of the odd chunks, and the P*V
# MMAs into each accumulator are issued by five threads with a chain of waits each.

def prefill_attention(nchunks, stages_k, stages_v, rng):
    k_full = [MBar(1) for _ in range(stages_k)]
    k_free = [MBar(1) for _ in range(stages_k)]
    v_full = [MBar(1) for _ in range(stages_v)]
    v_free = [MBar(1) for _ in range(stages_v)]
    s_full = [MBar(1) for _ in range(2)]
    n_sm = 2                                             # stands for the 128 softmax threads of a group
    s_free = [MBar(n_sm) for _ in range(2)]
    p_full = [MBar(n_sm) for _ in range(4)]             # chunk c uses probability tile c % 4: two tiles per group
    pv_done = [MBar(1) for _ in range(4)]
    o_final = MBar(2)                                   # one arrival per P*V issuer
    turn = [MBar(2 * n_sm) for _ in range(2)]           # named barriers: group g's turn at the exponentials
    in_exp = [0, 0]
    kbuf, vbuf = [None] * stages_k, [None] * stages_v
    k_reads, v_reads = [0] * stages_k, [0] * stages_v
    s_buf, s_readers = [None, None], [0, 0]
    p_tile = [{"rows": [None] * n_sm, "reads_pending": 0} for _ in range(4)]
    o_acc = [{"chunks": [], "mma_pending": 0, "rescaling": 0} for _ in range(2)]
    seen = [[[] for _ in range(n_sm)] for _ in range(2)]
    events = {"tma": [], "mma_s0": [], "mma_s1": [], "mma_pv0": [], "mma_pv1": []}   # an issuer's MMAs complete in its issue order

    def load_k(c):
        s = c % stages_k
        assert k_reads[s] == 0, "K stage overwritten while the score MMAs still read it"

        def land():
            kbuf[s] = c
            k_full[s].arrive()
        events["tma"].append(land)

    def load_v(c):
        s = c % stages_v
        assert v_reads[s] == 0, "V stage overwritten while the P*V MMAs still read it"

        def land():
            vbuf[s] = c
            v_full[s].arrive()
        events["tma"].append(land)

    def issue_scores(c):
        s = c % stages_k
        assert kbuf[s] == c and s_readers[c & 1] == 0
        k_reads[s] += 1

        def retire():
            s_buf[c & 1] = c
            k_reads[s] -= 1
            s_full[c & 1].arrive()
            k_free[s].arrive()
        events["mma_s%d" % (c & 1)].append(retire)

    def issue_pv(c):
        s = c % stages_v
        t, o = p_tile[c & 3], o_acc[c & 1]
        assert vbuf[s] == c and t["rows"] == [c] * n_sm, f"P*V of chunk {c}: V holds {vbuf[s]}, P holds {t['rows']}"
        assert o["rescaling"] == 0, "P*V issued while a softmax thread rescales its accumulator"
        v_reads[s] += 1
        t["reads_pending"] += 1
        o["mma_pending"] += 1

        def retire():
            o["chunks"].append(c)
            o["mma_pending"] -= 1
            v_reads[s] -= 1
            t["reads_pending"] -= 1
            pv_done[c & 3].arrive()
            v_free[s].arrive()
            if c + 2 >= nchunks:
                o_final.arrive()
        events["mma_pv%d" % (c & 1)].append(retire)

    def loader():
        for c in range(min(nchunks, stages_k)):
            load_k(c)
        for c in range(min(nchunks, stages_v)):
            load_v(c)
        for j in range(nchunks + 2):
            if j + stages_k < nchunks:
                yield from wait(k_free[j % stages_k], (j // stages_k) & 1)
                load_k(j + stages_k)
            i = j - 2
            if i >= 0 and i + stages_v < nchunks:
                yield from wait(v_free[i % stages_v], (i // stages_v) & 1)
                load_v(i + stages_v)
            yield ("step",)

    def score_issuer(first):
        for c in range(first, nchunks, 2):
            yield from wait(k_full[c % stages_k], (c // stages_k) & 1)
            if c >= 2:
                yield from wait(s_free[c & 1], ((c >> 1) - 1) & 1)
            issue_scores(c)
            yield ("step",)

    def pv_issuer(first):
        for c in range(first, nchunks, 2):
            yield from wait(p_full[c & 3], (c >> 2) & 1)
            yield from wait(v_full[c % stages_v], (c // stages_v) & 1)
            issue_pv(c)
            yield ("step",)

    def softmax(g, who):
        mine = list(range(g, nchunks, 2))
        if g == 1:
            turn[0].arrive()                            # group 0 has the first turn
        for it, i in enumerate(mine):
            yield from wait(s_full[g], (i >> 1) & 1)
            s_readers[g] += 1
            yield ("step",)
            assert s_buf[g] == i, f"softmax of chunk {i} read scores of {s_buf[g]}"
            s_readers[g] -= 1
            s_free[g].arrive()
            if i >= 2 and rng.random() < 0.3:           # the rare rescale of O_g: the group's latest product must be done
                yield from wait(pv_done[(i - 2) & 3], ((i - 2) >> 2) & 1)
                assert o_acc[g]["chunks"] == list(range(g, i, 2)) and o_acc[g]["mma_pending"] == 0, "O_g not stable"
                o_acc[g]["rescaling"] += 1
                yield ("step",)
                o_acc[g]["rescaling"] -= 1
            if i >= 4:
                yield from wait(pv_done[i & 3], ((i >> 2) - 1) & 1)
            turn[g].arrive()                            # bar.sync: arrive and wait for the phase
            yield from wait(turn[g], it & 1)
            assert in_exp[g ^ 1] == 0, "both groups in their exponential phase"
            in_exp[g] += 1
            assert p_tile[i & 3]["reads_pending"] == 0, "P tile overwritten while an MMA reads it"
            yield ("step",)
            p_tile[i & 3]["rows"][who] = i
            seen[g][who].append(i)
            in_exp[g] -= 1
            if g == 0 or i + 2 < nchunks:
                turn[g ^ 1].arrive()                    # bar.arrive: the other group's turn
            p_full[i & 3].arrive()
        yield from wait(o_final, 0)
        assert o_acc[0]["chunks"] == list(range(0, nchunks, 2)) and o_acc[1]["chunks"] == list(range(1, nchunks, 2))
        assert o_acc[0]["mma_pending"] == 0 and o_acc[1]["mma_pending"] == 0

    run([loader(), score_issuer(0), score_issuer(1), pv_issuer(0), pv_issuer(1)] + [softmax(g, w) for g in range(2) for w in range(n_sm)], events, rng)
    for g in range(2):
        assert all(x == list(range(g, nchunks, 2)) for x in seen[g])


@pytest.mark.parametrize("stages", [(2, 2), (2, 3), (4, 4)])
@pytest.mark.parametrize("nchunks", [2, 4, 6, 8, 16, 32])
def test_prefill_attention_pipeline(nchunks, stages):
    for seed in range(40):
        prefill_attention(nchunks, stages[0], stages[1], random.Random(seed))


# ---- persistent CTA-pair GEMM: tile loop and accumulator hand-back ------------------------------------------

def pair_gemm_persistent(ntiles, nkb, stages, rng):
    full = [TxBar(1) for _ in range(stages)]
    empty = [[MBar(1) for _ in range(stages)] for _ in range(2)]
    acc_full = [[MBar(1), MBar(1)] for _ in range(2)]               # [cta][buffer]
    n_warps = 2                                                      # stands for the four epilogue warps of a CTA
    acc_empty = [MBar(2 * n_warps) for _ in range(2)]                # leader's, arrivals from both CTAs
    data = [[None] * stages for _ in range(2)]
    busy = [[False] * stages for _ in range(2)]
    acc = [None, None]
    readers = [0, 0]
    stored = {(r, w): [] for r in range(2) for w in range(n_warps)}
    events = {"tma0": [], "tma1": [], "mma": []}

    def producer(rank):
        it = 0
        for t in range(ntiles):
            for kb in range(nkb):
                s = it % stages
                if it >= stages:
                    yield from wait(empty[rank][s], ((it // stages) - 1) & 1)
                assert not busy[rank][s]
                if rank == 0:
                    full[s].arrive_expect(2)

                def land(s=s, tag=(t, kb)):
                    data[rank][s] = tag
                    full[s].complete_tx(1)
                events[f"tma{rank}"].append(land)
                it += 1
                yield ("step",)

    def mma():
        it = 0
        for n in range(ntiles):
            buf = n & 1
            if n >= 2:
                yield from wait(acc_empty[buf], ((n >> 1) - 1) & 1)
            assert readers[buf] == 0, "accumulator overwritten while an epilogue warp reads it"
            for kb in range(nkb):
                s = it % stages
                yield from wait(full[s], (it // stages) & 1)
                assert data[0][s] == (n, kb) and data[1][s] == (n, kb)
                busy[0][s] = busy[1][s] = True
                acc[buf] = (n, [kb]) if kb == 0 else (acc[buf][0], acc[buf][1] + [kb])

                def retire(s=s):
                    busy[0][s] = busy[1][s] = False
                    empty[0][s].arrive()
                    empty[1][s].arrive()
                events["mma"].append(retire)
                it += 1
                yield ("step",)

            def done(buf=buf):
                acc_full[0][buf].arrive()
                acc_full[1][buf].arrive()
            events["mma"].append(done)

    def epilogue(rank, w):
        for n in range(ntiles):
            buf = n & 1
            yield from wait(acc_full[rank][buf], (n >> 1) & 1)
            readers[buf] += 1
            yield ("step",)
            assert acc[buf] == (n, list(range(nkb))), f"epilogue of tile {n} read {acc[buf]}"
            readers[buf] -= 1
            stored[(rank, w)].append(n)
            acc_empty[buf].arrive()

    run([producer(0), producer(1), mma()] + [epilogue(r, w) for r in range(2) for w in range(n_warps)], events, rng)
    assert all(v == list(range(ntiles)) for v in stored.values())


@pytest.mark.parametrize("ntiles,nkb,stages", [(1, 1, 6), (2, 7, 6), (3, 2, 6), (5, 1, 6), (6, 9, 6), (4, 3, 2)])
def test_persistent_cta_pair_gemm_pipeline(ntiles, nkb, stages):
    for seed in range(60):
        pair_gemm_persistent(ntiles, nkb, stages, random.Random(seed))


# ---- push epilogue of the persistent fused GEMM (csrc/gemm_fused_persist.cu) --------------------------------
# The four epilogue warps transpose 16 tokens at a time through one of TWO shared-memory buffers with ONE named
# barrier per step: write buffer (step & 1), barrier, read it. A thread can write the buffer of step k + 2 only after
# it passed the barrier of step k + 1, which every thread reaches only after its reads of step k.

def push_epilogue(nthreads, nsteps, nbuffers, rng):
    bar = MBar(nthreads)
    cells = [[None] * nthreads for _ in range(nbuffers)]          # cells[buffer][writer] = step it holds
    unread = [[0] * nthreads for _ in range(nbuffers)]            # reads still owed on the cell's current content
    seen = [[] for _ in range(nthreads)]

    def thread(me):
        for k in range(nsteps):
            b = k % nbuffers
            assert unread[b][me] == 0, f"step {k}: buffer {b} overwritten while {unread[b][me]} readers still owe a read"
            cells[b][me] = k
            unread[b][me] = nthreads
            yield ("step",)
            bar.arrive()
            yield from wait(bar, k & 1)
            for w in rng.sample(range(nthreads), nthreads):
                assert cells[b][w] == k, f"step {k}: thread {me} read step {cells[b][w]} of writer {w}"
                unread[b][w] -= 1
                yield ("step",)
            seen[me].append(k)

    run([thread(i) for i in range(nthreads)], {}, rng)
    assert all(s == list(range(nsteps)) for s in seen)


@pytest.mark.parametrize("nsteps", [1, 2, 3, 8, 17])
def test_push_epilogue_two_buffers_one_barrier(nsteps):
    for seed in range(40):
        push_epilogue(4, nsteps, 2, random.Random(seed))


def test_push_epilogue_one_buffer_would_race():
    """The model does see the race that a single buffer with one barrier per step has."""
    hits = 0
    for seed in range(40):
        try:
            push_epilogue(4, 6, 1, random.Random(seed))
        except AssertionError:
            hits += 1
    assert hits > 0
