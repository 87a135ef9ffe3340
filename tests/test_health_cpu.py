"""Host-side failure detection with CPU ranks: a rank that leaves between steps is noticed by the
others before their next launch; a rank that goes silent is noticed by heartbeat age. The failure
is made on the host (a process that returns); nothing runs on a GPU."""
import time
from datetime import timedelta

import torch.distributed as dist
import torch.multiprocessing as mp

from test_multiprocess_cpu import free_port


def _member(rank, world, port, q, scenario):
    from torch_dist_ext_b200.parallel.health import Membership, PeerLeft

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20))
    # the announced departure must be noticed through the announcement: a generous heartbeat age keeps a slow
    # machine (process start-up under load) from reporting a stale peer first
    m = Membership(rank, world, store=store, max_age_s=1.0 if scenario == "silent" else 10.0)
    store.add("ready", 1)
    while int(store.add("ready", 0)) < world:
        time.sleep(0.01)
    steps = 0
    try:
        for step in range(200):
            if scenario == "leave" and rank == 1 and step == 3:
                m.leave("done early")
                q.put((rank, "left", steps))
                store.add("acks", 0)
                # stay until the others have noticed, so that the store outlives the test
                while int(store.add("acks", 0)) < world - 1:
                    time.sleep(0.01)
                return
            if scenario == "silent" and rank == 1 and step == 3:
                time.sleep(3.0)      # stops beating without announcing
                q.put((rank, "silent", steps))
                return
            m.check()
            steps += 1
            time.sleep(0.02)
        q.put((rank, "finished", steps))
    except PeerLeft as e:
        store.add("acks", 1)
        q.put((rank, "peer-left", str(e)))
        if rank == 0:
            time.sleep(3.5)          # keep the store alive for the others


def _run(scenario):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = free_port()
    procs = [ctx.Process(target=_member, args=(r, 3, port, q, scenario)) for r in range(3)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(3):
        r, what, info = q.get(timeout=60)
        got[r] = (what, info)
    for p in procs:
        p.join(timeout=30)
    return got


def test_announced_departure_is_seen_before_the_next_step():
    got = _run("leave")
    assert got[1][0] == "left"
    assert got[0][0] == "peer-left" and "[1]" in got[0][1]
    assert got[2][0] == "peer-left"


def test_silent_rank_is_caught_by_heartbeat_age():
    got = _run("silent")
    assert got[0][0] == "peer-left" and got[2][0] == "peer-left"
