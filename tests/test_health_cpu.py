"""Rank-loss detection without any GPU: gloo-less child processes share a TCPStore; one of them stops
beating (exits) and the others must notice within the timeout, between steps."""
import multiprocessing as mp
import socket
import time

import pytest


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, die_rank, q):
    from datetime import timedelta
    from torch.distributed import TCPStore
    from phaseshift_b200.parallel.health import PeerMonitor, RankLostError
    store = TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=timedelta(seconds=20), wait_for_workers=True)
    mon = PeerMonitor(store, rank, world, interval_s=0.05, timeout_s=0.6).start()
    t0 = time.monotonic()
    steps = 0
    try:
        while time.monotonic() - t0 < 8.0:
            mon.assert_alive()               # "before the next launch"
            steps += 1
            time.sleep(0.02)
            if rank == die_rank and steps == 20:
                mon.stop()                    # leaves between steps: no more heartbeats
                q.put((rank, "left", steps))
                time.sleep(3.0)               # keep the process (and a rank-0 store) alive while the others notice
                return
        q.put((rank, "no-detection", steps))
    except RankLostError as e:
        q.put((rank, "detected", e.ranks))
        if rank == 0:
            time.sleep(1.5)                   # the store lives in rank 0: let the others finish reading it


@pytest.mark.timeout(60)
@pytest.mark.parametrize("die_rank", [1, 2])
def test_peers_detect_a_rank_that_stops(die_rank):
    ctx = mp.get_context("spawn")
    world, port = 3, _free_port()
    q = ctx.Queue()
    ps = [ctx.Process(target=_rank, args=(r, world, port, die_rank, q)) for r in range(world)]
    for p in ps:
        p.start()
    res = {}
    for _ in range(world):
        r, what, info = q.get(timeout=40)
        res[r] = (what, info)
    for p in ps:
        p.join(timeout=20)
    assert res[die_rank][0] == "left"
    for r in range(world):
        if r != die_rank:
            assert res[r] == ("detected", [die_rank]), res


def test_monitor_with_fake_store_reports_only_stale_peers():
    from phaseshift_b200.parallel.health import PeerMonitor, RankLostError

    class Store(dict):
        def set(self, k, v): self[k] = v
        def get(self, k): return self[k].encode()

    st = Store()
    mon = PeerMonitor(st, 0, 3, interval_s=0.02, timeout_s=0.25).start()
    try:
        t0 = time.monotonic()
        i = 0
        while time.monotonic() - t0 < 0.8:
            i += 1
            st.set("ps_hb/1", str(i))          # rank 1 keeps beating, rank 2 never shows up
            time.sleep(0.02)
        assert mon.lost() == [2]
        with pytest.raises(RankLostError):
            mon.assert_alive()
    finally:
        mon.stop()
