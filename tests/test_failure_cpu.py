"""Host-side failure detection on Gloo ranks: a rank that leaves between steps, a rank that silently stops, and a
collective that ends with an error under a short process-group timeout.  No GPU is involved."""
import datetime
import os
import time
import traceback

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from dist_utils import free_port


def _worker(rank, world, port, mode, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank))
    torch.set_num_threads(1)
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=3))
        from adaptivetrainingsystem_b200.parallel.health import Heartbeat, RankFailure
        hb = Heartbeat(interval_s=0.05, timeout_s=0.6).start()
        x = torch.ones(4)
        for _ in range(3):  # three healthy "steps"
            hb.check()
            dist.all_reduce(x)
        if mode == "leave":
            if rank == world - 1:
                hb.leave()  # orderly departure between steps: nothing in flight
                q.put((rank, "left", 0.0))
                time.sleep(1.5)  # keep the process (and, for rank 0, the store) alive while the others find out
                return
            t0 = time.monotonic()
            while time.monotonic() - t0 < 5.0:
                try:
                    hb.check()
                except RankFailure as e:
                    q.put((rank, "detected", time.monotonic() - t0, e.left, e.lost))
                    return
                time.sleep(0.02)
            q.put((rank, "missed", 5.0))
        elif mode == "silent":
            if rank == world - 1:
                hb.stop()  # no announcement: what a hung or crashed rank looks like
                q.put((rank, "stopped", 0.0))
                time.sleep(2.5)
                return
            t0 = time.monotonic()
            while time.monotonic() - t0 < 6.0:
                try:
                    hb.check()
                except RankFailure as e:
                    q.put((rank, "detected", time.monotonic() - t0, e.left, e.lost))
                    return
                time.sleep(0.02)
            q.put((rank, "missed", 6.0))
        elif mode == "collective":
            if rank == world - 1:
                q.put((rank, "absent", 0.0))
                time.sleep(5.0)  # never joins the next collective
                return
            t0 = time.monotonic()
            try:
                dist.all_reduce(x)
                q.put((rank, "no error", time.monotonic() - t0))
            except Exception as e:  # the short process-group timeout ends the collective with an error
                q.put((rank, "error", time.monotonic() - t0, type(e).__name__))
    except Exception:
        q.put((rank, "crash", traceback.format_exc()))


def _run(mode, world=2):
    ctx = mp.get_context("spawn")
    q = ctx.SimpleQueue()
    port = free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(60)
    for p in procs:
        if p.is_alive():
            p.terminate()
    out = []
    while not q.empty():
        out.append(q.get())
    return out


@pytest.mark.dist
def test_rank_that_leaves_between_steps_is_detected_on_the_host():
    out = _run("leave")
    assert not [o for o in out if o[1] == "crash"], out
    det = [o for o in out if o[1] == "detected"]
    assert len(det) == 1 and det[0][0] == 0 and det[0][3] == [1] and det[0][2] < 2.0, out


@pytest.mark.dist
def test_rank_that_stops_beating_is_detected_after_the_timeout():
    out = _run("silent")
    assert not [o for o in out if o[1] == "crash"], out
    det = [o for o in out if o[1] == "detected"]
    assert len(det) == 1 and det[0][4] == [1] and 0.3 < det[0][2] < 4.0, out


@pytest.mark.dist
def test_collective_without_a_peer_ends_with_an_error_within_the_group_timeout():
    out = _run("collective")
    assert not [o for o in out if o[1] == "crash"], out
    err = [o for o in out if o[1] == "error"]
    assert len(err) == 1 and err[0][2] < 20.0, out
