"""Failure detection on the host: a rank that dies or leaves between steps is noticed by the others before their next
collective, through the heartbeat table (gloo ranks on the CPU; nothing here touches a GPU)."""
import os
import socket
import time

import pytest
import torch


def _free_port():
    s = socket.socket(); s.bind(("127.0.0.1", 0)); p = s.getsockname()[1]; s.close()
    return p


def _worker(rank, world, port, ns, mode, q):
    import datetime
    import torch.distributed as dist
    from recstore_b200 import ipc
    from recstore_b200.utils.liveness import Heartbeat, RankLostError
    os.environ["MASTER_ADDR"] = "127.0.0.1"; os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    ipc.set_namespace(ns)
    if mode == "store":
        store = dist.TCPStore("127.0.0.1", port + 1, world_size=None, is_master=(rank == 0), wait_for_workers=False)
        hb = Heartbeat(rank, world, period_s=0.05, backend="store", store=store)
    else:
        hb = Heartbeat(rank, world, name="hb_test", period_s=0.05)
    hb.start()
    hb.wait_all_alive(20.0)
    victim = world - 1
    steps_done, noticed_after, err = 0, None, None
    t_gone = None
    try:
        for step in range(200):
            if rank == victim and step == 3:
                # between steps, nothing in flight: the victim goes away
                if mode == "leave":
                    hb.stop(leaving=True)
                    q.put((rank, "left", step, 0.0))
                    return                                   # a clean exit of the function; the group is torn down below
                q.put((rank, "died", step, 0.0))
                q.close(); q.join_thread()
                os._exit(0)                                  # no goodbye: the word simply stops moving
            if step >= 3 and rank != victim:
                if t_gone is None:
                    t_gone = time.monotonic()
                # the survivors poll instead of entering the collective that the victim will never join
                deadline = time.monotonic() + 20
                while time.monotonic() < deadline:
                    hb.check(timeout_s=1.5)
                    time.sleep(0.02)
                raise AssertionError("the loss of the victim went unnoticed for 20 s")
            hb.check(timeout_s=1.5)
            t = torch.ones(4) * (rank + 1)
            dist.all_reduce(t)
            assert float(t[0]) == world * (world + 1) / 2
            steps_done += 1
    except RankLostError as e:
        noticed_after = time.monotonic() - t_gone
        err = (sorted(e.lost), sorted(e.left))
    hb.stop(leaving=False)
    q.put((rank, err, steps_done, noticed_after))


@pytest.mark.parametrize("mode", ["die", "leave", "store"])
def test_a_rank_that_goes_away_between_steps_is_noticed_before_the_next_collective(mode):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, port, ns = 3, _free_port(), f"pytest_hb_{os.getpid()}_{mode}"
    ps = [ctx.Process(target=_worker, args=(r, world, port, ns, mode, q)) for r in range(world)]
    [p.start() for p in ps]
    res = {}
    for _ in range(world):
        r = q.get(timeout=120)
        res[r[0]] = r[1:]
    [p.join(30) for p in ps]
    for p in ps:
        if p.is_alive():
            p.terminate()
    from recstore_b200 import ipc
    ipc.set_namespace(ns)
    ipc.IPCTensorFactory.ClearIPCMemory()                    # leave nothing in shared memory
    victim = world - 1
    assert res[victim][0] in ("died", "left")
    for r in range(world - 1):
        err, steps, noticed = res[r]
        assert steps == 3, res                               # the three common steps ran, nobody entered a fourth
        if mode == "leave":
            assert err == ([], [victim]), res
        else:       # a survivor that notices late may also miss the survivor that noticed first and has stopped already
            assert err is not None and victim in err[0] and err[1] == [], res
        assert noticed is not None and noticed < (1.0 if mode == "leave" else 8.0), res      # limit 1.5 s + slack for a loaded box


def test_heartbeat_status_unseen_left_and_context_manager():
    from recstore_b200 import ipc
    from recstore_b200.utils.liveness import Heartbeat, RankLostError
    ipc.set_namespace(f"pytest_hb1_{os.getpid()}")
    a = Heartbeat(0, 3, name="hb_unit", period_s=0.02)
    b = Heartbeat(1, 3, name="hb_unit", period_s=0.02)
    assert a.status(5.0) == {"lost": [], "left": [], "unseen": [1, 2]}
    with pytest.raises(RankLostError) as e:
        a.wait_all_alive(0.2)                                # rank 2 never shows up
    assert 2 in e.value.lost
    with b:
        time.sleep(0.1)
        st = a.status(5.0)
        assert 1 not in st["unseen"] and 1 not in st["lost"]
    assert a.status(5.0)["left"] == [1]                      # leaving the block says goodbye
    with pytest.raises(RankLostError) as e:
        a.check(5.0)
    assert e.value.left == [1] and "left the job" in str(e.value)
    b2 = Heartbeat(1, 3, name="hb_unit", period_s=0.02)      # the same rank comes back: its row starts afresh
    b2.beat()
    assert 1 not in a.status(5.0)["left"]
    b2.stop(leaving=False)
    time.sleep(0.15)
    assert 1 in a.status(0.1)["lost"]                        # silent for longer than the limit
    ipc.IPCTensorFactory.ClearIPCMemory()


def _barrier_worker(rank, world, ns, dies, q):
    from recstore_b200 import ipc
    from recstore_b200.utils.liveness import Heartbeat, RankLostError
    ipc.set_namespace(ns)
    hb = Heartbeat(rank, world, name="hb_barrier", period_s=0.05).start()
    hb.wait_all_alive(30.0)
    done = 0
    try:
        for i in range(6):
            if dies and rank == world - 1 and i == 3:
                os._exit(0)                                  # gone between barriers, without a word
            time.sleep(0.01 * rank)                          # ranks arrive at different times
            hb.barrier(timeout_s=1.5)
            done += 1
        hb.stop(leaving=False)
        q.put((rank, done, None))
    except RankLostError as e:
        hb.stop(leaving=False)
        q.put((rank, done, sorted(e.lost)))


@pytest.mark.parametrize("dies", [False, True])
def test_heartbeat_barrier_releases_together_and_cannot_hang_on_a_dead_rank(dies):
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    world, ns = 3, f"pytest_hbb_{os.getpid()}_{int(dies)}"
    ps = [ctx.Process(target=_barrier_worker, args=(r, world, ns, dies, q)) for r in range(world)]
    [p.start() for p in ps]
    expect = world - 1 if dies else world
    res = dict((r[0], r[1:]) for r in (q.get(timeout=120) for _ in range(expect)))
    [p.join(30) for p in ps]
    from recstore_b200 import ipc
    ipc.set_namespace(ns)
    ipc.IPCTensorFactory.ClearIPCMemory()
    if not dies:
        assert all(res[r] == (6, None) for r in range(world)), res
    else:
        for r in range(world - 1):
            done, lost = res[r]
            assert done == 3 and lost is not None and world - 1 in lost, res   # three common barriers, then the loss is reported
