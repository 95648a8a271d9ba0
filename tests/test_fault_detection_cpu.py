"""Host-side failure detection among real gloo ranks: a rank that leaves between steps (nothing of it in flight) is
reported to the survivors through the process group's store before they launch anything else.  No GPU is involved
and nothing is made to fault or hang."""
import os
import socket
import time

import pytest

import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, leaver, out_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from llm_systems_from_scratch_b200.utils.watchdog import Heartbeat, RankFailure
    store = dist.distributed_c10d._get_default_store()
    hb = Heartbeat(store, rank, world, interval=0.1, timeout=1.0).start()
    result = "finished"
    t_detect = None
    try:
        for step in range(200):
            hb.check()                        # between steps, before anything is launched
            if step < 3:
                t = torch.ones(4) * (rank + 1)
                dist.all_reduce(t)            # every rank is still here: the collective completes
                assert t[0].item() == world * (world + 1) / 2
            if rank == leaver and step == 2:
                hb.stop()                     # leaves between steps without saying goodbye (no mark_done)
                result = "left"
                return
            if step >= 3:
                time.sleep(0.05)              # survivors: host-side work only, the next collective is never entered
    except RankFailure as e:
        result = f"detected:{e.dead}"
        t_detect = time.time()
    finally:
        with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
            f.write(f"{result}|{t_detect}")
        if result != "left":
            hb.stop()
        # no destroy_process_group: a collective shutdown would wait for the rank that left


def test_heartbeat_reports_a_rank_that_left_between_steps(tmp_path):
    world, leaver = 3, 2
    t0 = time.time()
    mp.spawn(_rank, args=(world, _free_port(), leaver, str(tmp_path)), nprocs=world, join=True)
    res = {r: open(tmp_path / f"r{r}.txt").read().split("|") for r in range(world)}
    assert res[leaver][0] == "left"
    for r in range(world):
        if r != leaver:
            assert res[r][0] == f"detected:[{leaver}]", res
            assert float(res[r][1]) - t0 < 30.0


def test_heartbeat_done_rank_is_not_a_failure(tmp_path):
    """A rank that finished and said so (mark_done) is never reported, however long ago it stopped beating."""
    from llm_systems_from_scratch_b200.utils.watchdog import Heartbeat
    store = dist.TCPStore("127.0.0.1", _free_port(), 1, True)
    now = [1000.0]
    a = Heartbeat(store, 0, 2, interval=10, timeout=1.0, clock=lambda: now[0])
    b = Heartbeat(store, 1, 2, interval=10, timeout=1.0, clock=lambda: now[0])
    b.mark_done()
    now[0] += 100.0
    a.check()
    assert a.silent_ranks() == []


def test_heartbeat_late_rank_and_dropped_key_on_a_real_store():
    """Two more failures made on the host, against a real TCPStore: a rank whose heartbeat stalls is reported while it
    is silent and no longer once it beats again (a late rank is not a dead one); a rank whose key has been dropped
    from the store is reported at once - the check must not sit in the store's own wait for a missing key."""
    from llm_systems_from_scratch_b200.utils.watchdog import Heartbeat, RankFailure
    store = dist.TCPStore("127.0.0.1", _free_port(), 1, True)
    now = [1000.0]
    a = Heartbeat(store, 0, 3, interval=10, timeout=2.0, clock=lambda: now[0])
    b = Heartbeat(store, 1, 3, interval=10, timeout=2.0, clock=lambda: now[0])
    c = Heartbeat(store, 2, 3, interval=10, timeout=2.0, clock=lambda: now[0])
    a.check()
    now[0] += 5.0           # b and c stall (nobody beats); a beats
    a.beat()
    with pytest.raises(RankFailure) as err:
        a.check()
    assert sorted(err.value.dead) == [1, 2]
    b.beat()                # b was only late
    c.beat()
    a.check()
    store.delete_key("hb/2")
    t0 = time.time()
    with pytest.raises(RankFailure) as err:
        a.check()
    assert err.value.dead == [2] and time.time() - t0 < 5.0
