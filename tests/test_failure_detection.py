"""CPU tests of host-side failure detection between ranks (world size 2 and 3, TCP store on 127.0.0.1):
failures are produced on the host - a rank that raises, a rank that never reports - never on a GPU."""
import os
import socket
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, scenario, out_dir):
    sys.path.insert(0, ROOT)
    import datetime

    import torch.distributed as dist

    from spork_b200.multi_gpu import RankFailure, RankHealth

    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    health = RankHealth(store, rank, world)
    launched = []
    outcome = "finished"
    try:
        for step in range(3):
            def my_part(step=step):
                if scenario == "rank1_raises_at_step1" and rank == 1 and step == 1:
                    raise RuntimeError("device status reported a timeout")
                return step

            if scenario == "rank1_silent_at_step1" and rank == 1 and step == 1:
                outcome = "went silent"
                break  # leaves between steps, nothing in flight, without reporting
            health.guard(step, my_part, timeout_s=3.0)
            launched.append(step)  # stands for the kernel launch of this step
    except RankFailure as f:
        outcome = "stopped: " + ",".join(str(r) for r in sorted(f.failed))
    except RuntimeError as e:
        outcome = "raised: " + str(e)
    with open(os.path.join(out_dir, f"rank{rank}.txt"), "w") as fh:
        fh.write(outcome + "|" + ",".join(map(str, launched)))
    if rank == 0:
        # the store lives in rank 0: keep it up until the others have written their outcome
        import time

        deadline = time.time() + 20
        while time.time() < deadline and not all(os.path.exists(os.path.join(out_dir, f"rank{r}.txt")) for r in range(world)):
            time.sleep(0.05)


def _run(scenario, world, tmp_path):
    import torch.multiprocessing as mp

    port = _free_port()
    mp.spawn(_worker, args=(world, port, scenario, str(tmp_path)), nprocs=world, join=True)
    return [open(tmp_path / f"rank{r}.txt").read().split("|") for r in range(world)]


def test_all_ranks_healthy(tmp_path):
    res = _run("healthy", 2, tmp_path)
    assert res == [["finished", "0,1,2"], ["finished", "0,1,2"]]


def test_a_rank_that_raises_stops_the_others_before_their_next_launch(tmp_path):
    res = _run("rank1_raises_at_step1", 3, tmp_path)
    assert res[1] == ["raised: device status reported a timeout", "0"]
    # ranks 0 and 2 completed step 0, learnt of the failure at step 1 and launched nothing more
    assert res[0] == ["stopped: 1", "0"]
    assert res[2] == ["stopped: 1", "0"]


def test_a_rank_that_goes_silent_is_detected_by_timeout(tmp_path):
    res = _run("rank1_silent_at_step1", 2, tmp_path)
    assert res[1] == ["went silent", "0"]
    assert res[0] == ["stopped: 1", "0"]


def test_argument_checks():
    sys.path.insert(0, ROOT)
    from spork_b200.multi_gpu import RankFailure, RankHealth

    with pytest.raises(ValueError):
        RankHealth(None, 2, 2)
    f = RankFailure(4, {1: "failed: x"})
    assert "rank 1" in str(f) and f.step == 4
