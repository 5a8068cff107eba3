"""Failure detection and elastic recovery, entirely on the host: three gloo ranks train, one exits between
steps, the survivors notice through the heartbeat store, re-rendezvous as a world of two, reload the last
checkpoint and finish; a collective against the vanished rank ends with an error, not a hang."""
import os

import pytest
import torch


def _rank_main(rank, world, store_port, base_port, q, tmpdir):
    import torch.distributed as dist
    from rust_neural_network_b200 import nn, serialize
    from rust_neural_network_b200.distributed import TcpStore
    from rust_neural_network_b200.loss import MSELoss
    from rust_neural_network_b200.optim import SGD
    from rust_neural_network_b200.parallel.elastic import ElasticGroup
    store = TcpStore(port=store_port, is_master=False, timeout=20.0)
    eg = ElasticGroup(rank, world, store, backend="gloo", base_port=base_port, heartbeat_interval=0.05, heartbeat_timeout=0.5, pg_timeout=5.0)
    torch.manual_seed(0)
    model = nn.Sequential().add(nn.Linear(4, 1))
    opt = SGD(model.parameters(), lr=0.05)
    g = torch.Generator().manual_seed(100 + rank)
    x = torch.randn(8, 4, generator=g)
    y = x.sum(-1, keepdim=True)
    ckpt = os.path.join(tmpdir, "ckpt.rnnb")
    losses, events = [], []

    def step():
        opt.zero_grad()
        loss = MSELoss("mean")(model(x), y)
        loss.backward()
        for p in model.parameters():
            dist.all_reduce(p.grad)
            p.grad.div_(eg.world)
        opt.step()
        losses.append(float(loss))

    for s in range(3):
        step()
    if eg.rank == 0:
        with open(ckpt, "wb") as f:
            f.write(serialize.save_model(model))
    dist.barrier()
    if rank == 2:                       # leaves between steps, with nothing in flight
        eg.monitor.stop()
        q.put((rank, "left", losses, events))
        return
    # survivors: wait until the heartbeat of rank 2 goes stale, then shrink
    import time
    deadline = time.time() + 10
    dead = []
    while time.time() < deadline and not dead:
        time.sleep(0.1)
        dead = eg.dead_ranks()
    events.append(("dead", dead))
    eg.shrink(dead, on_reload=lambda: serialize.load_model(model, open(ckpt, "rb").read()))
    events.append(("world", eg.world, "rank", eg.rank, "gen", eg.generation))
    for s in range(5):
        step()
    t = torch.tensor([float(eg.rank + 1)])
    dist.all_reduce(t)
    events.append(("allreduce", float(t)))
    q.put((rank, "done", losses, events))
    eg.close()
    store.close()


def test_rank_loss_is_detected_and_survivors_continue(tmp_path):
    import torch.multiprocessing as mp
    from rust_neural_network_b200.distributed import TcpStore
    master = TcpStore(is_master=True)
    try:
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        procs = [ctx.Process(target=_rank_main, args=(r, 3, master.port, 29850, q, str(tmp_path))) for r in range(3)]
        for p in procs:
            p.start()
        res = {}
        for _ in procs:
            r = q.get(timeout=120)
            res[r[0]] = r
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        assert res[2][1] == "left"
        for r in (0, 1):
            _, state, losses, events = res[r]
            assert state == "done" and events[0] == ("dead", [2])
            assert events[1][:2] == ("world", 2) and events[1][5] == 1
            assert events[2] == ("allreduce", 3.0)                      # ranks renumbered 0, 1 -> 1 + 2
            assert len(losses) == 8 and losses[-1] < losses[0]
    finally:
        master.close()


def test_collective_against_a_missing_rank_errors_out(tmp_path):
    """A process-group timeout turns a collective with an absent peer into an exception (no endless wait)."""
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_lonely_rank, args=(q,))
    p.start()
    out = q.get(timeout=90)
    p.join(timeout=30)
    assert out[0] == "raised" and out[1] < 30.0


def _lonely_rank(q):
    import datetime
    import time
    import torch.distributed as dist
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "29871"})
    t0 = time.time()
    try:
        # world of two, the second rank never joins: rendezvous itself has to time out
        dist.init_process_group("gloo", rank=0, world_size=2, timeout=datetime.timedelta(seconds=3))
        t = torch.ones(1)
        dist.all_reduce(t)
        q.put(("finished", time.time() - t0))
    except Exception:
        q.put(("raised", time.time() - t0))
