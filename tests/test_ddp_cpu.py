"""Data-parallel gradient exchange logic on CPU ranks (gloo, world_size 2): bucket layout, issue order,
sum over ranks, and that a rank failing before the exchange surfaces as an error on its peer instead of a hang."""
import os
import socket
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, q):
    sys.path.insert(0, ROOT)
    import datetime

    from mograd_b200.train import ParamStore, _Model

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    try:
        m = _Model(torch.float32, "cpu", None, world_size=world, process_group=dist.group.WORLD, bucket_bytes=4 * 1000)
        for i in range(5):
            m.store.declare(f"p{i}", (37, 19))
        m.store.allocate()
        m._setup_buckets()
        m.store.g.copy_(torch.arange(m.store.size, dtype=torch.float32) * (rank + 1))
        if mode == "fail" and rank == 1:
            raise RuntimeError("rank 1 leaves before the exchange")
        # gradients become final from the end of the buffer backwards, one parameter at a time
        for i in range(4, -1, -1):
            m._grads_ready_down_to(m.store.range[f"p{i}"][0])
        m._finish_exchange()
        want = torch.arange(m.store.size, dtype=torch.float32) * sum(r + 1 for r in range(world))
        ok = torch.equal(m.store.g, want)
        covered = sorted(m.exchanged)
        contiguous = covered[0][0] == 0 and covered[-1][1] == m.store.size and all(
            a[1] == b[0] for a, b in zip(covered, covered[1:]))
        descending = all(a[0] >= b[0] for a, b in zip(m.exchanged, m.exchanged[1:]))
        q.put((rank, "ok" if (ok and contiguous and descending) else f"bad {ok} {contiguous} {descending}"))
    except Exception as e:  # reported to the parent, never swallowed
        q.put((rank, f"error: {type(e).__name__}"))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:
            pass


def _run(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    out = dict(q.get(timeout=120) for _ in range(2))
    for p in procs:
        p.join(timeout=60)
    return out


def test_bucketed_allreduce_sums_and_covers_the_buffer():
    assert _run("ok") == {0: "ok", 1: "ok"}


def test_peer_failure_surfaces_as_error_not_hang():
    out = _run("fail")
    assert out[1].startswith("error")
    assert out[0].startswith("error")  # rank 0's all_reduce times out / connection closed
