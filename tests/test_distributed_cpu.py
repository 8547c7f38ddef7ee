"""World-size-2 gloo tests (CPU) of the host side of the multi-GPU path: the count exchange, the
variable-size all-to-all of destination-major buffers and the exchange plan."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cudf_b200 import distributed as D


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _records_for(src: int, dst: int, n: int, words: int) -> np.ndarray:
    """Deterministic fake partial records sent from rank src to rank dst: [key, cells...] uint64."""
    base = np.arange(n * words, dtype=np.uint64).reshape(n, words)
    return base + np.uint64(1_000_000 * src + 1_000 * dst)


def _worker(rank, world, port, words, counts_matrix, result_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        send_counts = counts_matrix[rank]
        chunks = [_records_for(rank, d, send_counts[d], words) for d in range(world)]
        flat = np.concatenate([c.reshape(-1) for c in chunks]) if sum(send_counts) else np.zeros(0, np.uint64)
        buf = torch.from_numpy(flat.view(np.uint8).copy())
        recv_counts = D.exchange_counts(send_counts, buf.device)
        assert recv_counts == [counts_matrix[s][rank] for s in range(world)]
        out, n = D.exchange_records(buf, send_counts, words * 8)
        got = out.numpy().view(np.uint64).reshape(-1, words) if n else np.zeros((0, words), np.uint64)
        exp = np.concatenate([_records_for(s, rank, counts_matrix[s][rank], words) for s in range(world)])
        assert n == exp.shape[0]
        assert np.array_equal(got, exp)
        # a second exchange with different sizes on the same group (buffers are not reused across calls)
        out2 = D.exchange_buffer(buf, send_counts, recv_counts, words * 8)
        assert torch.equal(out, out2)
        result_queue.put((rank, "ok"))
    except Exception as e:  # pragma: no cover
        result_queue.put((rank, repr(e)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("counts_matrix", [[[3, 5], [2, 0]], [[0, 0], [0, 7]], [[1000, 1], [4, 2500]]])
def test_exchange_of_partial_records_world2(counts_matrix):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, 3, counts_matrix, q)) for r in range(2)]
    for p in procs:
        p.start()
    results = [q.get(timeout=120) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    assert sorted(results) == [(0, "ok"), (1, "ok")], results


def test_plan_exchange_offsets():
    ins, outs, offs = D.plan_exchange([2, 0, 5], [1, 4, 0], 24)
    assert ins == [48, 0, 120] and outs == [24, 96, 0] and offs == [0, 1, 5, 5]


def test_single_process_falls_back_to_local_groupby_path():
    # with no process group a DistributedGroupBy is a plain GroupBy: nothing to exchange
    assert not dist.is_initialized()


def _status_worker(rank, world, port, failing_rank, result_queue):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        ok = D.agree_on_status(rank != failing_rank, torch.device("cpu"))
        # whatever happened, every rank is still in step: a following collective completes
        t = torch.tensor([rank + 1])
        dist.all_reduce(t)
        result_queue.put((rank, ok, int(t.item())))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("failing_rank", [-1, 0, 1])
def test_a_failing_rank_is_seen_by_every_rank(failing_rank):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_status_worker, args=(r, 2, port, failing_rank, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = sorted(q.get(timeout=120) for _ in procs)
    for p in procs:
        p.join(timeout=60)
    assert [g[1] for g in got] == [failing_rank < 0] * 2
    assert [g[2] for g in got] == [3, 3]
