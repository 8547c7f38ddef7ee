"""Two-rank NCCL runs of the distributed groupby (skipped on a single-GPU box): both strategies must
equal the oracle on the union of the ranks' rows."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
sys.path.insert(0, os.environ["B2_ROOT"])
import numpy as np, torch, torch.distributed as dist
import workloads, cudf_b200 as cb
from cudf_b200.aggregation import Aggregation
from cudf_b200.distributed import DistributedGroupBy
from cudf_b200.types import HostColumn, Kind, TypeId
from oracle import oracle
from tests import helpers as H
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(rank)
dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
# native = the whole plan inside the library (b2_groupby_aggregate_multi); python = torch.distributed collectives
# between library calls; C3 with 300K rows holds ~30K groups per destination: more than a 16384-record chunk,
# so both forms take their exact-size fallback over NCCL; string keys (C5): the partial aggregates travel as a table
# table_variant 6: the local pass takes the partitioned path (as it does by itself from half a million groups), whose
# group list is packed by owner instead of a table
for config, strategy, n, python_exchange, variant in (
        (2, "partials", 200_000, False, 0), (2, "partials", 200_000, True, 0), (4, "partials", 200_000, False, 0),
        (3, "partials", 300_000, False, 0), (3, "partials", 300_000, True, 0), (3, "rows", 150_000, False, 0),
        (5, "rows", 40_000, False, 0), (5, "partials", 40_000, False, 0),
        (4, "partials", 200_000, False, 6), (3, "partials", 300_000, False, 6),
        (1, "partials", 200_000, False, 0)):   # Σ, n of one FLOAT64 column: the lean kernel's fixed-point limbs
    shards = [workloads.make(config, n, rank=r, scale_domain=(config in (3, 4))) for r in range(world)]
    w = shards[rank]
    keys = cb.Table([cb.Column.from_host(k) for k in w.keys])
    cache = {}
    reqs = []
    for v, aggs in w.requests:
        cache.setdefault(id(v), cb.Column.from_host(v))
        reqs.append(cb.GroupByRequest(cache[id(v)], [Aggregation(Kind(a)) for a in aggs]))
    filt = [cache[id(f)] for f in w.row_filters]
    dgb = DistributedGroupBy(keys, w.null_policy, strategy=strategy, row_filters=filt, python_exchange=python_exchange,
                             table_variant=variant)
    okeys, ores = dgb.aggregate(reqs)
    mine = ([c.to_host() for c in okeys.columns()], [[c.to_host() for c in t.columns()] for t in ores])
    # a second call on the same object sizes its tables from the first and must give the same groups
    okeys2, ores2 = dgb.aggregate(reqs)
    again = ([c.to_host() for c in okeys2.columns()], [[c.to_host() for c in t.columns()] for t in ores2])
    o1, o2 = H.sort_order(mine[0]), H.sort_order(again[0])
    H.assert_keys_equal(again[0], mine[0], o2, o1)
    for (v, _), t1, t2 in zip(w.requests, mine[1], again[1]):
        # the order of the atomic additions differs between two runs: fp32 sources are summed in short fp32
        # partial sums (a few ulps of fp32 apart), everything else in fp64
        rt = 1e-5 if v.type_id == TypeId.FLOAT32 else 1e-9
        for c1, c2 in zip(t1, t2):
            assert np.array_equal(c1.valid()[o1], c2.valid()[o2])
            a, b = c1.values()[o1][c1.valid()[o1]], c2.values()[o2][c2.valid()[o2]]
            if a.dtype.kind == "f":
                assert np.allclose(a, b, rtol=rt, atol=rt * (np.abs(a).max() if a.size else 1.0), equal_nan=True)
            else:
                assert np.array_equal(a, b)
    gathered = [None] * world
    dist.all_gather_object(gathered, mine)
    if rank == 0:
        # union of the ranks' (disjoint) groups against the oracle on the concatenated input
        def cat(cols):
            if cols[0].type_id == TypeId.STRING:
                return HostColumn.from_strings([x for c in cols for x in c.to_pylist()], large_offsets=True)
            valid = np.concatenate([c.valid() for c in cols]) if any(c.mask is not None for c in cols) else None
            return HostColumn.from_numpy(np.concatenate([c.values() for c in cols]), valid, type_id=cols[0].type_id)
        got_keys = [cat([g[0][k] for g in gathered]) for k in range(len(w.keys))]
        got_res = [[cat([g[1][q][a] for g in gathered]) for a in range(len(w.requests[q][1]))] for q in range(len(w.requests))]
        full_keys = [cat([s.keys[k] for s in shards]) for k in range(len(w.keys))]
        vals = {}
        full_reqs = []
        for q, (v, aggs) in enumerate(w.requests):
            full_reqs.append((cat([s.requests[q][0] for s in shards]), aggs))
        full_filt = [cat([s.row_filters[i] for s in shards]) for i in range(len(w.row_filters))]
        fm = [f.mask for f in full_filt if f.mask is not None]
        exp = oracle.groupby(full_keys, full_reqs, w.null_policy, row_filters=fm)
        H.assert_same_result((got_keys, got_res), exp, full_reqs, check_nullable=False,
                             scales=H.result_scales(full_keys, full_reqs, w.null_policy, fm))
        print(f"config {config} strategy {strategy} {'python' if python_exchange else 'native'} exchange"
              f"{', partitioned local pass' if variant == 6 else ''}: {got_keys[0].size} groups OK", flush=True)
dist.barrier()
dist.destroy_process_group()
'''


def test_two_rank_distributed_groupby_matches_oracle(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, B2_ROOT=ROOT, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, timeout=600, env=env, cwd=ROOT)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("OK") == 11
    log_dir = os.environ.get("B2_TEST_LOG_DIR")   # keep rank 0's summary lines where the caller collects its logs
    if log_dir and os.path.isdir(log_dir):
        with open(os.path.join(log_dir, "two_rank_worker.log"), "w", encoding="utf-8") as f:
            f.write("".join(ln + "\n" for ln in out.stdout.splitlines() if ln.endswith("OK")))
