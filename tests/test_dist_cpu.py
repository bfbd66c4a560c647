"""CPU tests of the multi-rank host logic, as two gloo ranks: sharding, unique-id hand-off, timing reduction and the
averaging arithmetic (against the reference's Net::sync_weights through the oracle)."""
import os
import socket
import subprocess
import sys
import textwrap

import numpy as np
import pytest

from eddl_b200 import dist as ebd
from oracle import eddl_oracle as orc

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_rows_follow_the_reference_partitioning():
    assert [ebd.shard_rows(512, 8, r) for r in range(8)] == [(64 * r, 64 * r + 64) for r in range(8)]
    assert [ebd.shard_rows(10, 3, r) for r in range(3)] == [(0, 3), (3, 6), (6, 10)]      # last replica takes the remainder
    assert ebd.shard_rows(7, 1, 0) == (0, 7)
    with pytest.raises(ValueError):
        ebd.shard_rows(2, 4, 0)                                                          # batch smaller than the replica count
    with pytest.raises(ValueError):
        ebd.shard_rows(8, 2, 2)


def test_host_average_equals_sync_weights_arithmetic(refout):
    reps = refout["sync_reps"]
    np.testing.assert_array_equal(ebd.average_replicas_host(list(reps)), refout["sync_avg"])
    np.testing.assert_array_equal(ebd.average_replicas_host(list(reps)), orc.sync_weights(reps))


WORKER = textwrap.dedent("""
    import os, sys, json
    import numpy as np
    sys.path.insert(0, %r)
    from eddl_b200 import dist as ebd
    import torch, torch.distributed as dist
    rank, world, local = ebd.rendezvous("gloo")
    uid = ebd.share_unique_id(lambda: bytes([(7 * i + 3) %% 256 for i in range(128)]))
    s, e = ebd.shard_rows(11, world, rank)
    rng = np.random.default_rng(100 + rank)
    w = rng.standard_normal(1000).astype(np.float32)
    t = torch.from_numpy(w.copy()); dist.all_reduce(t)            # gloo sum, then the 1.0f/N multiply of sync_weights
    avg = (t.numpy() * (np.float32(1.0) / np.float32(world))).astype(np.float32)
    tmax = ebd.max_over_ranks(10.0 + rank)
    ebd.barrier()
    print(json.dumps({"rank": rank, "uid_ok": uid == bytes([(7 * i + 3) %% 256 for i in range(128)]), "shard": [s, e],
                      "avg": avg[:8].tolist(), "avg_sum": float(avg.astype(np.float64).sum()), "tmax": tmax}))
""")


def test_two_gloo_ranks(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % ROOT)
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0)); port = s.getsockname()[1]
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port),
                   OMP_NUM_THREADS="1")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        o, e = p.communicate(timeout=180)
        assert p.returncode == 0, e[-2000:]
        import json
        outs.append(json.loads(o.strip().splitlines()[-1]))
    outs.sort(key=lambda d: d["rank"])
    assert all(o["uid_ok"] for o in outs)
    assert [o["shard"] for o in outs] == [[0, 5], [5, 11]]
    assert outs[0]["tmax"] == outs[1]["tmax"] == 11.0
    ws = [np.random.default_rng(100 + r).standard_normal(1000).astype(np.float32) for r in range(2)]
    want = orc.sync_weights(np.stack(ws))
    np.testing.assert_allclose(outs[0]["avg"], want[:8], rtol=1e-6)
    assert outs[0]["avg"] == outs[1]["avg"] and abs(outs[0]["avg_sum"] - float(want.astype(np.float64).sum())) < 1e-4


LAYOUT_WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    from eddl_b200 import dist as ebd
    rank, world, local = ebd.rendezvous("gloo", timeout_s=60)
    ebd.check_same_layout([3, 5, 7])                               # agreed: passes on both
    try:
        ebd.check_same_layout([3, 5, 7] if rank == 0 else [3, 5, 8])
        print("NOT DETECTED")
    except ebd.RankFailure as e:
        print("detected on rank %%d" %% rank)
    ebd.barrier()
""")


def _spawn(script, world, ranks, port, extra_env=None):
    procs = []
    for r in ranks:
        env = dict(os.environ, RANK=str(r), WORLD_SIZE=str(world), LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), OMP_NUM_THREADS="1")
        env.update(extra_env or {})
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    return procs


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ranks_that_disagree_on_the_tensor_sizes_are_stopped_on_the_host(tmp_path):
    """A size mismatch between ranks is found by a host-side comparison over gloo and raised on every rank, before any
    collective is enqueued (a mismatched collective would wait for ever)."""
    script = tmp_path / "layout.py"
    script.write_text(LAYOUT_WORKER % ROOT)
    for p in _spawn(script, 2, (0, 1), _free_port()):
        o, e = p.communicate(timeout=180)
        assert p.returncode == 0, e[-2000:]
        assert "detected on rank" in o and "NOT DETECTED" not in o


LONELY_WORKER = textwrap.dedent("""
    import os, sys, time
    sys.path.insert(0, %r)
    from eddl_b200 import dist as ebd
    t0 = time.time()
    try:
        ebd.rendezvous("gloo", timeout_s=4)
        print("JOINED?")
    except ebd.RankFailure as e:
        print("gave up after %%.1f s" %% (time.time() - t0))
""")


def test_a_rank_that_never_joins_ends_the_rendezvous_with_an_error(tmp_path):
    """World size 2 but only rank 0 is started: the rendezvous gives up after its deadline with RankFailure instead of
    waiting for ever (failure made on the host; no GPU involved)."""
    script = tmp_path / "lonely.py"
    script.write_text(LONELY_WORKER % ROOT)
    (p,) = _spawn(script, 2, (0,), _free_port())
    o, e = p.communicate(timeout=120)
    assert p.returncode == 0, e[-2000:]
    assert "gave up after" in o and "JOINED?" not in o
