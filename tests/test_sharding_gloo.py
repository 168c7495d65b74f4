"""The multi-GPU path shards samples across ranks with no data-path collective.  Here two CPU
ranks (gloo) each take their shard_range of a small batch, evaluate it with the oracle, and the
gathered result must equal the unsharded evaluation; the max-over-ranks timing reduction that
bench.py uses is exercised too."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/oracle")
    import __graft_entry__ as ge
    zb = ge.load_package(); zo = ge.load_oracle()
    import graph_oracle
    from zant_b200 import models
    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    total = 7
    scales = dict(relu1=0.02, relu2=0.05, relu3=0.05, logits=0.1)
    x = models.small_cnn_input(total, 42)
    b, c = zb.shard_range(total, world, rank)
    g = models.small_cnn_int8(c, act_scales=scales)
    mine = graph_oracle.run(zo, g, x[b:b + c])[g.output]
    parts = [None] * world
    dist.all_gather_object(parts, (b, mine))
    t = torch.tensor([float(rank + 1)], dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    if rank == 0:
        full = models.small_cnn_int8(total, act_scales=scales)
        want = graph_oracle.run(zo, full, x)[full.output]
        got = np.concatenate([p for _, p in sorted(parts, key=lambda bp: bp[0])])
        assert np.array_equal(got, want)
        assert t.item() == world
        print("SHARD_OK")
    dist.destroy_process_group()
""")


def test_two_rank_sample_sharding(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER.format(root=ROOT))
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(port), str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "SHARD_OK" in res.stdout


FAILING_WORKER = textwrap.dedent("""
    import os, sys
    import numpy as np
    import torch, torch.distributed as dist
    sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + "/oracle")
    import __graft_entry__ as ge
    zb = ge.load_package(); zo = ge.load_oracle()
    import graph_oracle
    from zant_b200 import models, health
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    store = dist.TCPStore("127.0.0.1", {store_port}, world, rank == 0)
    dist.init_process_group("gloo", store=dist.PrefixStore("pg", store), rank=rank, world_size=world)
    hp = health.RankHealth(store, rank, world, timeout_s=5.0)
    scales = dict(relu1=0.02, relu2=0.05, relu3=0.05, logits=0.1)
    x = models.small_cnn_input(6, 7)
    b, c = zb.shard_range(6, world, rank)
    g = models.small_cnn_int8(c, act_scales=scales)
    done = []
    for step in range(3):
        status = 0
        try:
            if rank == 1 and step == 1:
                raise zb.ZantError(-106, "DeviceTimeout", "injected on the host")      # the failure is made here, no GPU involved
            done.append(graph_oracle.run(zo, g, x[b:b + c])[g.output])
        except zb.ZantError as e:
            status = e.status
        hp.report(step, status)                      # between steps: nothing of this rank is in flight
        ok, per_rank = hp.all_ok(step)
        if not ok:
            # the failed rank leaves; the healthy one names it and keeps its own results, and neither enters the barrier
            print(f"RANK {{rank}} STEP {{step}} STATUS {{per_rank}} KEPT {{len(done)}}", flush=True)
            break
        dist.barrier()
    dist.destroy_process_group()
""")


def test_a_failing_rank_is_reported_not_waited_for(tmp_path):
    """One of two ranks fails between steps (an error made on the host): the other learns of it from the store before
    its next collective and reports the per-rank status array instead of hanging in the barrier."""
    script = tmp_path / "failing_worker.py"
    ports = []
    for _ in range(2):
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            ports.append(s.getsockname()[1])
    script.write_text(FAILING_WORKER.format(root=ROOT, store_port=ports[1]))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(ports[0]), str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert res.returncode == 0, res.stdout + res.stderr
    assert "RANK 0 STEP 1 STATUS [0, -106] KEPT 2" in res.stdout
    assert "RANK 1 STEP 1 STATUS [0, -106] KEPT 1" in res.stdout
