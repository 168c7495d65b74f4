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
