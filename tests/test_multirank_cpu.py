"""The N > 1 path on CPU: two gloo ranks shard independent streams with no data-path collective and agree on
the max-over-ranks timing / sum-over-ranks token reduction the benchmark uses."""
import os
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import pyoracle as oracle

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    # each rank owns its own streams: stream s of the job lives on rank s %% world (replicas, no exchange)
    total_streams = 6
    mine = [s for s in range(total_streams) if s %% world == rank]
    committed = 0
    for s in mine:
        cfg = oracle.shaping(temperature=0.7, top_k=64, top_p=0.95, seed=100 + s)
        rc = oracle.run_config(cfg, 16, 3)
        err, toks, emitted, res, _ = oracle.run_scripted(97, s %% 3, 1, 1, [1, 2, 3, 4, 5], rc, 256)
        assert err == 0
        committed += res.new_tokens
    t = torch.tensor([float(rank + 1), float(committed)], dtype=torch.float64)
    mx, sm = t.clone(), t.clone()
    dist.all_reduce(mx, op=dist.ReduceOp.MAX)
    dist.all_reduce(sm, op=dist.ReduceOp.SUM)
    assert mx[0].item() == world and sm[1].item() == 16 * total_streams
    dist.barrier()
    if rank == 0:
        print("OK", int(sm[1].item()))
    dist.destroy_process_group()
""") % ROOT


def test_two_gloo_ranks_shard_streams_without_a_collective_on_the_data_path(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "OK 96" in out.stdout
