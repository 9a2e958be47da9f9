"""The N > 1 paths on CPU with two gloo ranks: (1) independent streams sharded with no data-path collective, agreeing
on the max-over-ranks timing / sum-over-ranks token reduction the benchmark uses; (2) the partition and recombination
of the sharded routed model - head shards, o_proj column shards, expert shards - through the oracle's operators, with
the two sums that cross the ranks taken by a real all-reduce."""
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


SHARD_WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np
    import torch
    import torch.distributed as dist
    from oracle import pyoracle as oracle
    from turbospark_b200.sharding import HeadShard, expert_range, slice_block_columns, slice_experts

    dist.init_process_group("gloo")
    rank, world = dist.get_rank(), dist.get_world_size()
    rng = np.random.default_rng(5)           # the same numbers on both ranks: they stand for replicated inputs
    nq, nkv, hd, d, rows, ctx_len = 4, 2, 128, 256, 3, 40
    E, k, F = 4, 2, 256
    hs = HeadShard(nq, nkv, hd, rank, world)
    assert (hs.q_local, hs.kv_local) == (2, 1)

    # ---- attention heads are independent: a rank's heads give the matching slice of the full result, bit for bit
    q = rng.standard_normal((nq * hd)).astype(np.float32)
    kk = rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32)
    vv = rng.standard_normal((ctx_len, nkv * hd)).astype(np.float32)
    full = oracle.causal_attention(q, kk, vv, hd, nq, nkv, ctx_len, 1.0 / np.sqrt(hd))
    part = oracle.causal_attention(q[hs.q_rows()], kk[:, hs.kv_rows()], vv[:, hs.kv_rows()], hd, hs.q_local, hs.kv_local, ctx_len,
                                   1.0 / np.sqrt(hd))
    assert np.array_equal(part, full[hs.o_cols()])

    # ---- o_proj: every rank multiplies its heads' columns; the f32 shares summed over the ranks give the projection
    wo = oracle.quantize(oracle.Q4K, (rng.standard_normal((d, nq * hd)) * 0.02).astype(np.float32))
    a16 = oracle.f32_to_f16_bits(rng.standard_normal((rows, nq * hd)).astype(np.float32))
    a = oracle.f16_bits_to_f32(a16)
    want = oracle.gemm_quant(oracle.Q4K, wo, d, nq * hd, a)
    mine = oracle.gemm_quant(oracle.Q4K, slice_block_columns(wo, oracle.Q4K, nq * hd, hs.o_cols()), d, hs.q_local * hd, a[:, hs.o_cols()])
    t = torch.from_numpy(mine.copy())
    dist.all_reduce(t)
    got = t.numpy()
    assert np.all(np.abs(got - want) <= 1e-3 + 2e-3 * np.abs(want))
    # every rank rounds the same sum: the f16 rows that go on are identical everywhere
    both = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(both, t)
    assert all(torch.equal(both[0], b) for b in both)

    # ---- experts: a rank computes the (row, slot) outputs of its own experts and zeros elsewhere; the sum over the
    # ranks adds only zeros, so it equals the unsharded per-slot outputs exactly, and so does the slot-ordered combine
    gu = np.concatenate([oracle.quantize(oracle.MXFP4, (rng.standard_normal((2 * F, d)) * 0.05).astype(np.float32)) for _ in range(E)])
    dn = np.concatenate([oracle.quantize(oracle.MXFP4, (rng.standard_normal((d, F)) * 0.05).astype(np.float32)) for _ in range(E)])
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((rows, d)).astype(np.float32))
    ids = np.array([[0, 3], [2, 1], [3, 2]], dtype=np.int32)
    w16 = oracle.f32_to_f16_bits(np.array([[0.6, 0.4], [0.7, 0.3], [0.55, 0.45]], dtype=np.float32))
    zero16 = np.zeros((rows, d), dtype=np.uint16)
    e_lo, e_n = expert_range(E, rank, world)
    gu_r, dn_r = slice_experts(gu, E, e_lo, e_n), slice_experts(dn, E, e_lo, e_n)
    one16 = oracle.f32_to_f16_bits(np.ones((1, 1), dtype=np.float32))

    def slot_values(gate_up, down, n_exp, lo):
        # f32 output of every (row, slot) whose expert lies in [lo, lo + n_exp), zeros elsewhere: gate|up sums, the f16
        # activation, the down sums - the operators the routed layer is made of
        out = np.zeros((rows, k, d), dtype=np.float32)
        for r in range(rows):
            for s in range(k):
                e = int(ids[r, s]) - lo
                if not 0 <= e < n_exp:
                    continue
                per_gu, per_dn = gate_up.shape[0] // n_exp, down.shape[0] // n_exp
                g_u = oracle.gemm_quant(oracle.MXFP4, gate_up[e * per_gu:(e + 1) * per_gu], 2 * F, d, oracle.f16_bits_to_f32(x16[r:r + 1]))[0]
                act = oracle.silu_mul(g_u[:F], g_u[F:])
                act = oracle.f16_bits_to_f32(oracle.f32_to_f16_bits(act))
                out[r, s] = oracle.gemm_quant(oracle.MXFP4, down[e * per_dn:(e + 1) * per_dn], d, F, act.reshape(1, -1))[0]
        return out

    full_vals = slot_values(gu, dn, E, 0)
    local_vals = torch.from_numpy(slot_values(gu_r, dn_r, e_n, e_lo))
    dist.all_reduce(local_vals)
    assert np.array_equal(local_vals.numpy(), full_vals)      # exact: only zeros were added
    # the slot-ordered weighted sum over those values is the routed layer's output (moe_gguf.metal:625-678)
    w = oracle.f16_bits_to_f32(w16)
    acc = np.zeros((rows, d), dtype=np.float32)
    for s in range(k):
        acc = acc + w[:, s:s + 1] * local_vals.numpy()[:, s]
    want_y = oracle.moe_ffn(oracle.MXFP4, gu, dn, E, d, F, x16, zero16, ids, w16)
    assert np.array_equal(oracle.f32_to_f16_bits(acc), want_y)
    dist.barrier()
    if rank == 0:
        print("SHARD OK")
    dist.destroy_process_group()
""") % ROOT


def test_two_gloo_ranks_partition_and_recombine_the_sharded_routed_layer(tmp_path):
    script = tmp_path / "shard_worker.py"
    script.write_text(SHARD_WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                         capture_output=True, text=True, env=env, timeout=300)
    assert out.returncode == 0, out.stdout + out.stderr
    assert "SHARD OK" in out.stdout
