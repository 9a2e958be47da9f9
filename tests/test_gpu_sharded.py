"""The routed model spread over two GPUs (attention tensor-parallel over heads, experts sharded, NCCL all-reduces on
the session's stream) against the same model on one GPU: the logits agree within the model-level tolerance, both
ranks hold bit-identical logits, and the per-slot expert outputs cross the ranks exactly.  Needs two GPUs."""
import os
import subprocess
import sys
import textwrap

import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = textwrap.dedent("""
    import os, sys
    sys.path.insert(0, %r)
    import numpy as np
    import torch
    import torch.distributed as dist
    import turbospark_b200 as tsb
    from turbospark_b200.comm import Comm
    from turbospark_b200.model import W_Q, W_K, W_V, W_O, W_EMBED, W_LM_HEAD
    from turbospark_b200.sharding import HeadShard, expert_range, slice_block_columns, slice_experts
    from oracle import pyoracle as oracle
    from tests import weights

    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    ctx = tsb.Ctx(local)
    comm = Comm.from_torch_distributed(ctx)

    E, K, F = 4, 2, 256
    full_cfg = tsb.ModelConfig(2, 256, 4, 2, 128, 256, 512, 128, 1e-6, 1e4)
    mats, norms = weights.random_weights(full_cfg, 11, oracle)        # the same seeded bytes on both ranks
    moe = weights.random_moe_weights(full_cfg, E, F, 12, oracle)
    prompt = np.random.default_rng(3).integers(0, full_cfg.vocab, size=9).astype(np.int32)

    # ---- the whole model on this rank's GPU (the single-GPU reference)
    whole = tsb.Model(ctx, full_cfg)
    whole.set_moe(E, K, F)
    weights.load_weights(whole, mats, norms, skip=weights.DENSE_FFN)
    weights.load_moe_weights(whole, moe)
    s1 = tsb.Session(ctx, whole, None, 1, 8)
    for i, t in enumerate(prompt[:3]):
        s1.produce_prefill(int(t), i)
    want = s1.verify(prompt[3:], 3)

    # ---- this rank's shard: its heads, its o_proj columns, its experts; router, norms, embedding, head replicated
    hs = HeadShard(full_cfg.n_q_heads, full_cfg.n_kv_heads, full_cfg.head_dim, rank, world)
    cfg = tsb.ModelConfig(2, 256, hs.q_local, hs.kv_local, 128, 256, 512, 128, 1e-6, 1e4)
    e_lo, e_n = expert_range(E, rank, world)
    part = tsb.Model(ctx, cfg)
    part.set_moe(E, K, F)
    part.set_expert_shard(e_lo, e_n)
    qd = full_cfg.n_q_heads * full_cfg.head_dim
    for l in range(2):
        q, _, cols, qt = mats[(l, W_Q)]
        part.set_matrix(l, W_Q, qt, q[hs.q_rows()], hs.q_local * 128, cols)
        for which in (W_K, W_V):
            b, _, cols, qt = mats[(l, which)]
            part.set_matrix(l, which, qt, b[hs.kv_rows()], hs.kv_local * 128, cols)
        o, rows_o, _, qt = mats[(l, W_O)]
        part.set_matrix(l, W_O, qt, slice_block_columns(o, qt, qd, hs.o_cols()), rows_o, hs.q_local * 128)
        rq, sc, bi, gu, dn = moe[l]
        part.set_router(l, rq, sc, bi)
        part.set_experts(l, tsb.MXFP4, slice_experts(gu, E, e_lo, e_n), slice_experts(dn, E, e_lo, e_n))
    for which in (W_EMBED, W_LM_HEAD):
        b, r, c, qt = mats[(-1, which)]
        part.set_matrix(0, which, qt, b, r, c)
    for (l, which), bits in norms.items():
        part.set_norm(max(l, 0), which, bits)
    s2 = tsb.Session(ctx, part, None, 1, 8)
    s2.set_comm(comm)
    for i, t in enumerate(prompt[:3]):
        s2.produce_prefill(int(t), i)
    got = s2.verify(prompt[3:], 3)

    g, w = oracle.f16_bits_to_f32(got), oracle.f16_bits_to_f32(want)
    assert not np.isnan(g).any()
    err = np.abs(g - w)
    # only the o_proj sum changes its order (per-rank partial sums, then the sum over ranks); the routed layer's own
    # chained-f16 bound applies to what follows
    assert np.all(err <= 1e-2 + 1e-2 * np.abs(w)), float(err.max())
    assert np.sqrt((err ** 2).mean()) <= 2e-3 * np.sqrt((w ** 2).mean()), float(np.sqrt((err ** 2).mean()))
    # both ranks hold the same bits
    t = torch.from_numpy(got.astype(np.int32)).cuda()
    both = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(both, t)
    assert all(torch.equal(both[0], b) for b in both)
    # the exchange as an operator: each rank owns one half of a buffer and holds zeros in the other
    n = 4096
    x = np.zeros(n, dtype=np.float32)
    x[rank * n // world:(rank + 1) * n // world] = np.random.default_rng(20 + rank).standard_normal(n // world).astype(np.float32)
    buf = ctx.to_device(x)
    comm.all_reduce_f32(buf, n)
    ctx.sync()
    summed = buf.download(np.float32, n)
    assert np.array_equal(summed[rank * n // world:(rank + 1) * n // world], x[rank * n // world:(rank + 1) * n // world])
    dist.barrier()
    if rank == 0:
        print("SHARDED GPU OK", float(err.max()))
    s1.close(), s2.close(), whole.close(), part.close(), comm.close(), ctx.close()
    dist.destroy_process_group()
""") % ROOT


def test_two_gpus_run_the_sharded_routed_model_like_one(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    script = tmp_path / "sharded_worker.py"
    script.write_text(WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29547", str(script)],
                         capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert "SHARDED GPU OK" in out.stdout


def test_two_contexts_on_two_devices_in_one_process(oracle):
    """A kernel's opt-in to large shared memory belongs to the device: the second device of a process must get its own."""
    import numpy as np
    import torch
    import turbospark_b200 as tsb
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    rows, cols = 64, 4096
    rng = np.random.default_rng(1)
    q = oracle.quantize(0, (rng.standard_normal((rows, cols)) * 0.02).astype(np.float32))
    x16 = oracle.f32_to_f16_bits(rng.standard_normal((3, cols)).astype(np.float32))
    want = oracle.gemm_quant(0, q, rows, cols, oracle.f16_bits_to_f32(x16))
    for dev in (0, 1):
        c = tsb.Ctx(dev)
        yd = c.alloc(3 * rows * 4)
        c.gemm_quant(0, c.upload_weights(q), rows, cols, c.to_device(x16), yd, 3, y_f32=True)
        c.sync()
        got = yd.download(np.float32, 3 * rows).reshape(3, rows)
        assert np.all(np.abs(got - want) <= 1e-3 + 2e-3 * np.abs(want))
        c.close()
