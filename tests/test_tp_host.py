"""Tensor-parallel sharding arithmetic on the CPU, two gloo ranks: gate/up rows and down column blocks
are split over the ranks (the split the device table uses), each rank forms its partial MoE output with
the oracle's integer dots, and an all-reduce(sum) must reproduce the unsharded oracle result."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import helpers as H

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _partial(orc, fb, rank, world, h, experts, scores, down_type, n_embd, inter):
    """sum_e score_e * down_e[:, cols_r] . Q8K(act_e)[cols_r], using only rank's gate/up rows."""
    from oracle.oracle import Q8K_BLOCK, row_bytes
    il = inter // world
    gs = fb.matrix_bytes(H.Q4, inter, n_embd)
    q8h = orc.quantize_q8k(h)
    rb_g = row_bytes(H.Q4, n_embd)
    blk = {H.Q4: 144, H.Q6: 210}[down_type]
    bpr = inter // 256
    bl = il // 256
    out = np.zeros(n_embd, dtype=np.float32)
    for e, s in zip(experts, scores):
        act = np.zeros(il, dtype=np.float32)
        for i in range(il):
            r = rank * il + i
            g = orc.vec_dot(e[r * rb_g:(r + 1) * rb_g], H.Q4, q8h, n_embd // 256)
            u = orc.vec_dot(e[gs + r * rb_g:gs + (r + 1) * rb_g], H.Q4, q8h, n_embd // 256)
            act[i] = np.float32(g / np.float32(1.0 + np.exp(-np.float64(g)))) * u
        q8a = orc.quantize_q8k(act)  # windows of 256 are rank-local for world <= inter/256
        down = e[2 * gs:]
        for row in range(n_embd):
            off = (row * bpr + rank * bl) * blk
            out[row] += np.float32(s) * orc.vec_dot(down[off:off + bl * blk], down_type, q8a, bl)
    return out


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import fomoe_b200 as fb
    from oracle.oracle import Oracle
    orc = Oracle()
    n_embd, inter, seed = 256, 512, 13
    h = H.hidden(fb, seed, 0, n_embd)
    for down_type in (H.Q6, H.Q4):
        ex = [H.expert_record(fb, seed, 0, e, down_type, n_embd, inter) for e in range(3)]
        sc = np.array([0.5, 0.3, 0.2], dtype=np.float32)
        part = torch.from_numpy(_partial(orc, fb, rank, world, h, ex, sc, down_type, n_embd, inter))
        dist.all_reduce(part, op=dist.ReduceOp.SUM)
        gs = fb.matrix_bytes(H.Q4, inter, n_embd)
        want = orc.moe_block(h, ex, sc, None, H.Q4, H.Q4, down_type, gs, gs, n_embd, inter)
        q.put((rank, down_type, H.rel_l2(part.numpy(), want)))
    dist.barrier()
    dist.destroy_process_group()


def test_two_rank_partials_allreduce_to_full(fb):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = [q.get(timeout=300) for _ in range(4)]
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for rank, dt, err in res:
        assert err < 1e-5, (rank, dt, err)
