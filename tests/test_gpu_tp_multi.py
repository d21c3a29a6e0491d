"""Tensor parallelism across real GPUs (needs at least two): one process per GPU, the ranks exchange the handles of
their receive buffers, then every rank runs the whole stack and must end with the same bits as every other rank and
with the single-GPU result up to fp32 reassociation of the per-rank partial sums.  The all-reduce is fused into the
stack kernel as peer stores (the reference's counterpart: tp_allreduce_sum, src/tp.hip:85-124, tested by
tests/test_tp.hip:221-289 on the pattern a[i] = i, b[i] = 1000 + i)."""
import os
import sys

import numpy as np
import pytest

import helpers as H

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHAPE = dict(n_layers=3, n_embd=1024, n_inter=1024, n_experts=32, top_k=4)
SEED = 19


def _worker(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import fomoe_b200 as fb
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.cuda.set_device(rank)
    dts = [H.Q6, H.Q4, H.Q6]
    d = fb.MoeDecoder(SHAPE["n_layers"], SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True, dts,
                      device=rank, tp_rank=rank, tp_size=world, rms_eps=1e-6, max_tokens=4)
    d.generate(SEED)
    handles = [None] * world
    dist.all_gather_object(handles, d.tp_export())
    d.tp_connect(handles)
    toks = np.stack([H.hidden(fb, SEED, t, SHAPE["n_embd"]) for t in range(4)])
    d.tokens_upload(0, toks)
    dist.barrier()
    d.tokens_run(0, 4)
    out = d.tokens_download(0, 4)
    one = d.stack_run(toks[1])
    ids = [d.get_routing(l)[0] for l in range(SHAPE["n_layers"])]
    st = d.status()
    dist.barrier()
    q.put((rank, out, one, ids, st))
    dist.barrier()
    d.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_tensor_parallel_stack_across_gpus(fb, world):
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=600) for _ in range(world)], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    dts = [H.Q6, H.Q4, H.Q6]
    single = fb.MoeDecoder(SHAPE["n_layers"], SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True,
                           dts, rms_eps=1e-6, max_tokens=4)
    single.generate(SEED)
    toks = np.stack([H.hidden(fb, SEED, t, SHAPE["n_embd"]) for t in range(4)])
    single.tokens_upload(0, toks)
    single.tokens_run(0, 4)
    want = single.tokens_download(0, 4)
    for rank, out, one, ids, st in res:
        assert st == 0
        assert (H.bits(out) == H.bits(res[0][1])).all()        # every rank holds the same bits
        assert (H.bits(one) == H.bits(out[1])).all()           # host-to-host call == resident run
        assert H.rel_l2(out, want) < 1e-4                       # == single GPU up to reassociation
    single.close()
