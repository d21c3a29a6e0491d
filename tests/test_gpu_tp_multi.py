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
    try:
        _run_rank(rank, world, port, q)
    except Exception as e:      # report instead of leaving the parent waiting for its time-out
        import traceback
        q.put(("error", rank, repr(e), traceback.format_exc()))


def _run_rank(rank, world, port, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import torch
    import torch.distributed as dist
    import fomoe_b200 as fb
    dist.init_process_group("cpu:gloo,cuda:nccl", rank=rank, world_size=world)
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
    # the same stack through the per-phase kernels with the CALLER's collective between them: NCCL on the
    # library's own stream (the arrangement of the reference's tp_allreduce_sum, include/tp.h:53-79)
    stream = torch.cuda.ExternalStream(d.stream_handle(), device=rank)

    class _Dev:
        def __init__(self, ptr, n):
            self.__cuda_array_interface__ = dict(shape=(n,), typestr="<f4", data=(ptr, False), version=2)

    def hook(ptr, n, _stream):
        t = torch.as_tensor(_Dev(ptr, n), device=f"cuda:{rank}")
        with torch.cuda.stream(stream):
            dist.all_reduce(t)
        return 0

    d.set_variant(0)
    d.set_allreduce(hook)
    d.tokens_run(0, 4)
    out_nccl = d.tokens_download(0, 4)
    d.set_allreduce(None)
    d.set_variant(2)
    st = d.status()
    dist.barrier()
    q.put((rank, out, one, ids, st, out_nccl))
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
    res = [q.get(timeout=240) for _ in range(world)]
    errors = [r for r in res if r[0] == "error"]
    if errors:
        for p in procs:
            p.join(timeout=30)
            if p.is_alive():
                p.terminate()
        pytest.fail("rank %d: %s\n%s" % errors[0][1:])
    res.sort(key=lambda t: t[0])
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
    for rank, out, one, ids, st, out_nccl in res:
        assert st == 0
        assert H.rel_l2(out_nccl, out) < 1e-5                   # NCCL between per-phase kernels == fused exchange
        assert (H.bits(out) == H.bits(res[0][1])).all()        # every rank holds the same bits
        assert (H.bits(one) == H.bits(out[1])).all()           # host-to-host call == resident run
        assert H.rel_l2(out, want) < 1e-4                       # == single GPU up to reassociation
    single.close()
