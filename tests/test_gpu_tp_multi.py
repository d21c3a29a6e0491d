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


def _worker(rank, world, port, q, n_inter=1024):
    try:
        SHAPE["n_inter"] = n_inter
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
    # the batched (tensor-core) path, sharded the same way, with NCCL summing the ranks' [tokens x hidden] partial
    # outputs on the library's stream after every layer
    bat_out = None
    if SHAPE["n_inter"] % (256 * world) == 0:
        bat = fb.BatchedMoe(2, SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True, max_tokens=24,
                            device=rank, tp_rank=rank, tp_size=world)
        bat.generate(SEED, with_logits=True)

        def bhook(ptr, n, s):
            t = torch.as_tensor(_Dev(ptr, n), device=f"cuda:{rank}")
            with torch.cuda.stream(torch.cuda.ExternalStream(s, device=rank)):
                dist.all_reduce(t)
            return 0

        bat.set_allreduce(bhook)
        bat.tokens_upload(np.stack([H.hidden(fb, SEED, t, SHAPE["n_embd"]) for t in range(24)]))
        bat.stack_run(24)
        bat_out = bat.tokens_download(24)
        st = st or bat.status()
        bat.close()
    dist.barrier()
    q.put((rank, out, one, ids, st, out_nccl, bat_out))
    dist.barrier()
    d.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_inter", [(2, 1024), (4, 1024), (4, 512), (8, 1024)])
def test_tensor_parallel_stack_across_gpus(fb, world, n_inter):
    """(4, 512) and (8, 1024) have twice as many ranks as 256-wide windows: two ranks share a window, each owns one
    half of the down super-blocks (see the C header)."""
    import torch
    import torch.multiprocessing as mp
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    SHAPE["n_inter"] = n_inter
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 1000 + world + (16 if n_inter != 1024 else 0)
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, n_inter)) for r in range(world)]
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
    bat_want = None
    if n_inter % (256 * world) == 0:
        bs = fb.BatchedMoe(2, SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True, max_tokens=24)
        bs.generate(SEED, with_logits=True)
        bs.tokens_upload(np.stack([H.hidden(fb, SEED, t, SHAPE["n_embd"]) for t in range(24)]))
        bs.stack_run(24)
        bat_want = bs.tokens_download(24)
        bs.close()
    for rank, out, one, ids, st, out_nccl, bat_out in res:
        assert st == 0
        if bat_want is not None:
            assert (H.bits(bat_out) == H.bits(res[0][6])).all()   # NCCL leaves the same bits on every rank
            assert max(H.rel_l2(bat_out[t], bat_want[t]) for t in range(24)) < 1e-3
        assert H.rel_l2(out_nccl, out) < 1e-5                   # NCCL between per-phase kernels == fused exchange
        assert (H.bits(out) == H.bits(res[0][1])).all()        # every rank holds the same bits
        assert (H.bits(one) == H.bits(out[1])).all()           # host-to-host call == resident run
        assert H.rel_l2(out, want) < 1e-4                       # == single GPU up to reassociation
    single.close()


def test_two_ranks_in_one_process(fb):
    """Both ranks live in ONE process (one context per GPU, as the reference drives its two GPUs, src/tp.hip): plain
    device pointers instead of IPC handles, peer access enabled by the library, one host thread per rank.  Also covers
    kernel attributes that are per device (dynamic shared memory of the stack kernel on a second device)."""
    import threading
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    dts = [H.Q6, H.Q4, H.Q6]
    SHAPE["n_inter"] = 1024
    ds = [fb.MoeDecoder(SHAPE["n_layers"], SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True, dts,
                        device=r, tp_rank=r, tp_size=2, rms_eps=1e-6, max_tokens=4) for r in range(2)]
    for r, d in enumerate(ds):
        d.generate(SEED)
        d.tp_enable_peer(1 - r)
    ptrs = [d.tp_recv_ptr() for d in ds]
    for d in ds:
        d.tp_connect_ptrs(ptrs)
        d.set_wait_limit(1 << 21)
    toks = np.stack([H.hidden(fb, SEED, t, SHAPE["n_embd"]) for t in range(4)])
    outs, errs = [None, None], []

    def run(r):
        try:
            ds[r].tokens_upload(0, toks)
            ds[r].tokens_run(0, 4)
            outs[r] = ds[r].tokens_download(0, 4)
        except Exception as e:      # a failed rank makes the other give up after its bounded wait
            errs.append((r, repr(e)))

    ths = [threading.Thread(target=run, args=(r,)) for r in range(2)]
    for t in ths:
        t.start()
    for t in ths:
        t.join(timeout=120)
    assert not errs, errs
    assert all(d.status() == 0 for d in ds)
    assert (H.bits(outs[0]) == H.bits(outs[1])).all()
    single = fb.MoeDecoder(SHAPE["n_layers"], SHAPE["n_embd"], SHAPE["n_inter"], SHAPE["n_experts"], SHAPE["top_k"], True,
                           dts, rms_eps=1e-6, max_tokens=4)
    single.generate(SEED)
    single.tokens_upload(0, toks)
    single.tokens_run(0, 4)
    assert H.rel_l2(outs[0], single.tokens_download(0, 4)) < 1e-4
    single.close()
    for d in ds:
        d.close()
