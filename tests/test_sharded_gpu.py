"""Head sharding over two GPUs against the single-GPU result, with both exchanges of the output: rows stored
into the other rank's buffer by the attention epilogue ("peer") and the grouped NCCL all-gather ("nccl").

Needs two GPUs: on a one-GPU machine the test is skipped.  Each rank is a child process with its own
GPU; rank 0 also computes the whole problem alone and compares.
"""
import os
import socket
import sys

import pytest
import torch

from gpu_util import cuda_or_fail

pytestmark = pytest.mark.gpu


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank(rank, world, port, layout, hq, hkv, groups, via, queue):
    import torch.distributed as dist
    for p in (os.path.dirname(os.path.dirname(os.path.abspath(__file__))),):
        sys.path.insert(0, os.path.join(p, "sageattention-autotune_b200"))
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        import sageattention
        from sageattention.parallel import local_heads, release_peer_outputs, sageattn_sharded, slice_heads
        g = torch.Generator().manual_seed(3)
        shape = (lambda h: (1, h, 1500, 128)) if layout == "HND" else (lambda h: (1, 1500, h, 128))
        q, k, v = (torch.randn(shape(h), generator=g).half().to(dev) for h in (hq, hkv, hkv))
        (ql, qh), (kl, kh) = local_heads(hq, hkv, world, rank)
        kw = dict(tensor_layout=layout, is_causal=True, pv_accum_dtype="fp16+fp32")
        local = (slice_heads(q, layout, ql, qh), slice_heads(k, layout, kl, kh), slice_heads(v, layout, kl, kh))
        out, lse = sageattn_sharded(*local, num_q_heads=hq, num_kv_heads=hkv, gather_groups=groups, gather_via=via,
                                    return_lse=True, **kw)
        # a second call on other data (no LSE this time: the ranks then meet through the small all-reduce);
        # the first call's tensor must survive it
        q2 = -q
        out2 = sageattn_sharded(slice_heads(q2, layout, ql, qh), local[1], local[2], num_q_heads=hq, num_kv_heads=hkv,
                                gather_groups=groups, gather_via=via, **kw)
        torch.cuda.synchronize()
        exp, exp_lse = sageattention.sageattn(q, k, v, return_lse=True, **kw)
        exp2 = sageattention.sageattn(q2, k, v, **kw)
        # (the LSE carries the q.km^T correction, a cuBLAS product whose summation order may follow the batch
        # of heads it is called with: equal to rounding, not to the bit)
        same_out = out.shape == q.shape and torch.equal(out, exp) and torch.equal(out2, exp2)
        lse_err = float((lse - exp_lse).abs().max())
        queue.put((rank, bool(same_out and lse_err <= 1e-4), f"output equal: {same_out}, LSE max diff: {lse_err:.3g}"))
        release_peer_outputs()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("via", ["peer", "nccl"])
@pytest.mark.parametrize("layout,hq,hkv,groups", [("HND", 8, 8, None), ("HND", 8, 4, 1), ("NHD", 6, 3, 2)])
def test_sharded_call_ends_with_the_single_gpu_result_on_every_rank(layout, hq, hkv, groups, via):
    cuda_or_fail()
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    queue = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_rank, args=(r, 2, port, layout, hq, hkv, groups, via, queue)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
        assert p.exitcode == 0
    results = sorted(queue.get(timeout=5) for _ in range(2))
    assert [r[:2] for r in results] == [(0, True), (1, True)], results
