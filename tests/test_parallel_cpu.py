"""Head sharding and the optional all-gather, on CPU with the gloo backend (world_size 2 and 3)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sageattention.parallel import local_heads, shard_range, slice_heads, sageattn_sharded


def test_shard_range_partitions_exactly():
    for n in (0, 1, 3, 8, 24, 64, 160):
        for world in (1, 2, 3, 4, 8):
            got = [shard_range(n, world, r) for r in range(world)]
            covered = [i for lo, hi in got for i in range(lo, hi)]
            assert covered == list(range(n))
            assert max(hi - lo for lo, hi in got) == -(-n // world) or n == 0
    with pytest.raises(ValueError):
        shard_range(4, 2, 2)


def test_local_heads_keeps_gqa_groups_together():
    (q_lo, q_hi), (k_lo, k_hi) = local_heads(32, 8, 8, 3)
    assert (k_lo, k_hi) == (3, 4) and (q_lo, q_hi) == (12, 16)
    with pytest.raises(ValueError):
        local_heads(30, 8, 2, 0)


def _fake_attn(q, k, v, tensor_layout="HND", return_lse=False, **_):
    # deterministic stand-in with the real call's shapes: mean of V broadcast over queries + q
    seq = 2 if tensor_layout == "HND" else 1
    hd = 1 if tensor_layout == "HND" else 2
    rep = q.size(hd) // k.size(hd)
    vm = v.mean(dim=seq, keepdim=True).repeat_interleave(rep, dim=hd)
    out = q + vm
    if return_lse:
        lse = out.float().sum(-1)
        return out, (lse if tensor_layout == "HND" else lse.transpose(1, 2))
    return out


def _worker(rank, world, port, layout, hq, hkv, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(1)
        shape = lambda h: (2, h, 16, 8) if layout == "HND" else (2, 16, h, 8)
        qf, kf, vf = (torch.randn(shape(h), generator=g) for h in (hq, hkv, hkv))
        (ql, qh), (kl, kh) = local_heads(hq, hkv, world, rank)
        args = (slice_heads(qf, layout, ql, qh), slice_heads(kf, layout, kl, kh), slice_heads(vf, layout, kl, kh))
        out, lse = sageattn_sharded(*args, num_q_heads=hq, num_kv_heads=hkv, tensor_layout=layout, attn_fn=_fake_attn,
                                    return_lse=True)
        exp, exp_lse = _fake_attn(qf, kf, vf, layout, True)
        ok = torch.allclose(out, exp) and torch.allclose(lse, exp_lse) and out.shape == qf.shape
        loc = sageattn_sharded(*args, num_q_heads=hq, tensor_layout=layout, attn_fn=_fake_attn, gather=False)
        ok = ok and loc.shape == args[0].shape
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("world,layout,hq,hkv", [(2, "HND", 8, 4), (2, "NHD", 6, 3), (3, "HND", 8, 8)])
def test_sharded_attention_gathers_full_output(world, layout, hq, hkv):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, layout, hq, hkv, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    res = sorted(q.get(timeout=5) for _ in range(world))
    assert res == [(r, True) for r in range(world)]
