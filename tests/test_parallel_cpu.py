"""Head sharding and the optional all-gather, on CPU with the gloo backend (world_size 2 and 3)."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from sageattention.parallel import (gather_blocks, local_block, local_heads, shard_grid, shard_range, slice_block,
                                    slice_heads, sageattn_sharded)


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
    # deterministic stand-in with the real call's shapes: first row of V broadcast over queries + q (no
    # reduction, so the value does not depend on how the heads are grouped)
    seq = 2 if tensor_layout == "HND" else 1
    hd = 1 if tensor_layout == "HND" else 2
    rep = q.size(hd) // k.size(hd)
    vm = v.narrow(seq, 0, 1).repeat_interleave(rep, dim=hd)
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


@pytest.mark.parametrize("world,layout,hq,hkv", [(2, "HND", 8, 4), (2, "NHD", 6, 3), (3, "HND", 8, 8), (3, "HND", 4, 2),
                                                 (2, "NHD", 16, 8)])
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


def test_shard_grid_balances_batch_and_heads():
    assert shard_grid(1, 64, 8) == (1, 8)             # long-context config: heads only
    wb, wh = shard_grid(16, 10, 8)                    # 16 x 10 heads: 20 units per rank instead of the 32 of head-only sharding
    assert wb * wh == 8 and -(-16 // wb) * -(-10 // wh) == 20
    assert shard_grid(4, 8, 8) == (1, 8)              # GQA prefill: one kv-head per rank
    assert shard_grid(1, 24, 8) == (1, 8)             # 24 heads on 8 ranks: 3 each
    for batch, hkv, world in ((16, 10, 8), (3, 5, 4), (2, 2, 8), (1, 1, 2), (5, 7, 6)):
        rep = 2
        seen = set()
        for r in range(world):
            (b_lo, b_hi), (q_lo, q_hi), (k_lo, k_hi) = local_block(batch, hkv * rep, hkv, world, r)
            assert (q_lo, q_hi) == (k_lo * rep, k_hi * rep)
            for b in range(b_lo, b_hi):
                for h in range(k_lo, k_hi):
                    assert (b, h) not in seen
                    seen.add((b, h))
        assert len(seen) == batch * hkv


def _grid_worker(rank, world, port, layout, batch, hq, hkv, q):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(2)
        shape = lambda h: (batch, h, 12, 8) if layout == "HND" else (batch, 12, h, 8)
        qf, kf, vf = (torch.randn(shape(h), generator=g) for h in (hq, hkv, hkv))
        b_r, q_r, k_r = local_block(batch, hq, hkv, world, rank)
        ql, kl, vl = slice_block(qf, layout, b_r, q_r), slice_block(kf, layout, b_r, k_r), slice_block(vf, layout, b_r, k_r)
        loc = _fake_attn(ql, kl, vl, layout) if ql.numel() else ql
        full = gather_blocks(loc, batch, hq, hkv, layout)
        exp = _fake_attn(qf, kf, vf, layout)
        q.put((rank, bool(torch.allclose(full, exp)) and full.shape == qf.shape))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,layout,batch,hq,hkv", [(2, "HND", 4, 6, 3), (3, "NHD", 3, 4, 2), (2, "NHD", 1, 4, 4)])
def test_grid_sharding_gathers_full_output(world, layout, batch, hq, hkv):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_grid_worker, args=(r, world, port, layout, batch, hq, hkv, q)) for r in range(world)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    results = dict(q.get(timeout=10) for _ in range(world))
    assert all(results.get(r) for r in range(world)), results

