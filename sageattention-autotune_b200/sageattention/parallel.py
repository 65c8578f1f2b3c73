"""Head sharding across the GPUs of one node.

The reference is single-GPU.  Every (batch, kv-head) pair of the forward path is independent - the
K mean, the quantisation and the attention core never look across heads - so the natural
multi-GPU form is one process per GPU, each running the unchanged single-GPU pipeline on a
contiguous range of kv-heads together with the query heads that share them (GQA groups are never
split).  No kernel touches another GPU's memory.  NCCL is used for exactly one thing: an
all-gather of the output (and LSE) when the caller asks for the whole tensor on every rank.

On the GPUs of one node the default exchange is not a collective at all: every rank keeps the whole output
in a buffer that the other ranks have mapped (sage_b200_peer_alloc / sage_b200_peer_open), and the attention
epilogue stores each finished row into every rank's buffer (sage_b200_set_output_peers), so the transfer
over NVLink runs tile by tile under the compute and only a small collective that makes the ranks meet
follows the kernel.
"""
from __future__ import annotations

import ctypes
import os
import warnings
from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def shard_range(n_units: int, world_size: int, rank: int) -> Tuple[int, int]:
    """Contiguous [begin, end) of `n_units` owned by `rank`: ceil(n/world) per rank, last ranks may
    own fewer (or none)."""
    if n_units < 0 or world_size <= 0 or not 0 <= rank < world_size:
        raise ValueError("bad shard request")
    per = -(-n_units // world_size)
    lo = min(n_units, rank * per)
    return lo, min(n_units, lo + per)


def local_heads(num_q_heads: int, num_kv_heads: int, world_size: int, rank: int):
    """(q_head_range, kv_head_range) for this rank; kv-heads are the sharded unit."""
    if num_q_heads % num_kv_heads:
        raise ValueError("num_qo_heads must be divisible by num_kv_heads")
    rep = num_q_heads // num_kv_heads
    lo, hi = shard_range(num_kv_heads, world_size, rank)
    return (lo * rep, hi * rep), (lo, hi)


def slice_heads(t: torch.Tensor, tensor_layout: str, lo: int, hi: int) -> torch.Tensor:
    return t[:, lo:hi] if tensor_layout == "HND" else t[:, :, lo:hi]


_gather_groups = {}


def _gather_group(group):
    """The process group the overlapped all-gather runs on.  The attention kernel fills every SM (one CTA
    per SM, all registers), so a collective issued on an ordinary stream only gets SMs when the kernel it
    is meant to overlap with has almost finished.  NCCL kernels of a group created with a high-priority
    stream are placed as soon as any attention CTA retires.  A caller-supplied group is used as it is."""
    if group is not None or dist.get_backend() != "nccl":
        return group
    key = id(dist.group.WORLD)
    if key not in _gather_groups:
        opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
        _gather_groups[key] = dist.new_group(backend="nccl", pg_options=opts)
    return _gather_groups[key]


class _RawCuda:
    """A device allocation seen through the CUDA array interface, for torch.as_tensor."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}


class PeerOutput:
    """The whole output on every rank, each rank's copy mapped by all the others.

    Two buffers are used in turn: the tensor a call returns stays valid until the call after the next
    one with the same shapes, and a rank that is already storing the next call's rows into its peers'
    memory never touches what they may still be reading."""

    def __init__(self, shape, dtype, device, group):
        from . import _capi as C
        self._C = C
        L = C.lib()
        self.shape, self.dtype, self.device = tuple(shape), dtype, device
        self.nbytes = -(-(torch.empty((), dtype=dtype).element_size() * int(torch.Size(shape).numel())) // 256) * 256
        world, rank = dist.get_world_size(group), dist.get_rank(group)
        self.bases, self.opened, self.tensors, self.offsets = [], [], [], []
        self.ok = True
        self.turn = 0
        for _ in range(2):
            ptr, handle = ctypes.c_void_p(), ctypes.create_string_buffer(64)
            with torch.cuda.device(device):
                rc = L.sage_b200_peer_alloc(self.nbytes, ctypes.byref(ptr), handle)
            mine = bytes(handle.raw) if rc == 0 else None
            handles = [None] * world
            dist.all_gather_object(handles, mine, group=group)
            peers = []
            if all(h is not None for h in handles):
                with torch.cuda.device(device):
                    for r in range(world):
                        if r == rank:
                            continue
                        mapped = ctypes.c_void_p()
                        if L.sage_b200_peer_open(handles[r], ctypes.byref(mapped)) != 0:
                            self.ok = False
                            break
                        peers.append(mapped.value)
                        self.opened.append(mapped.value)
            else:
                self.ok = False
            if rc == 0:
                self.bases.append(ptr.value)
            flags = [None] * world
            dist.all_gather_object(flags, self.ok, group=group)
            self.ok = all(flags)
            if not self.ok:
                self.reason = L.sage_b200_last_error().decode() or "a peer could not allocate or map its buffer"
                self.close()                                          # nothing half-built stays behind
                break
            raw = torch.as_tensor(_RawCuda(ptr.value, self.nbytes), device=device)
            n = int(torch.Size(shape).numel())
            self.tensors.append(raw.view(dtype)[:n].view(self.shape))
            self.offsets.append((ctypes.c_int64 * max(1, len(peers)))(*[b - ptr.value for b in peers]))
        self.n_peer = world - 1

    def next(self):
        """(tensor, offsets) of the buffer this call writes"""
        self.turn ^= 1
        return self.tensors[self.turn], self.offsets[self.turn]

    def close(self):
        """Unmap the peers' buffers and free the own ones (every rank, after a barrier of the caller's)."""
        L = self._C.lib()
        with torch.cuda.device(self.device):
            for p in self.opened:
                L.sage_b200_peer_close(p)
            for p in self.bases:
                L.sage_b200_peer_free(p)
        self.opened, self.bases, self.tensors = [], [], []


_peer_outputs = {}
_last_exchange = {"via": None}


def last_gather_via() -> Optional[str]:
    """How the last gathering sageattn_sharded call of this process exchanged the output: "peer", "nccl"
    (or the caller's backend), or None before the first such call."""
    return _last_exchange["via"]


def _peer_output(shape, dtype, device, group) -> Optional[PeerOutput]:
    key = (tuple(shape), dtype, device, id(group))
    if key not in _peer_outputs:
        ws = PeerOutput(shape, dtype, device, group)
        if not ws.ok:
            warnings.warn(f"peer-mapped output buffers are not available ({ws.reason}); the output is gathered by NCCL",
                          stacklevel=3)
        _peer_outputs[key] = ws
    ws = _peer_outputs[key]
    return ws if ws.ok else None


def release_peer_outputs() -> None:
    """Free every peer-mapped output buffer of this process (collective: all ranks call it together,
    with no attention call in flight)."""
    if dist.is_initialized():
        dist.barrier()
    for ws in _peer_outputs.values():
        ws.close()
    _peer_outputs.clear()


def _sharded_into_peers(q_local, k_local, v_local, num_q_heads, num_kv_heads, tensor_layout, group, attn_fn, kwargs):
    """The head-sharded call with the exchange fused into the attention epilogue; None when the peer
    buffers cannot be had (the caller then gathers by NCCL)."""
    from . import _capi as C
    from .core import output_into, sageattn
    attn_fn = attn_fn or sageattn
    h_dim = 1 if tensor_layout == "HND" else 2
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    full_shape = list(q_local.shape)
    full_shape[h_dim] = num_q_heads
    ws = _peer_output(full_shape, q_local.dtype, q_local.device, group)
    if ws is None:
        return None
    want_lse = bool(kwargs.get("return_lse"))
    (q_lo, q_hi), _ = local_heads(num_q_heads, num_kv_heads, world, rank)
    full, offsets = ws.next()
    L = C.lib()
    lse = None
    if q_hi > q_lo:
        C.check(L.sage_b200_set_output_peers(ws.n_peer, offsets))
        try:
            with output_into(slice_heads(full, tensor_layout, q_lo, q_hi)):
                res = attn_fn(q_local, k_local, v_local, tensor_layout=tensor_layout, **kwargs)
        finally:
            L.sage_b200_set_output_peers(0, None)
        lse = res[1] if want_lse else None
    # the ranks meet: once this collective has completed here, every rank's attention kernel has, and with it
    # its stores into this rank's buffer
    per = -(-num_kv_heads // world) * (num_q_heads // num_kv_heads)
    if want_lse:
        b, n = q_local.size(0), q_local.size(3 - h_dim)
        slot = torch.zeros((per, b, n), dtype=torch.float32, device=q_local.device)
        if lse is not None:
            slot[: lse.size(1)] = lse.movedim(1, 0)
        lse_full = torch.empty((world * per, b, n), dtype=torch.float32, device=q_local.device)
        dist.all_gather_into_tensor(lse_full, slot, group=group)
        return full, lse_full[:num_q_heads].movedim(0, 1)
    meet = torch.zeros(1, dtype=torch.int32, device=q_local.device)
    dist.all_reduce(meet, group=group)
    return full


def sageattn_sharded(q_local, k_local, v_local, num_q_heads: int, tensor_layout: str = "HND",
                     group: Optional[dist.ProcessGroup] = None, gather: bool = True,
                     attn_fn: Optional[Callable] = None, num_kv_heads: Optional[int] = None,
                     gather_groups: Optional[int] = None, gather_via: Optional[str] = None, **kwargs):
    """Run attention on this rank's heads; optionally all-gather the full output.

    q_local/k_local/v_local hold only this rank's heads (as produced by `local_heads` +
    `slice_heads`); `num_kv_heads` is the global kv-head count (defaults to num_q_heads).  With
    gather=False the local result is returned untouched and no collective is issued (a rank that
    owns no head returns an empty tensor).  With gather=True every rank returns the output for all
    `num_q_heads` heads in the input layout, and the collective is overlapped with the compute: the
    local kv-heads are processed in `gather_groups` groups (default: up to 4), and while group g+1 is
    computed on the current stream, group g is all-gathered by NCCL on a side stream.  `attn_fn`
    defaults to sageattention.sageattn.

    `gather_via`: "peer" stores the output rows straight into every rank's copy of the output from the
    attention epilogue (GPUs of one node, at most eight ranks, an attention function of this package, a head_dim
    of 64, 128 or 256); the returned tensor then lives in a buffer that is reused by the call after the
    next one with the same shapes.  "nccl" is the grouped all-gather described above.  The default (also
    settable as SAGE_B200_GATHER) is "peer" where it applies, else "nccl"."""
    via = gather_via or os.environ.get("SAGE_B200_GATHER", "peer")
    if via not in ("peer", "nccl"):
        raise ValueError("gather_via must be 'peer' or 'nccl'")
    own_fn = attn_fn is None or getattr(attn_fn, "__module__", "") == __name__.rsplit(".", 1)[0] + ".core"
    if (via == "peer" and gather and own_fn and q_local.is_cuda and dist.is_initialized()
            and 1 < dist.get_world_size(group) <= 8 and dist.get_backend(group) == "nccl"
            and q_local.size(-1) in (64, 128, 256)):
        kv = num_q_heads if num_kv_heads is None else num_kv_heads
        res = _sharded_into_peers(q_local, k_local, v_local, num_q_heads, kv, tensor_layout, group, attn_fn, kwargs)
        if res is not None:
            _last_exchange["via"] = "peer"
            return res
    if gather and dist.is_initialized() and dist.get_world_size(group) > 1:
        _last_exchange["via"] = dist.get_backend(group)
    if attn_fn is None:
        from .core import sageattn as attn_fn
    h_dim = 1 if tensor_layout == "HND" else 2
    n_q_local, n_kv_local = q_local.size(h_dim), k_local.size(h_dim)
    want_lse = bool(kwargs.get("return_lse"))
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    if not gather or world == 1:
        if n_kv_local == 0:                               # more ranks than kv-heads: nothing to compute here
            empty_lse = q_local.new_empty((q_local.size(0), 0, q_local.size(3 - h_dim)), dtype=torch.float32)
            return (q_local.new_empty(q_local.shape), empty_lse) if want_lse else q_local.new_empty(q_local.shape)
        return attn_fn(q_local, k_local, v_local, tensor_layout=tensor_layout, **kwargs)

    num_kv_heads = num_q_heads if num_kv_heads is None else num_kv_heads
    rep = num_q_heads // num_kv_heads
    per_kv = -(-num_kv_heads // world)                    # kv-head slots per rank (the last ranks may fill fewer)
    per = per_kv * rep                                    # q-head slots per rank
    groups = max(1, min(gather_groups or int(os.environ.get("SAGE_B200_GATHER_GROUPS", "4")), per_kv))
    bounds = [(g * per_kv // groups, (g + 1) * per_kv // groups) for g in range(groups)]
    on_gpu = q_local.is_cuda
    if on_gpu:
        group = _gather_group(group)
    # the gathered output, head-major: (world, per, *rest) with rest = the other dimensions in order
    rest = tuple(q_local.movedim(h_dim, 0).shape[1:])
    full = torch.empty((world, per) + rest, dtype=q_local.dtype, device=q_local.device)
    lse_rest = (q_local.size(0), q_local.size(3 - h_dim))             # (batch, seq)
    lse_full = torch.empty((world, per) + lse_rest, dtype=torch.float32, device=q_local.device) if want_lse else None
    main = torch.cuda.current_stream(q_local.device) if on_gpu else None
    side = torch.cuda.Stream(q_local.device, priority=-1) if on_gpu else None      # high priority, see _gather_group

    def gather_into(dst, slot, lo, hi):
        """all-gather `slot` ((hi - lo) head slots, head-major, contiguous) into dst[:, lo:hi] of every rank"""
        n = hi - lo
        if lo == 0 and hi == dst.size(1):                             # straight into the final buffer
            dist.all_gather_into_tensor(dst.view((world * n,) + tuple(dst.shape[2:])), slot, group=group)
        else:
            tmp = torch.empty((world * n,) + tuple(slot.shape[1:]), dtype=slot.dtype, device=slot.device)
            dist.all_gather_into_tensor(tmp, slot, group=group)
            dst[:, lo:hi].copy_(tmp.view((world, n) + tuple(slot.shape[1:])))
            if on_gpu:
                tmp.record_stream(side)

    for lo_kv, hi_kv in bounds:
        n_here = max(0, min(hi_kv, n_kv_local) - lo_kv)               # local kv-heads that fall into this group
        lo, hi = lo_kv * rep, hi_kv * rep
        slot = lse_slot = None
        if n_here > 0:
            res = attn_fn(slice_heads(q_local, tensor_layout, lo, lo + n_here * rep),
                          slice_heads(k_local, tensor_layout, lo_kv, lo_kv + n_here),
                          slice_heads(v_local, tensor_layout, lo_kv, lo_kv + n_here), tensor_layout=tensor_layout, **kwargs)
            out, lse = res if want_lse else (res, None)
            slot = out.movedim(h_dim, 0)
            lse_slot = lse.movedim(1, 0) if want_lse else None
        if n_here < hi_kv - lo_kv:                                    # a ragged or empty group: pad the slots
            pad = torch.zeros((hi - lo,) + rest, dtype=q_local.dtype, device=q_local.device)
            if slot is not None:
                pad[: slot.size(0)] = slot
            slot = pad
            if want_lse:
                lpad = torch.zeros((hi - lo,) + lse_rest, dtype=torch.float32, device=q_local.device)
                if lse_slot is not None:
                    lpad[: lse_slot.size(0)] = lse_slot
                lse_slot = lpad
        slot = slot.contiguous()
        if want_lse:
            lse_slot = lse_slot.contiguous()
        if on_gpu:
            side.wait_stream(main)
            with torch.cuda.stream(side):
                gather_into(full, slot, lo, hi)
                if want_lse:
                    gather_into(lse_full, lse_slot, lo, hi)
            slot.record_stream(side)
            if want_lse:
                lse_slot.record_stream(side)
        else:
            gather_into(full, slot, lo, hi)
            if want_lse:
                gather_into(lse_full, lse_slot, lo, hi)
    if on_gpu:
        main.wait_stream(side)
    out_full = full.reshape((world * per,) + rest)[:num_q_heads].movedim(0, h_dim)
    if want_lse:
        return out_full, lse_full.reshape((world * per,) + lse_rest)[:num_q_heads].movedim(0, 1)
    return out_full


# ---------------------------------------------------------------------------------------------------
# (batch x kv-head) grid sharding: for shapes whose head count does not divide over the GPUs
# (16 x 10 heads on 8 GPUs) the ranks form a wb x wh grid and each owns a rectangle of batches and
# kv-heads.  The grid is the factorisation of the world size that leaves the busiest rank the least
# work; with batch 1 it reduces to the head sharding above.
# ---------------------------------------------------------------------------------------------------
def shard_grid(batch: int, num_kv_heads: int, world_size: int) -> Tuple[int, int]:
    """(wb, wh) with wb * wh == world_size minimising ceil(batch/wb) * ceil(num_kv_heads/wh);
    ties go to the grid with more head shards."""
    if batch <= 0 or num_kv_heads <= 0 or world_size <= 0:
        raise ValueError("bad shard request")
    best = None
    for wb in range(1, world_size + 1):
        if world_size % wb:
            continue
        wh = world_size // wb
        load = -(-batch // wb) * -(-num_kv_heads // wh)
        if best is None or load < best[0] or (load == best[0] and wh > best[2]):
            best = (load, wb, wh)
    return best[1], best[2]


def local_block(batch: int, num_q_heads: int, num_kv_heads: int, world_size: int, rank: int):
    """(batch_range, q_head_range, kv_head_range) of this rank in the grid of `shard_grid`
    (rank = ib * wh + ih)."""
    if num_q_heads % num_kv_heads:
        raise ValueError("num_qo_heads must be divisible by num_kv_heads")
    wb, wh = shard_grid(batch, num_kv_heads, world_size)
    ib, ih = divmod(rank, wh)
    rep = num_q_heads // num_kv_heads
    b_lo, b_hi = shard_range(batch, wb, ib)
    k_lo, k_hi = shard_range(num_kv_heads, wh, ih)
    return (b_lo, b_hi), (k_lo * rep, k_hi * rep), (k_lo, k_hi)


def slice_block(t: torch.Tensor, tensor_layout: str, b_range, h_range) -> torch.Tensor:
    return slice_heads(t[b_range[0]:b_range[1]], tensor_layout, h_range[0], h_range[1])


def gather_blocks(out_local: torch.Tensor, batch: int, num_q_heads: int, num_kv_heads: int,
                  tensor_layout: str = "HND", group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """All-gather of the rectangles of `local_block` into the full (batch, ..., heads, ...) output on every
    rank: one NCCL all-gather of equal-sized slots, then one copy per rank's rectangle."""
    world = dist.get_world_size(group)
    wb, wh = shard_grid(batch, num_kv_heads, world)
    rep = num_q_heads // num_kv_heads
    pb, ph = -(-batch // wb), -(-num_kv_heads // wh) * rep
    h_dim = 1 if tensor_layout == "HND" else 2
    full_shape = list(out_local.shape)
    full_shape[0], full_shape[h_dim] = batch, num_q_heads
    slot_shape = list(out_local.shape)
    slot_shape[0], slot_shape[h_dim] = pb, ph
    slot = torch.zeros(slot_shape, dtype=out_local.dtype, device=out_local.device)
    if out_local.numel():
        slice_heads(slot[: out_local.size(0)], tensor_layout, 0, out_local.size(h_dim)).copy_(out_local)
    cat_shape = list(slot_shape)
    cat_shape[0] = world * pb                        # slots concatenated along the batch dimension
    gathered = torch.empty(cat_shape, dtype=out_local.dtype, device=out_local.device)
    dist.all_gather_into_tensor(gathered, slot, group=group)
    full = torch.empty(full_shape, dtype=out_local.dtype, device=out_local.device)
    for r in range(world):
        (b_lo, b_hi), (q_lo, q_hi), _ = local_block(batch, num_q_heads, num_kv_heads, world, r)
        if b_hi > b_lo and q_hi > q_lo:
            src = slice_heads(gathered[r * pb: r * pb + (b_hi - b_lo)], tensor_layout, 0, q_hi - q_lo)
            slice_heads(full[b_lo:b_hi], tensor_layout, q_lo, q_hi).copy_(src)
    return full
