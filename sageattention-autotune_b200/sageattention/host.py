"""Host-buffer entry point: Q, K, V in (pinned) host memory, result back in host memory.

Heads are independent, so the call is pipelined over groups of kv-heads: while one group is being
computed, the next one is copied in and the previous result is copied out, each on its own stream.
This is the end-to-end path the benchmark reports as `e2e`.
"""
from __future__ import annotations

from typing import Optional

import torch

from .core import sageattn
from .parallel import slice_heads


def sageattn_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                  tensor_layout: str = "HND", kv_heads_per_chunk: Optional[int] = None,
                  device: Optional[torch.device] = None, attn_fn=None, **kwargs) -> torch.Tensor:
    """q, k, v: CPU tensors (pin them for asynchronous copies).  Returns a CPU tensor shaped like q
    (written into `out` when given).  Extra keyword arguments go to `attn_fn` (default `sageattn`)."""
    attn_fn = sageattn if attn_fn is None else attn_fn
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("sageattn_host takes host tensors; use sageattn for device tensors.")
    if kwargs.get("return_lse"):
        raise ValueError("return_lse is not supported by sageattn_host.")
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    h_dim = 1 if tensor_layout == "HND" else 2
    hq, hkv = q.size(h_dim), k.size(h_dim)
    if hq % hkv:
        raise ValueError("num_qo_heads must be divisible by num_kv_heads")
    rep = hq // hkv
    # 32 chunks: the copies in are the bound (29.1 ms for 64 heads x 32768 fp16, 30.0 ms with the copy out
    # running against them), so what counts is how little is left after the last one lands: the last
    # chunk's compute and copy out.  Measured for that case: 34.2 ms with 8 chunks, 32.6-33.1 with 16,
    # 31.7 with 32 (two heads = 512 CTAs still fill the GPU), 33.8 with 64.
    step = kv_heads_per_chunk or max(1, hkv // 32)
    if out is None:
        out = torch.empty(q.shape, dtype=q.dtype, pin_memory=True)
    main = torch.cuda.current_stream(device)
    s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
    pending = []
    with torch.cuda.device(device):
        # the last group goes head by head: whatever follows the last copy in is not overlapped
        bounds = [(lo, min(hkv, lo + step)) for lo in range(0, hkv, step)]
        if step > 1:
            lo_last, hi_last = bounds.pop()
            bounds += [(h, h + 1) for h in range(lo_last, hi_last)]
        for lo, hi in bounds:
            with torch.cuda.stream(s_in):
                dq = slice_heads(q, tensor_layout, lo * rep, hi * rep).to(device, non_blocking=True)
                dk = slice_heads(k, tensor_layout, lo, hi).to(device, non_blocking=True)
                dv = slice_heads(v, tensor_layout, lo, hi).to(device, non_blocking=True)
                ready = torch.cuda.Event()
                ready.record(s_in)
            main.wait_event(ready)
            o = attn_fn(dq, dk, dv, tensor_layout=tensor_layout, **kwargs)
            for t in (dq, dk, dv):
                t.record_stream(main)
            done = torch.cuda.Event()
            done.record(main)
            s_out.wait_event(done)
            with torch.cuda.stream(s_out):
                slice_heads(out, tensor_layout, lo * rep, hi * rep).copy_(o, non_blocking=True)
                o.record_stream(s_out)
            pending.append(o)
        s_out.synchronize()
    return out
