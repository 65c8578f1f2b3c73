"""Host-buffer entry point: Q, K, V in (pinned) host memory, result back in host memory.

Heads are independent, so the call is pipelined over groups of kv-heads: while one group is being
computed, the next one is copied in and the previous result is copied out, each on its own stream, through
a small ring of device buffers.  This is the end-to-end path the benchmark reports as `e2e`.

A step is some hundred stream operations (32 groups x copies, launches, events).  Issued from Python every
time, its duration follows the host: on a busy machine the GPU waits for the interpreter.  With pinned
buffers the whole step is therefore captured once into a CUDA graph (copies from and to the caller's
buffers included) and replayed with one launch on every later call with the same buffers and options.
"""
from __future__ import annotations

import os
import warnings
from collections import OrderedDict
from typing import Optional

import torch

from . import core
from .core import sageattn
from .parallel import slice_heads

_RING = 3             # device buffers per tensor: one being filled, one being computed on, one being copied out
_MAX_PLANS = 4        # captured steps kept per process (each holds its ring and the graph's private pool)
_plans: "OrderedDict[tuple, _Plan]" = OrderedDict()


class _Plan:
    """Ring buffers, streams and events of one (shapes, chunking, device) combination, and the captured
    graph of one (buffers, options) combination."""

    def __init__(self, q, k, device, tensor_layout, step, rep):
        h_dim = 1 if tensor_layout == "HND" else 2
        qs, ks = list(q.shape), list(k.shape)
        qs[h_dim], ks[h_dim] = step * rep, step
        self.slots = [{"q": torch.empty(qs, dtype=q.dtype, device=device),
                       "k": torch.empty(ks, dtype=k.dtype, device=device),
                       "v": torch.empty(ks, dtype=k.dtype, device=device),
                       "o": torch.empty(qs, dtype=q.dtype, device=device)} for _ in range(_RING)]
        self.s_in, self.s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
        self.copied_in = [torch.cuda.Event() for _ in range(_RING)]
        self.computed = [torch.cuda.Event() for _ in range(_RING)]
        self.copied_out = [torch.cuda.Event() for _ in range(_RING)]
        self.graph = None
        self.graph_failed = False


def _issue(plan, q, k, v, out, tensor_layout, bounds, rep, main, attn_fn, kwargs):
    """One pipelined step on `main` (compute), plan.s_in and plan.s_out.  Nothing is waited for here."""
    for idx, (lo, hi) in enumerate(bounds):
        s = idx % _RING
        slot = plan.slots[s]
        n = hi - lo
        dq, dk, dv, do = (slice_heads(slot[name], tensor_layout, 0, n * (rep if name in "qo" else 1))
                          for name in ("q", "k", "v", "o"))
        with torch.cuda.stream(plan.s_in):
            if idx >= _RING:
                plan.s_in.wait_event(plan.computed[s])          # the slot's previous inputs have been read
            dq.copy_(slice_heads(q, tensor_layout, lo * rep, hi * rep), non_blocking=True)
            dk.copy_(slice_heads(k, tensor_layout, lo, hi), non_blocking=True)
            dv.copy_(slice_heads(v, tensor_layout, lo, hi), non_blocking=True)
            plan.copied_in[s].record(plan.s_in)
        main.wait_event(plan.copied_in[s])
        if idx >= _RING:
            main.wait_event(plan.copied_out[s])                 # the slot's previous result has left
        with core.output_into(do):
            attn_fn(dq, dk, dv, tensor_layout=tensor_layout, **kwargs)
        plan.computed[s].record(main)
        plan.s_out.wait_event(plan.computed[s])
        with torch.cuda.stream(plan.s_out):
            slice_heads(out, tensor_layout, lo * rep, hi * rep).copy_(do, non_blocking=True)
            plan.copied_out[s].record(plan.s_out)


def sageattn_host(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, out: Optional[torch.Tensor] = None,
                  tensor_layout: str = "HND", kv_heads_per_chunk: Optional[int] = None,
                  device: Optional[torch.device] = None, attn_fn=None, use_graph: Optional[bool] = None,
                  **kwargs) -> torch.Tensor:
    """q, k, v: CPU tensors (pin them for asynchronous copies).  Returns a CPU tensor shaped like q
    (written into `out` when given).  Extra keyword arguments go to `attn_fn` (default `sageattn`; it must
    be one of this package's attention functions).

    `use_graph` (default on, SAGE_B200_HOST_GRAPH=0 turns it off; it needs pinned q, k, v and out whose head
    groups are contiguous, i.e. batch 1 in HND, and is ignored otherwise): the first call
    with a given set of buffers and options runs step by step and then captures the step; later calls
    replay it.  The graph reads and writes the same host addresses, so it is only reused while the
    caller passes the same tensors."""
    attn_fn = sageattn if attn_fn is None else attn_fn
    if q.is_cuda or k.is_cuda or v.is_cuda:
        raise ValueError("sageattn_host takes host tensors; use sageattn for device tensors.")
    if kwargs.get("return_lse"):
        raise ValueError("return_lse is not supported by sageattn_host.")
    if getattr(attn_fn, "__module__", "") != core.__name__:
        raise ValueError("sageattn_host runs this package's attention functions only.")
    if tensor_layout not in ("NHD", "HND"):
        raise ValueError("tensor_layout must be 'NHD' or 'HND'.")
    if q.size(-1) not in (64, 128, 256):
        # the ring holds unpadded tensors and the kernels write straight into it
        raise ValueError("sageattn_host needs a head_dim of 64, 128 or 256.")
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
    # the last group goes head by head: whatever follows the last copy in is not overlapped
    bounds = [(lo, min(hkv, lo + step)) for lo in range(0, hkv, step)]
    if step > 1:
        lo_last, hi_last = bounds.pop()
        bounds += [(h, h + 1) for h in range(lo_last, hi_last)]

    pinned = all(t.is_pinned() for t in (q, k, v, out))
    # a graph holds plain copies between fixed addresses: every group must be one contiguous range on
    # both sides (batch 1 in HND); strided groups are staged by torch on the host and run step by step
    lo0, hi0 = bounds[0]
    one_range = (slice_heads(q, tensor_layout, lo0 * rep, hi0 * rep).is_contiguous() and
                 slice_heads(k, tensor_layout, lo0, hi0).is_contiguous() and
                 slice_heads(v, tensor_layout, lo0, hi0).is_contiguous() and
                 slice_heads(out, tensor_layout, lo0 * rep, hi0 * rep).is_contiguous() and
                 (tensor_layout == "HND" and q.size(0) == 1))
    if use_graph is None:
        use_graph = os.environ.get("SAGE_B200_HOST_GRAPH", "1") != "0"
    use_graph = bool(use_graph) and pinned and one_range
    key = (tuple(q.shape), tuple(k.shape), q.dtype, tensor_layout, step, device.index,
           q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), attn_fn.__name__,
           tuple(sorted((name, repr(val)) for name, val in kwargs.items())))
    plan = _plans.get(key)
    if plan is None:
        plan = _Plan(q, k, device, tensor_layout, step, rep)
        _plans[key] = plan
        while len(_plans) > _MAX_PLANS:
            _plans.popitem(last=False)
    else:
        _plans.move_to_end(key)

    with torch.cuda.device(device):
        main = torch.cuda.current_stream(device)
        if plan.graph is not None:
            plan.graph.replay()
            main.synchronize()
            return out
        # step by step
        plan.s_in.wait_stream(main)
        plan.s_out.wait_stream(main)
        _issue(plan, q, k, v, out, tensor_layout, bounds, rep, main, attn_fn, kwargs)
        plan.s_out.synchronize()
        main.synchronize()
        if use_graph and not plan.graph_failed:
            # capture the same step for the following calls (nothing runs during the capture)
            graph = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream(device)
            try:
                with torch.cuda.graph(graph, stream=side):
                    cap = torch.cuda.current_stream(device)
                    plan.s_in.wait_stream(cap)
                    plan.s_out.wait_stream(cap)
                    _issue(plan, q, k, v, out, tensor_layout, bounds, rep, cap, attn_fn, kwargs)
                    cap.wait_stream(plan.s_in)
                    cap.wait_stream(plan.s_out)
                plan.graph = graph
            except Exception as err:                              # keep working step by step
                plan.graph_failed = True
                warnings.warn(f"sageattn_host: the step could not be captured into a graph ({err})", stacklevel=2)
                torch.cuda.synchronize(device)
    return out
