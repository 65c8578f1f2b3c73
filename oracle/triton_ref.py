"""Runs the reference's Triton quantisers on a GPU from prebuilt cubins.  TEST INFRASTRUCTURE.

``oracle/build_triton_ref.py`` compiles the reference's kernels
(sageattention/triton/quant_per_thread.py:22-115, quant_per_block.py:32-78) to
``oracle/_ref/triton_quant/*.cubin``.  This module loads them through the CUDA
driver API and launches them with the grids, strides and scale shapes of the
reference's host wrappers (quant_per_thread.py:118-205, quant_per_block.py:81-173),
so GPU tests can compare the product's quantisers with the reference's device
arithmetic bit for bit.  Only tests may import it.
"""
from __future__ import annotations

import ctypes
import json
import os

import torch

_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "_ref", "triton_quant")
_cache: dict = {}


def available() -> bool:
    return os.path.exists(os.path.join(_DIR, "manifest.json"))


def _check(res):
    err = res[0]
    if int(err) != 0:
        raise RuntimeError(f"CUDA driver error {err}")
    return res[1] if len(res) == 2 else res[1:]


def _kernel(key: str):
    from cuda.bindings import driver as drv
    if "manifest" not in _cache:
        with open(os.path.join(_DIR, "manifest.json")) as f:
            _cache["manifest"] = json.load(f)
    dev = torch.cuda.current_device()
    ck = (key, dev)
    if ck not in _cache:
        torch.cuda.init()
        torch.zeros(1, device="cuda")          # make torch's primary context current
        meta = _cache["manifest"][key]
        with open(os.path.join(_DIR, key + ".cubin"), "rb") as f:
            image = f.read()
        mod = _check(drv.cuModuleLoadData(image))
        fn = _check(drv.cuModuleGetFunction(mod, meta["name"].encode()))
        _cache[ck] = (fn, meta, mod)
    return _cache[ck][:2]


def _launch(key: str, grid, ptrs_and_ints):
    from cuda.bindings import driver as drv
    fn, meta = _kernel(key)
    vals, types = [], []
    for a in ptrs_and_ints:
        if isinstance(a, torch.Tensor):
            vals.append(a.data_ptr())
            types.append(ctypes.c_void_p)
        else:
            vals.append(int(a))
            types.append(ctypes.c_int32)
    # trailing global-scratch and profile-scratch pointers of Triton >= 3.4 kernels
    vals += [0, 0]
    types += [ctypes.c_void_p, ctypes.c_void_p]
    stream = torch.cuda.current_stream().cuda_stream
    _check(drv.cuLaunchKernel(fn, grid[0], grid[1], grid[2], 32 * meta["num_warps"], 1, 1,
                              meta["shared"], stream, (tuple(vals), tuple(types)), 0))


def _dt(t: torch.Tensor) -> str:
    return {torch.float16: "f16", torch.bfloat16: "bf16"}[t.dtype]


def _strides(t: torch.Tensor, layout: str):
    if layout == "HND":
        return t.stride(0), t.stride(1), t.stride(2)
    return t.stride(0), t.stride(2), t.stride(1)


def _dims(t: torch.Tensor, layout: str):
    if layout == "HND":
        b, h, n, d = t.shape
    else:
        b, n, h, d = t.shape
    return b, h, n, d


def per_thread_int8(q, k, km=None, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, tensor_layout="HND"):
    q8 = torch.empty(q.shape, dtype=torch.int8, device=q.device)
    k8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    b, hq, nq, d = _dims(q, tensor_layout)
    _, hkv, nk, _ = _dims(k, tensor_layout)
    qb = -(-nq // BLKQ)
    kb = -(-nk // BLKK)
    q_scale = torch.empty((b, hq, qb * (BLKQ // WARPQ) * 8), device=q.device, dtype=torch.float32)
    k_scale = torch.empty((b, hkv, kb * (BLKK // WARPK) * 4), device=q.device, dtype=torch.float32)
    _launch(f"q_thread_{_dt(q)}_c{d}_blk{WARPQ}", (qb * (BLKQ // WARPQ) * 8, hq, b),
            [q, q8, q_scale, nq, *_strides(q, tensor_layout), *_strides(q8, tensor_layout),
             q_scale.stride(0), q_scale.stride(1)])
    if km is not None:
        kms = km.squeeze(2 if tensor_layout == "HND" else 1)
        mstr = (kms.stride(0), kms.stride(1), kms.stride(2))
        mean = km
    else:
        mstr = (0, 0, 0)
        mean = k
    _launch(f"k_thread_{_dt(k)}_c{d}_blk{WARPK}_m{int(km is not None)}", (kb * (BLKK // WARPK) * 4, hkv, b),
            [k, mean, k8, k_scale, nk, *_strides(k, tensor_layout), *mstr, *_strides(k8, tensor_layout),
             k_scale.stride(0), k_scale.stride(1)])
    return q8, q_scale, k8, k_scale


def per_block_int8(q, k, km=None, BLKQ=128, BLKK=64, tensor_layout="HND"):
    q8 = torch.empty(q.shape, dtype=torch.int8, device=q.device)
    k8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    b, hq, nq, d = _dims(q, tensor_layout)
    _, hkv, nk, _ = _dims(k, tensor_layout)
    qb = -(-nq // BLKQ)
    kb = -(-nk // BLKK)
    q_scale = torch.empty((b, hq, qb), device=q.device, dtype=torch.float32)
    k_scale = torch.empty((b, hkv, kb), device=q.device, dtype=torch.float32)
    _launch(f"block_{_dt(q)}_c{d}_blk{BLKQ}_m0", (qb, hq, b),
            [q, q, q8, q_scale, nq, 0, *_strides(q, tensor_layout), 0, 0, 0,
             *_strides(q8, tensor_layout), q_scale.stride(0), q_scale.stride(1)])
    if km is not None:
        kms = km.squeeze(2 if tensor_layout == "HND" else 1)
        mstr = (kms.stride(0), kms.stride(1), kms.stride(2))
        mean = km
    else:
        mstr = (0, 0, 0)
        mean = k
    _launch(f"block_{_dt(k)}_c{d}_blk{BLKK}_m{int(km is not None)}", (kb, hkv, b),
            [k, mean, k8, k_scale, nk, 0, *_strides(k, tensor_layout), *mstr,
             *_strides(k8, tensor_layout), k_scale.stride(0), k_scale.stride(1)])
    return q8, q_scale, k8, k_scale
