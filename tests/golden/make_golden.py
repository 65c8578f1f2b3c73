"""Regenerates the golden vectors in this folder from the reference's own kernels.

Run where the reference checkout is available (it is not needed to *use* the
fixtures):

    TRITON_INTERPRET=1 python tests/golden/make_golden.py --ref /path/to/reference

The reference's Triton quantisers (sageattention/triton/quant_per_thread.py,
quant_per_block.py) and its Triton attention kernel
(sageattention/triton/attn_qk_int8_per_block.py) are executed on CPU tensors by
Triton's interpreter; their inputs and outputs are stored bit for bit.  The
``triton.autotune`` wrappers need a GPU driver to time candidates, so they are
bypassed by calling the wrapped ``.fn`` directly - the kernel bodies that run are
the reference's, unmodified.

Each fixture is one ``.npz``: 16-bit inputs are stored as their uint16 bit patterns
(``*_bits``) with the dtype name in ``dtype``.
"""
from __future__ import annotations

import argparse
import os
import sys

os.environ.setdefault("TRITON_INTERPRET", "1")

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16)


def make_inputs(case: dict):
    g = torch.Generator().manual_seed(case["seed"])
    dt = getattr(torch, case["dtype"])
    B, Hq, Hkv, N, D = case["B"], case["Hq"], case["Hkv"], case["N"], case["D"]
    def shape(h):
        return (B, N, h, D) if case["layout"] == "NHD" else (B, h, N, D)
    q = torch.randn(shape(Hq), generator=g).to(dt)
    k = torch.randn(shape(Hkv), generator=g)
    v = torch.randn(shape(Hkv), generator=g).to(dt)
    if case.get("k_bias"):
        bshape = (1, 1, Hkv, D) if case["layout"] == "NHD" else (1, Hkv, 1, D)
        k = k + case["k_bias"] * torch.randn(bshape, generator=g)
    if case.get("k_outliers"):
        for h in range(Hkv):
            ch = torch.randperm(D, generator=g)[:4]
            if case["layout"] == "NHD":
                k[:, :, h, ch] *= case["k_outliers"]
            else:
                k[:, h, :, ch] *= case["k_outliers"]
    return q, k.to(dt), v


CASES = [
    # the tiny correctness case
    dict(name="c1_nhd_fp16_d64", seed=0, B=1, Hq=2, Hkv=2, N=256, D=64, dtype="float16",
         layout="NHD", smooth_k=True, attn=True),
    # ragged tail + biased K + GQA, bf16, HND
    dict(name="tail_bias_gqa_hnd_bf16_d128", seed=3, B=1, Hq=4, Hkv=2, N=200, D=128,
         dtype="bfloat16", layout="HND", smooth_k=True, k_bias=2.0, attn=False),
    # outlier channels (x20), bf16, NHD
    dict(name="outliers_nhd_bf16_d128", seed=2, B=2, Hq=2, Hkv=2, N=320, D=128,
         dtype="bfloat16", layout="NHD", smooth_k=True, k_outliers=20.0, attn=False),
    # no smoothing, odd length, D=64
    dict(name="nosmooth_hnd_fp16_d64", seed=5, B=1, Hq=3, Hkv=3, N=129, D=64, dtype="float16",
         layout="HND", smooth_k=False, attn=True),
]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("SAGE_REFERENCE_DIR"), required="SAGE_REFERENCE_DIR" not in os.environ,
                    help="checkout of woct0rdho/sageattention-autotune (or set SAGE_REFERENCE_DIR)")
    args = ap.parse_args()
    sys.path.insert(0, args.ref)

    import importlib
    qpt = importlib.import_module("sageattention.triton.quant_per_thread")
    qpb = importlib.import_module("sageattention.triton.quant_per_block")
    att = importlib.import_module("sageattention.triton.attn_qk_int8_per_block")
    # bypass the autotuner wrappers (they benchmark on a GPU); the kernel body is unchanged
    qpb.quant_per_block_int8_kernel = qpb.quant_per_block_int8_kernel.fn
    att._attn_fwd = att._attn_fwd.fn

    for case in CASES:
        q, k, v = make_inputs(case)
        seq_dim = 1 if case["layout"] == "NHD" else 2
        km = k.mean(dim=seq_dim, keepdim=True) if case["smooth_k"] else None
        out = dict(dtype=case["dtype"], layout=case["layout"], smooth_k=case["smooth_k"],
                   q_bits=bits(q), k_bits=bits(k), v_bits=bits(v))
        if km is not None:
            out["km_bits"] = bits(km)
        for cfg in [(128, 64, 32, 64), (64, 64, 32, 64), (128, 64, 16, 64), (128, 32, 32, 32)]:
            tag = "pt_%d_%d_%d_%d" % cfg
            q8, qs, k8, ks = qpt.per_thread_int8(q, k, km, BLKQ=cfg[0], WARPQ=cfg[2], BLKK=cfg[1],
                                                 WARPK=cfg[3], tensor_layout=case["layout"])
            if cfg == (128, 64, 32, 64):
                out[tag + "_q8"], out[tag + "_k8"] = q8.numpy(), k8.numpy()
            out[tag + "_qs"], out[tag + "_ks"] = qs.numpy(), ks.numpy()
            # the int8 payloads of the other groupings are stored as a checksum only
            out[tag + "_q8sum"] = np.array([int(q8.long().sum()), int((q8.long() * q8.long()).sum())])
            out[tag + "_k8sum"] = np.array([int(k8.long().sum()), int((k8.long() * k8.long()).sum())])
        q8, qs, k8, ks = qpb.per_block_int8(q, k, km, BLKQ=128, BLKK=64, tensor_layout=case["layout"])
        out["pb_128_64_q8"], out["pb_128_64_k8"] = q8.numpy(), k8.numpy()
        out["pb_128_64_qs"], out["pb_128_64_ks"] = qs.numpy(), ks.numpy()
        if case["attn"]:
            # Triton attention kernel of the reference on the per-block tensors
            # (attn_qk_int8_per_block.py:264-350): fp32 accumulate, LSE in
            # base 2 exactly as the kernel writes it.
            for causal in (False, True):
                o, lse = att.forward(q8, k8, v.to(torch.float16), qs, ks, tensor_layout=case["layout"],
                                     is_causal=causal, pv_accum_dtype="fp32", BLOCK_M=128, BLOCK_N=64,
                                     output_dtype=q.dtype, return_lse=True)
                sfx = "_causal" if causal else ""
                out["tri_o_bits" + sfx] = bits(o)
                out["tri_lse" + sfx] = lse.numpy()
        path = os.path.join(HERE, case["name"] + ".npz")
        np.savez_compressed(path, **out)
        print("wrote", path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
