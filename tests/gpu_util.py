"""Shared helpers for the GPU parity tests."""
import os

import pytest
import torch

os.environ.setdefault("SAGE_B200_CHECK", "1")

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF_SO = os.path.join(ROOT, "oracle", "_ref", "libsage_ref_sm80.so")

requires_gpu = pytest.mark.gpu


def cuda_or_fail():
    # a GPU test on a machine without a GPU is a configuration error, not a skip
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    return torch.device("cuda:0")


def make_qkv(B, Hq, Hkv, N, D, dtype, layout, seed, k_bias=0.0, k_outliers=0.0, Nkv=None, device="cuda"):
    g = torch.Generator(device="cpu").manual_seed(seed)
    Nkv = N if Nkv is None else Nkv

    def shape(h, n):
        return (B, n, h, D) if layout == "NHD" else (B, h, n, D)
    q = torch.randn(shape(Hq, N), generator=g)
    k = torch.randn(shape(Hkv, Nkv), generator=g)
    v = torch.randn(shape(Hkv, Nkv), generator=g)
    if k_bias:
        bshape = (1, 1, Hkv, D) if layout == "NHD" else (1, Hkv, 1, D)
        k = k + k_bias * torch.randn(bshape, generator=g)
    if k_outliers:
        for h in range(Hkv):
            ch = torch.randperm(D, generator=g)[:4]
            if layout == "NHD":
                k[:, :, h, ch] *= k_outliers
            else:
                k[:, h, :, ch] *= k_outliers
    return q.to(dtype).to(device), k.to(dtype).to(device), v.to(dtype).to(device)


_ref_loaded = None


def reference_ops():
    """torch.ops namespace of the reference's sm80 kernels rebuilt for sm_100, or None."""
    global _ref_loaded
    if _ref_loaded is None:
        _ref_loaded = False
        if os.path.exists(REF_SO):
            try:
                torch.ops.load_library(REF_SO)
                _ref_loaded = torch.ops.sageattention_qattn_sm80
            except Exception as e:  # pragma: no cover - reported by the test that needs it
                print("could not load reference kernels:", e)
    return _ref_loaded or None
