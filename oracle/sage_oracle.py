"""CPU restatement of the SageAttention forward path.  TEST INFRASTRUCTURE ONLY.

Nothing in the shipped package may import this module: it exists so that the
tests, the smoke check and the ``cpu_baseline`` / ``--impl reference`` legs of
``bench.py`` have an independent statement of the algorithm to compare the CUDA
kernels with (and to time on the host cores).

What it follows in the reference (woct0rdho/sageattention-autotune):

* ``mean_k``                 sageattention/cuda_attn.py:167-170
* ``quant_per_thread``       sageattention/triton/quant_per_thread.py:39-57 (Q),
                             :82-115 (K), host wrapper :118-205
* ``quant_per_block``        sageattention/triton/quant_per_block.py:54-78, :81-173
* ``attend``                 csrc/qattn/qk_int8_sv_f16_kernel_sm80.cuh:105-126,
                             :240-347, :379-387, :476-528 and
                             csrc/qattn/attn_utils.cuh:222-406, :447-574
* ``sageattn``               sageattention/cuda_attn.py:126-274,
                             sageattention/utils.py:17-49

Parity pin: the two quantisers are checked bit for bit against the reference's
own Triton kernels run under ``TRITON_INTERPRET=1`` (the fixtures in
``tests/golden/`` and the script next to them); ``attend`` is checked against the
reference's Triton attention kernel run the same way (per-block scales, fp32
accumulate, with LSE) and, on a GPU, against the reference's sm80 CUDA kernel
rebuilt for sm_100 (``oracle/_ref``).  Pieces the reference does not implement
(``sm_scale`` argument, fp8 PV, multi-GPU gather) are parity-unpinned.

Division note: the interpreter evaluates ``/`` as IEEE division, the same Triton
source compiled for a GPU uses ``div.full.f32`` (approximate, <= 2 ulp).  This
file is IEEE; the CUDA quantisers have both modes.
"""
from __future__ import annotations

import math

import numpy as np
import torch

LOG2_E = 1.44269504088896340736
_NEG_BIG = -5000000.0


# --------------------------------------------------------------------------
# layout helpers: everything below works on (B, H, N, D) views
# --------------------------------------------------------------------------
def to_bhnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    if tensor_layout == "HND":
        return x
    if tensor_layout == "NHD":
        return x.transpose(1, 2)
    raise ValueError(f"Unknown tensor layout: {tensor_layout}")


def from_bhnd(x: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    return x if tensor_layout == "HND" else x.transpose(1, 2)


def padded_head_dim(head_dim: int) -> int:
    """sageattention/utils.py:17-26."""
    if head_dim <= 64:
        return 64
    if head_dim <= 128:
        return 128
    if head_dim <= 256:
        return 256
    raise ValueError(f"Unsupported head_dim: {head_dim}")


def mean_k(k: torch.Tensor, tensor_layout: str) -> torch.Tensor:
    """Channel mean of K over the sequence, rounded to k's dtype (cuda_attn.py:167-170)."""
    seq_dim = 2 if tensor_layout == "HND" else 1
    return k.float().mean(dim=seq_dim, keepdim=True).to(k.dtype)


# --------------------------------------------------------------------------
# quantisers
# --------------------------------------------------------------------------
def _round_to_int8(y: np.ndarray) -> np.ndarray:
    # y + (y >= 0 ? 0.5 : -0.5), then truncate toward zero (quant_per_thread.py:53-56)
    y = y + np.where(y >= 0, np.float32(0.5), np.float32(-0.5)).astype(np.float32)
    return np.trunc(y).astype(np.int8)


def _pad_rows(x: np.ndarray, mult: int) -> np.ndarray:
    n = x.shape[2]
    n_pad = -(-n // mult) * mult
    if n_pad == n:
        return x
    out = np.zeros(x.shape[:2] + (n_pad,) + x.shape[3:], dtype=x.dtype)
    out[:, :, :n] = x
    return out


def _quant_groups(x: np.ndarray, n_valid: int, blk: int, warp: int, rows_per_lane: int, eps: float):
    """x: fp32 (B,H,Npad,D) with Npad a multiple of blk (masked rows already hold what
    the reference's masked loads produce).  Rows of one ``warp``-row block are dealt
    to 8 // rows_per_lane groups: row r belongs to group (r % 8) // rows_per_lane.
    rows_per_lane = 1 is the reference's Q grouping, 2 its K grouping, 8 * (warp // 8)
    degenerates to one group per block (per-block quantisation, blk == warp)."""
    B, H, Np, D = x.shape
    nwb = Np // warp
    if rows_per_lane >= 8:
        g = 1
        xr = x.reshape(B, H, nwb, 1, warp, D)           # (.., group, rows, D)
        amax = np.abs(xr).max(axis=(4, 5))
    else:
        g = 8 // rows_per_lane
        xr = x.reshape(B, H, nwb, warp // 8, g, rows_per_lane, D)
        amax = np.abs(xr).max(axis=(3, 5, 6))            # (B,H,nwb,g)
    scale = (amax.astype(np.float32) / np.float32(127.0)).astype(np.float32)
    if eps:
        scale = (scale + np.float32(eps)).astype(np.float32)
    if rows_per_lane >= 8:
        sc_b = scale.reshape(B, H, nwb, 1, 1, 1)
    else:
        sc_b = scale.reshape(B, H, nwb, 1, g, 1, 1)
    with np.errstate(divide="ignore", invalid="ignore"):
        y = (xr / sc_b).astype(np.float32)
        q = _round_to_int8(np.nan_to_num(y, nan=0.0, posinf=0.0, neginf=0.0))
    q = q.reshape(B, H, Np, D)[:, :, :n_valid]
    return q, scale.reshape(B, H, nwb * g)


def quant_per_thread(q, k, km=None, BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, tensor_layout="HND"):
    """Restates per_thread_int8 (quant_per_thread.py:118-205).  Returns
    (q_int8, q_scale, k_int8, k_scale) with the int8 tensors in the input layout."""
    qb = to_bhnd(q, tensor_layout).float().numpy()
    kb = to_bhnd(k, tensor_layout).float().numpy()
    nq, nk = qb.shape[2], kb.shape[2]
    qp = _pad_rows(qb, BLKQ)
    kp = _pad_rows(kb, BLKK)
    if km is not None:
        kmb = to_bhnd(km, tensor_layout).float().numpy()      # (B,Hkv,1,D)
        kp = (kp - kmb).astype(np.float32)                      # masked rows too (:100-104)
    q8, qs = _quant_groups(qp, nq, BLKQ, WARPQ, 1, 1e-7)
    k8, ks = _quant_groups(kp, nk, BLKK, WARPK, 2, 1e-7)
    q8 = from_bhnd(torch.from_numpy(q8), tensor_layout).contiguous()
    k8 = from_bhnd(torch.from_numpy(k8), tensor_layout).contiguous()
    return q8, torch.from_numpy(qs), k8, torch.from_numpy(ks)


def quant_per_block(q, k, km=None, BLKQ=128, BLKK=64, tensor_layout="HND"):
    """Restates per_block_int8 (quant_per_block.py:81-173): one scale per BLK x D tile,
    no epsilon."""
    qb = to_bhnd(q, tensor_layout).float().numpy()
    kb = to_bhnd(k, tensor_layout).float().numpy()
    nq, nk = qb.shape[2], kb.shape[2]
    qp = _pad_rows(qb, BLKQ)
    kp = _pad_rows(kb, BLKK)
    if km is not None:
        kmb = to_bhnd(km, tensor_layout).float().numpy()
        kp = (kp - kmb).astype(np.float32)
    q8, qs = _quant_groups(qp, nq, BLKQ, BLKQ, 8, 0.0)
    k8, ks = _quant_groups(kp, nk, BLKK, BLKK, 8, 0.0)
    q8 = from_bhnd(torch.from_numpy(q8), tensor_layout).contiguous()
    k8 = from_bhnd(torch.from_numpy(k8), tensor_layout).contiguous()
    return q8, torch.from_numpy(qs), k8, torch.from_numpy(ks)


# --------------------------------------------------------------------------
# attention on quantised inputs
# --------------------------------------------------------------------------
def expand_q_scale(q_scale: torch.Tensor, nq: int, BLKQ: int, WARPQ: int, granularity: str) -> torch.Tensor:
    """(B,H,groups) -> per-row scale (B,H,nq) using the kernel's fragment contract
    (qk_int8_sv_f16_kernel_sm80.cuh:116-119): row r reads group (r // WARPQ) * 8 + r % 8."""
    r = torch.arange(nq)
    idx = (r // WARPQ) * 8 + (r % 8) if granularity == "per_thread" else r // BLKQ
    return q_scale[:, :, idx]


def expand_k_scale(k_scale: torch.Tensor, nk: int, BLKK: int, WARPK: int, granularity: str) -> torch.Tensor:
    """(B,Hkv,groups) -> per-key scale: key c reads group (c // WARPK) * 4 + (c % 8) // 2
    (qk_int8_sv_f16_kernel_sm80.cuh:121-126)."""
    c = torch.arange(nk)
    idx = (c // WARPK) * 4 + (c % 8) // 2 if granularity == "per_thread" else c // BLKK
    return k_scale[:, :, idx]


def attend(q_int8, k_int8, v16, q_scale, k_scale, tensor_layout="HND", is_causal=False,
           sm_scale=None, pv_accum_dtype="fp32", granularity="per_thread",
           BLKQ=128, WARPQ=32, BLKK=64, WARPK=64, out_dtype=torch.float16,
           return_lse=False, p_dtype=torch.float16, p_gain=1.0, sum_rounded=True, v_mean=None):
    """Flash-style forward on pre-quantised Q/K, in the reference's operation order:
    per BLKK-key block  S -> scale -> running max (base 2) -> P = 2^(S*a - m) -> P16 ->
    d += rowsum(P16) -> O = O*alpha + P16 @ V16, then O * (1/d).  ``pv_accum_dtype``:
    "fp32" keeps O in fp32; "fp16+fp32" rounds each block's P16@V16 to fp16 before the
    fp32 add (attn_utils.cuh:447-518); "fp16" keeps O itself in fp16 and rescales it
    with alpha rounded to fp16 (attn_utils.cuh:313-336).  Returns O in the input layout
    (and the base-2 LSE = log2(d) + m as (B,Hq,Nq) when asked).  ``v_mean`` ((B,Hkv,D), fp16
    accumulate only): the channel mean of a smoothed V, added to the output after its rounding to
    the output type (qk_int8_sv_f16_kernel_sm80.cuh:551-569)."""
    q8 = to_bhnd(q_int8, tensor_layout).float()
    k8 = to_bhnd(k_int8, tensor_layout).float()
    v = to_bhnd(v16, tensor_layout).float()
    B, Hq, Nq, D = q8.shape
    Hkv, Nk = k8.shape[1], k8.shape[2]
    grp = Hq // Hkv
    if sm_scale is None:
        sm_scale = D ** -0.5
    qs = expand_q_scale(q_scale, Nq, BLKQ, WARPQ, granularity)          # (B,Hq,Nq)
    ks = expand_k_scale(k_scale, Nk, BLKK, WARPK, granularity)          # (B,Hkv,Nk)
    if grp > 1:
        k8 = k8.repeat_interleave(grp, dim=1)
        v = v.repeat_interleave(grp, dim=1)
        ks = ks.repeat_interleave(grp, dim=1)
    c = np.float32(sm_scale * LOG2_E)

    o = torch.zeros(B, Hq, Nq, D, dtype=torch.float32)
    lse = torch.empty(B, Hq, Nq, dtype=torch.float32)
    rows = torch.arange(Nq)
    for q0 in range(0, Nq, BLKQ):
        q1 = min(q0 + BLKQ, Nq)
        # keys a causal Q tile visits: qk_int8_sv_f16_kernel_sm80.cuh:210-214
        kv_end = min(Nk, q0 + BLKQ) if is_causal else Nk
        qt = q8[:, :, q0:q1]
        qst = qs[:, :, q0:q1, None]
        m = torch.full((B, Hq, q1 - q0), _NEG_BIG, dtype=torch.float32)
        d = torch.ones(B, Hq, q1 - q0, dtype=torch.float32)
        acc = torch.zeros(B, Hq, q1 - q0, D, dtype=torch.float32)
        if pv_accum_dtype == "fp16":
            acc = acc.half()
        for k0 in range(0, kv_end, BLKK):
            k1 = min(k0 + BLKK, Nk)
            s = torch.matmul(qt, k8[:, :, k0:k1].transpose(2, 3))       # exact in fp32
            a = (qst * ks[:, :, None, k0:k1]) * c                        # (B,H,q,k)
            s = s * a
            if is_causal:
                vis = rows[q0:q1, None] >= torch.arange(k0, k1)[None, :]
                s = torch.where(vis, s, torch.full_like(s, _NEG_BIG))
            m_new = torch.maximum(m, s.max(dim=-1).values)
            alpha = torch.exp2(m - m_new)
            p = torch.exp2(s - m_new[..., None])
            p16 = (p * p_gain).to(p_dtype).float() / p_gain
            d = d * alpha + (p16 if sum_rounded else p).sum(dim=-1)
            pv = torch.matmul(p16, v[:, :, k0:k1])
            if pv_accum_dtype == "fp32":
                acc = acc * alpha[..., None] + pv
            elif pv_accum_dtype == "fp16+fp32":
                acc = acc * alpha[..., None] + pv.half().float()
            elif pv_accum_dtype == "fp16":
                acc = (acc * alpha.half()[..., None]).float()
                acc = (acc + pv).half()
            else:
                raise ValueError("pv_accum_dtype must be 'fp32', 'fp16', or 'fp16+fp32'.")
            m = m_new
        o[:, :, q0:q1] = acc.float() / d[..., None]
        lse[:, :, q0:q1] = torch.log2(d) + m
    if pv_accum_dtype == "fp16":
        o = o.half().float()                 # normalize_d leaves a half accumulator (attn_utils.cuh:565-567)
    o = o.to(out_dtype)
    if v_mean is not None:
        if pv_accum_dtype != "fp16":
            raise ValueError("v_mean goes with pv_accum_dtype='fp16' only.")
        vm = v_mean.to(out_dtype)
        if grp > 1:
            vm = vm.repeat_interleave(grp, dim=1)
        o = (o.float() + vm[:, :, None, :].float()).to(out_dtype)      # __hadd2 in the output type
    out = from_bhnd(o, tensor_layout).contiguous()
    if return_lse:
        return out, lse
    return out


def smooth_v(v, tensor_layout="HND"):
    """(smoothed_v fp16, vm): vm = v.mean over the sequence in v's dtype, smoothed = (v - vm) in
    v's dtype, then .to(float16) (cuda_attn.py:209-211)."""
    seq_dim = 2 if tensor_layout == "HND" else 1
    vm = v.float().mean(dim=seq_dim).to(v.dtype)
    sm = (v - vm.unsqueeze(seq_dim)).to(torch.float16)
    return sm, vm


def quant_v_fp8(v, tensor_layout="HND"):
    """V in fp8 e4m3 with one scale per (batch, head, channel): scale = max(max|v|, 1e-8) * (1/448),
    v_q = e4m3(v / scale).  No counterpart in the reference tree (its fp8 kernels live on an
    un-vendored branch); this follows the published SageAttention2 scheme and is parity-unpinned."""
    vb = to_bhnd(v, tensor_layout).float()
    amax = vb.abs().amax(dim=2)                                        # (B,H,D)
    scale = (torch.clamp(amax, min=1e-8).numpy().astype(np.float32) * np.float32(1.0 / 448.0)).astype(np.float32)
    scale = torch.from_numpy(scale)
    vq = (vb / scale[:, :, None, :]).to(torch.float8_e4m3fn)
    return from_bhnd(vq, tensor_layout).contiguous(), scale


def attend_fp8(q_int8, k_int8, v_fp8, v_scale, q_scale, k_scale, tensor_layout="HND", is_causal=False,
               sm_scale=None, granularity="per_thread", BLKQ=128, WARPQ=32, BLKK=64, WARPK=64,
               out_dtype=torch.float16, return_lse=False):
    """attend() with e4m3 P.V: P is scaled by 448 and rounded to e4m3 before the product (the factor
    cancels against the row sum, which adds the unrounded values), V carries its per-channel scale."""
    v_deq = to_bhnd(v_fp8, tensor_layout).float() * v_scale[:, :, None, :]
    # reuse attend(): 448 * P rounded to e4m3 == 448 * (P rounded to e4m3 with the exponent shifted)
    res = attend(q_int8, k_int8, from_bhnd(v_deq, tensor_layout), q_scale, k_scale, tensor_layout, is_causal,
                 sm_scale, "fp32", granularity, BLKQ, WARPQ, BLKK, WARPK, out_dtype, return_lse,
                 p_dtype=torch.float8_e4m3fn, p_gain=448.0, sum_rounded=False)
    return res


def lse_correction(q, km, tensor_layout):
    """q . km^T with GQA broadcast (sageattention/utils.py:39-49), fp32 result."""
    qb = to_bhnd(q, tensor_layout)
    kmb = to_bhnd(km, tensor_layout)
    grp = qb.shape[1] // kmb.shape[1]
    if grp > 1:
        kmb = kmb.repeat_interleave(grp, dim=1)
    return torch.matmul(qb.float(), kmb.float().transpose(2, 3)).squeeze(-1)


def sageattn(q, k, v, tensor_layout="HND", is_causal=False, pv_accum_dtype="fp32",
             smooth_k=True, return_lse=False, sm_scale=None, granularity="per_thread",
             qk_config=(128, 64, 32, 64), smooth_v=False):
    """The whole front end (cuda_attn.py:126-274) on CPU tensors: pad D, K mean, quantise,
    attend, slice, LSE fix-up."""
    head_dim = q.size(-1)
    pad_to = padded_head_dim(head_dim)
    if pad_to != head_dim:
        pad = (0, pad_to - head_dim)
        q, k, v = (torch.nn.functional.pad(t, pad) for t in (q, k, v))
    if sm_scale is None:
        sm_scale = head_dim ** -0.5
    blk_q, blk_k, warp_q, warp_k = qk_config
    km = mean_k(k, tensor_layout) if smooth_k else None
    if granularity == "per_thread":
        q8, qs, k8, ks = quant_per_thread(q, k, km, blk_q, warp_q, blk_k, warp_k, tensor_layout)
    else:
        q8, qs, k8, ks = quant_per_block(q, k, km, blk_q, blk_k, tensor_layout)
    v16, vm = v.to(torch.float16), None
    if smooth_v and pv_accum_dtype == "fp16":
        v16, vm = globals()["smooth_v"](v, tensor_layout)
    res = attend(q8, k8, v16, qs, ks, tensor_layout, is_causal, sm_scale,
                 pv_accum_dtype, granularity, blk_q, warp_q, blk_k, warp_k, q.dtype, return_lse, v_mean=vm)
    if not return_lse:
        return res[..., :head_dim]
    out, lse = res
    lse = lse / LOG2_E
    if smooth_k:
        lse = lse + lse_correction(q, km, tensor_layout) * sm_scale
    return out[..., :head_dim], lse


def sdpa_fp32(q, k, v, tensor_layout="HND", is_causal=False, sm_scale=None):
    """Unquantised fp32 attention, for sanity bounds (tests/test_sageattn.py:40-49 uses
    SDPA-math the same way)."""
    qb, kb, vb = (to_bhnd(t, tensor_layout).float() for t in (q, k, v))
    grp = qb.shape[1] // kb.shape[1]
    if grp > 1:
        kb = kb.repeat_interleave(grp, dim=1)
        vb = vb.repeat_interleave(grp, dim=1)
    if sm_scale is None:
        sm_scale = q.size(-1) ** -0.5
    s = torch.matmul(qb, kb.transpose(2, 3)) * sm_scale
    if is_causal:
        nq, nk = s.shape[-2:]
        vis = torch.arange(nq)[:, None] >= torch.arange(nk)[None, :]
        s = s.masked_fill(~vis, float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.matmul(torch.softmax(s, dim=-1), vb)
    return from_bhnd(o, tensor_layout).contiguous(), lse


def compare(a: torch.Tensor, b: torch.Tensor) -> dict:
    """Cosine similarity, max-abs and Frobenius-relative error in fp32."""
    a = a.float().flatten()
    b = b.float().flatten()
    diff = (a - b)
    return {
        "cos": float(torch.dot(a, b) / (a.norm() * b.norm() + 1e-30)),
        "max_abs": float(diff.abs().max()) if diff.numel() else 0.0,
        "fro_rel": float(diff.norm() / (b.norm() + 1e-30)),
    }
