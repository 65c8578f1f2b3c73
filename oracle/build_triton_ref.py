"""Compiles the reference's Triton quantisers to sm_100a cubins.  TEST INFRASTRUCTURE.

The reference's quantisation kernels are Triton source
(sageattention/triton/quant_per_thread.py, quant_per_block.py).  The Python
package cannot travel to a GPU machine that has no reference checkout, but
Triton can compile those kernels ahead of time without a GPU.  This script
compiles them *where they lie* and writes, into ``oracle/_ref/``:

    triton_quant/<key>.cubin      one per specialisation
    triton_quant/manifest.json    kernel name, shared memory, warps, signature

``oracle/triton_ref.py`` loads those with the CUDA driver API and launches them
with the grids of the reference's host wrappers, which gives the GPU parity
tests the reference's real device arithmetic (``div.full.f32``, ``cvt.rzi``)
to compare with bit for bit.

Usage: python oracle/build_triton_ref.py [--ref /path/to/reference]
"""
from __future__ import annotations

import argparse
import importlib.util
import json
import os

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref", "triton_quant")


def _load(path: str, name: str):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("SAGE_REFERENCE_DIR"), required="SAGE_REFERENCE_DIR" not in os.environ,
                    help="checkout of woct0rdho/sageattention-autotune (or set SAGE_REFERENCE_DIR)")
    args = ap.parse_args()
    os.environ.pop("TRITON_INTERPRET", None)

    import sys
    sys.path.insert(0, args.ref)          # quant_per_block imports ..autotune_utils
    import triton
    from triton.backends.compiler import GPUTarget
    from triton.compiler import ASTSource

    qpt = importlib.import_module("sageattention.triton.quant_per_thread")
    qpb = importlib.import_module("sageattention.triton.quant_per_block")
    target = GPUTarget("cuda", 100, 32)
    os.makedirs(OUT, exist_ok=True)
    manifest = {}

    def emit(key, fn, sig, constexprs):
        full = dict(sig)
        for c in constexprs:
            full[c] = "constexpr"
        src = ASTSource(fn=fn, signature=full, constexprs=constexprs)
        cc = triton.compile(src, target=target, options={"num_warps": 4})
        with open(os.path.join(OUT, key + ".cubin"), "wb") as f:
            f.write(cc.asm["cubin"])
        manifest[key] = dict(name=cc.metadata.name, shared=cc.metadata.shared,
                             num_warps=cc.metadata.num_warps, args=list(sig.keys()),
                             global_scratch=cc.metadata.global_scratch_size,
                             profile_scratch=cc.metadata.profile_scratch_size)
        print("built", key)

    i32 = "i32"
    for dt, tname in (("fp16", "f16"), ("bf16", "bf16")):
        for C in (64, 128):
            for blk in (32, 16):
                sig = {"Input": "*" + dt, "Output": "*i8", "Scale": "*fp32", "L": i32,
                       "stride_iz": i32, "stride_ih": i32, "stride_in": i32,
                       "stride_oz": i32, "stride_oh": i32, "stride_on": i32,
                       "stride_sz": i32, "stride_sh": i32}
                emit(f"q_thread_{tname}_c{C}_blk{blk}", qpt.quant_query_per_thread_int8_kernel,
                     sig, {"C": C, "BLK": blk})
            ksig = {"Input": "*" + dt, "Mean": "*" + dt, "Output": "*i8", "Scale": "*fp32", "L": i32,
                    "stride_iz": i32, "stride_ih": i32, "stride_in": i32,
                    "stride_mz": i32, "stride_mh": i32, "stride_mk": i32,
                    "stride_oz": i32, "stride_oh": i32, "stride_on": i32,
                    "stride_sz": i32, "stride_sh": i32}
            for blk in (64, 32):
                for has_mean in (0, 1):
                    emit(f"k_thread_{tname}_c{C}_blk{blk}_m{has_mean}",
                         qpt.quant_key_per_thread_int8_kernel, ksig,
                         {"C": C, "BLK": blk, "HAS_MEAN": bool(has_mean)})
            bsig = {"Input": "*" + dt, "Mean": "*" + dt, "Output": "*i8", "Scale": "*fp32", "L": i32,
                    "L_BUCKET": i32,
                    "stride_iz": i32, "stride_ih": i32, "stride_in": i32,
                    "stride_mz": i32, "stride_mh": i32, "stride_mk": i32,
                    "stride_oz": i32, "stride_oh": i32, "stride_on": i32,
                    "stride_sz": i32, "stride_sh": i32}
            for blk in (128, 64):
                for has_mean in (0, 1):
                    emit(f"block_{tname}_c{C}_blk{blk}_m{has_mean}",
                         qpb.quant_per_block_int8_kernel.fn, bsig,
                         {"C": C, "BLK": blk, "HAS_MEAN": bool(has_mean)})

    with open(os.path.join(OUT, "manifest.json"), "w") as f:
        json.dump(manifest, f, indent=1)
    print("wrote", len(manifest), "kernels to", OUT)


if __name__ == "__main__":
    main()
