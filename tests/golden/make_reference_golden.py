"""Produce tests/golden/reference_*.npz by running the REFERENCE implementation on a Blackwell GPU.

The reference's quantizers (kernels/kernel_ScaleSweep_MSE.py, kernels/kernel_ScaleSweep.py of
efsotr/nvfp4quant_test) are Triton kernels with Blackwell-only inline PTX and cannot run on a
CPU; vllm's scaled_fp4_quant / cutlass_scaled_fp4_mm are compiled CUDA.  So the fixtures are
captured once on a B200 from an unmodified checkout of the reference and committed; the tests
then compare both the CPU oracle and the CUDA kernels of this repository with them.

  python tests/golden/make_reference_golden.py --reference /path/to/nvfp4quant_test --out tests/golden

Needs: torch + triton + vllm (for create_fp4_output_tensors and the two vllm ops) and an
sm_100 GPU.  Inputs are defined in tests/golden/cases.py (CPU generator, seeded).
"""
from __future__ import annotations

import argparse
import json
import pathlib
import sys
import traceback

import numpy as np
import torch

HERE = pathlib.Path(__file__).resolve().parent
sys.path.insert(0, str(HERE))
import cases as C  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, type=pathlib.Path)
    ap.add_argument("--out", default=HERE, type=pathlib.Path)
    args = ap.parse_args()
    sys.path.insert(0, str(args.reference))
    args.out.mkdir(parents=True, exist_ok=True)
    dev = torch.device("cuda")

    import helper as ref_helper  # reference helper.py
    from kernels.kernel_ScaleSweep import scalesweep_weighted_mse_nvfp4_quant_impl
    from kernels.kernel_ScaleSweep_MSE import scalesweep_mse_nvfp4_quant_impl

    try:
        from vllm._custom_ops import cutlass_scaled_fp4_mm, scaled_fp4_quant
        have_vllm_ops = hasattr(torch.ops, "_C") and hasattr(torch.ops._C, "scaled_fp4_quant")
    except Exception:  # noqa: BLE001
        traceback.print_exc()
        have_vllm_ops = False
    print("vllm compiled ops available:", have_vllm_ops)

    meta = {"torch": torch.__version__, "gpu": torch.cuda.get_device_name(0), "cases": {}, "gemm": {},
            "vllm_ops": have_vllm_ops}
    arrays = {}
    for name, c in C.build_cases().items():
        x = c["x"].to(dev)
        if c["gs_inv"] is None:
            gs, gs_inv = ref_helper.get_nvfp4_global_scale(x, FP8_MAX=c["fp8_max"])
        else:
            gs_inv = torch.tensor(c["gs_inv"], dtype=torch.float32, device=dev)
            gs = gs_inv.reciprocal()
        try:
            if c["variant"] == "mse":
                codes, scales = scalesweep_mse_nvfp4_quant_impl(x, gs_inv, c["swizzled"], c["padded_n"])
            elif c["variant"] == "weighted":
                kw = {}
                if c["lower"] is not None:
                    kw = dict(lower_bound=c["lower"], upper_bound=c["upper"])
                codes, scales = scalesweep_weighted_mse_nvfp4_quant_impl(
                    x, c["importance"].to(dev), gs_inv, c["swizzled"], c["padded_n"], **kw)
            else:
                if not have_vllm_ops:
                    print("skip", name)
                    continue
                codes, scales = scaled_fp4_quant(x, gs_inv, c["swizzled"], padded_n=c["padded_n"])
        except Exception:  # noqa: BLE001
            traceback.print_exc()
            continue
        torch.cuda.synchronize()
        arrays[name + ".codes"] = codes.cpu().numpy()
        arrays[name + ".scales"] = scales.view(torch.uint8).cpu().numpy()
        meta["cases"][name] = {
            "x_sha256": C.sha(c["x"]), "gs": float(gs.item()), "gs_inv": float(gs_inv.item()),
            "gs_inv_bits": int(gs_inv.view(torch.int32).item()), "gs_bits": int(gs.view(torch.int32).item()),
            "shape": list(c["x"].shape), "variant": c["variant"],
        }
        print("ok", name, tuple(codes.shape), tuple(scales.shape))

    if have_vllm_ops:
        for name, (M, N, K, seed) in C.gemm_cases().items():
            a, b = C.gemm_operands(M, N, K, seed)
            a, b = a.to(dev), b.to(dev)
            imp_a = (b.float() ** 2).sum(0, keepdim=True)
            imp_b = (a.float() ** 2).sum(0, keepdim=True)
            gsa, gsa_inv = ref_helper.get_nvfp4_global_scale(a, FP8_MAX=256.0)
            gsb, gsb_inv = ref_helper.get_nvfp4_global_scale(b, FP8_MAX=256.0)
            try:
                qa, sa = scalesweep_weighted_mse_nvfp4_quant_impl(a, imp_a, gsa_inv, True)
                qb, sb = scalesweep_weighted_mse_nvfp4_quant_impl(b, imp_b, gsb_inv, True)
                # the reference leaves scale padding uninitialised; zero it so the fixture is reproducible
                alpha = (gsa * gsb).reshape(1).float()
                out = cutlass_scaled_fp4_mm(qa, qb, sa, sb, alpha, torch.bfloat16)
                torch.cuda.synchronize()
            except Exception:  # noqa: BLE001
                traceback.print_exc()
                continue
            arrays[name + ".qa"] = qa.cpu().numpy()
            arrays[name + ".qb"] = qb.cpu().numpy()
            arrays[name + ".sa"] = sa.view(torch.uint8).cpu().numpy()
            arrays[name + ".sb"] = sb.view(torch.uint8).cpu().numpy()
            arrays[name + ".out_bf16_bits"] = out.view(torch.int16).cpu().numpy()
            meta["gemm"][name] = {"M": M, "N": N, "K": K, "alpha": float(alpha.item()),
                                  "alpha_bits": int(alpha.view(torch.int32).item())}
            print("ok", name, tuple(out.shape))

    np.savez_compressed(args.out / "reference_golden.npz", **arrays)
    (args.out / "reference_golden.json").write_text(json.dumps(meta, indent=1) + "\n")
    print("wrote", args.out / "reference_golden.npz")


if __name__ == "__main__":
    main()
