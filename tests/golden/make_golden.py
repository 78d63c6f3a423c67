"""Generates the golden fixtures in this folder from the reference's own helpers.

Runs only where a checkout of the reference is at hand (``REFERENCE_ROOT`` names it); the
tests read the committed ``.npz`` files and never the reference. Modules are loaded by file path because the example package's
``__init__`` needs a full TileLang build:
  examples/dequantize_gemm/dequantize_utils.py  (torch_convert, torch_convert_bit_twiddling)
  examples/dequantize_gemm/quantize/utils.py    (general_compress, interleave_weight, gen_quant4)
  examples/dequantize_gemm/quantize/nvfp4.py    (e2m1 encode / pack / decode, UE4M3 codec, scale
                                                 swizzle, quantize_bf16_to_nvfp4_blockscaled)
  examples/deepseek_v4/act_quant.py             (fp4_act_quant_ref, the bf16 -> MXFP4 quantiser)
  examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py (quantize_mxfp4_with_packed_ue8m0, group-major words)

    REFERENCE_ROOT=<reference checkout> python tests/golden/make_golden.py
"""
import importlib.util
import os
import sys

import numpy as np
import torch

REF = os.environ.get("REFERENCE_ROOT")
if not REF or not os.path.isdir(REF):
    sys.exit("set REFERENCE_ROOT to a checkout of the reference")
HERE = os.path.dirname(os.path.abspath(__file__))


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def main():
    du = load("ref_dequantize_utils", "examples/dequantize_gemm/dequantize_utils.py")
    qu = load("ref_quantize_utils", "examples/dequantize_gemm/quantize/utils.py")
    nv = load("ref_nvfp4", "examples/dequantize_gemm/quantize/nvfp4.py")
    g = torch.Generator().manual_seed(1234)

    # --- integer codecs -----------------------------------------------------
    codes4 = torch.randint(0, 16, (6, 64), generator=g, dtype=torch.int8)
    codes2 = torch.randint(0, 4, (6, 64), generator=g, dtype=torch.int8)
    raw = torch.randint(-128, 128, (8, 32), generator=g, dtype=torch.int8)
    out = {
        "codes4": codes4.numpy(), "codes2": codes2.numpy(), "raw": raw.numpy(),
        "compress4": qu.general_compress(codes4.clone(), 4).numpy(),
        "compress2": qu.general_compress(codes2.clone(), 2).numpy(),
        # the cases of interleave_weight the reference's torch version can execute
        "interleave_4_float16": qu.interleave_weight(raw.clone(), 4, "float16").numpy(),
        "interleave_4_int8": qu.interleave_weight(raw.clone(), 4, "int8").numpy(),
        "interleave_2_int8": qu.interleave_weight(raw.clone(), 2, "int8").numpy(),
    }
    np.savez_compressed(os.path.join(HERE, "codecs.npz"), **out)

    # --- gen_quant4: symmetric group quantiser, ref = (q - 8) * s ------------
    torch.manual_seed(7)
    w, linear, s, q_minus_8 = qu.gen_quant4(128, 16, groupsize=64)
    np.savez_compressed(os.path.join(HERE, "gen_quant4.npz"), w=w.float().numpy(), s=s.float().numpy(),
                        q_minus_8=q_minus_8.numpy(), ref_kn=linear.weight.data.t().float().numpy())

    # --- fp4 decoders ---------------------------------------------------------
    qb = torch.randint(0, 256, (5, 64), generator=g, dtype=torch.uint8)
    scale = torch.randint(0, 5, (5, 4), generator=g, dtype=torch.uint8)
    allb = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    np.savez_compressed(
        os.path.join(HERE, "fp4_decode.npz"), qb=qb.numpy(), scale=scale.numpy(),
        simple=du.torch_convert(qb).view(torch.int16).numpy(),
        simple_scaled=du.torch_convert(qb, 32, scale).view(torch.int16).numpy(),
        twiddled=du.torch_convert_bit_twiddling(qb).view(torch.int16).numpy(),
        simple_all=du.torch_convert(allb).view(torch.int16).numpy(),
        twiddled_all=du.torch_convert_bit_twiddling(allb).view(torch.int16).numpy())

    # --- e2m1 encode / pack / decode -----------------------------------------
    vals = (torch.randn((4, 64), generator=g) * 2.5)
    vals[0, :16] = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.0, -1.5, -2.0, -3.0, -4.0, -6.0, 0.0])
    vals[1, :8] = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, -0.25])   # exactly on the thresholds
    codes = nv.encode_fp4_e2m1_values(vals)
    packed = nv.pack_fp4_e2m1_codes(codes)
    np.savez_compressed(os.path.join(HERE, "e2m1.npz"), vals=vals.numpy(), codes=codes.numpy(),
                        packed=packed.numpy(), decoded=nv.decode_packed_fp4_e2m1(packed).numpy(),
                        lut=np.array(nv._FP4_E2M1_VALUES, dtype=np.float32))
    # --- block-scale formats: UE4M3 codec, scale swizzle, NVFP4 and MXFP4 quantisers ---------
    aq = load("ref_act_quant", "examples/deepseek_v4/act_quant.py")
    fg = load("ref_fp8_fp4_gemm", "examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py")
    allbytes = torch.arange(256, dtype=torch.uint8)
    sweep = torch.cat((torch.linspace(0, 0.05, 400), torch.linspace(0.05, 500, 600),
                       torch.tensor([2.0 ** -9, 2.0 ** -6, 448.0, 1e9, float("nan"), -1.0])))
    words = torch.randint(0, 2 ** 31, (256, 8), generator=g, dtype=torch.int64).to(torch.uint32)
    xa = torch.randn((128, 256), generator=g).to(torch.bfloat16) * 3
    xa[5, :16] = 0                                                      # an all-zero scale block
    nv_packed, nv_words, nv_bytes = nv.quantize_bf16_to_nvfp4_blockscaled(xa, return_scale_bytes=True)
    xm = (torch.randn((16, 256), generator=g) * torch.logspace(-3, 2, 16).unsqueeze(1)).to(torch.bfloat16)
    q32, s32 = aq.fp4_act_quant_ref(xm, 32)
    q128, w128, sf128 = fg.quantize_mxfp4_with_packed_ue8m0(xm.float(), 128)
    np.savez_compressed(
        os.path.join(HERE, "blockscale.npz"),
        ue4m3_decode_all=nv.decode_ue4m3_scale_bytes(allbytes).numpy(), sweep=sweep.numpy(),
        ue4m3_nearest=nv.encode_ue4m3_scale_bytes(sweep).numpy(),
        ue4m3_ceil=nv.encode_ue4m3_scale_bytes(sweep, rounding="ceil").numpy(),
        ue4m3_ceil_minpos=nv.encode_ue4m3_scale_bytes(sweep, rounding="ceil", min_positive=True).numpy(),
        words=words.view(torch.int32).numpy(),
        swizzled=nv.swizzle_blockscaled_chunk_kmajor_scale_words(words).view(torch.int32).numpy(),
        xa=xa.view(torch.int16).numpy(), nv_packed=nv_packed.numpy(), nv_words=nv_words.view(torch.int32).numpy(),
        nv_bytes=nv_bytes.numpy(),
        xm=xm.view(torch.int16).numpy(), mx32_packed=q32.view(torch.uint8).numpy(), mx32_scale=s32.numpy(),
        mx128_packed=q128.view(torch.uint8).numpy(), mx128_words=w128.view(torch.int32).numpy(), mx128_sf=sf128.numpy())
    print("wrote", sorted(f for f in os.listdir(HERE) if f.endswith(".npz")))


if __name__ == "__main__":
    sys.exit(main())
