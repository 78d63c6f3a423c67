"""CPU: the C-ABI library loads and exports every symbol ``include/b200dq.h``
declares; host-side helpers and argument checks that need no GPU."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

import tilelang_b200
from tilelang_b200 import _lib, kernels, quantize
from oracle import ref_programs as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200dq.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200dq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    syms = declared_symbols()
    assert syms, "header declares no entry points?"
    for s in syms:
        assert hasattr(lib, s), f"{s} declared in include/b200dq.h but not exported"
    assert set(_lib.EXPORTED_SYMBOLS) <= set(syms)
    assert lib.b200dq_version() >= 1


def test_size_queries_need_no_gpu():
    lib = _lib.load()
    # 28672 x 8192 uint4, group 128: 224 tiles x 64 stages x (8192 + 512) bytes
    assert lib.b200dq_packed_weight_bytes(28672, 8192, 128, _lib.WF_U4_SZ) == 224 * 64 * 8704
    assert lib.b200dq_packed_weight_bytes(3200, 8640, 0, _lib.WF_I2_I8) == 25 * 34 * 8192
    assert lib.b200dq_gemm_workspace_bytes(16, 28672, 8192, _lib.WF_U4_SZ, _lib.ACT_BF16, 0, 0) > 0
    assert lib.b200dq_gemm_workspace_bytes(0, 1, 1, 0, 0, 0, 0) == 0


def test_gemm_args_struct_matches_header_field_order():
    text = open(os.path.join(ROOT, "include", "b200dq.h")).read()
    body = text[text.index("typedef struct b200dq_gemm_args {"):text.index("} b200dq_gemm_args;")]
    body = re.sub(r"/\*.*?\*/", "", body, flags=re.S)
    names = []
    for decl in body.split("{", 1)[1].split(";"):
        decl = decl.strip()
        if not decl:
            continue
        parts = [p.strip().lstrip("*") for p in decl.split(",")]
        names.append(re.sub(r"\[\d+\]$", "", parts[0].split()[-1].lstrip("*")))     # array fields: name[7]
        names.extend(parts[1:])
    assert names == [f[0] for f in _lib.GemmArgs._fields_]


def test_errors_are_reported_not_thrown():
    lib = _lib.load()
    assert lib.b200dq_gemm(None, None) == -1
    assert "null" in _lib.last_error()
    args = _lib.GemmArgs(M=-1, N=4, K=4)
    assert lib.b200dq_gemm(ctypes.byref(args), None) == -1


def test_codecs_match_oracle():
    torch.manual_seed(1)
    codes = torch.randint(0, 16, (4, 64), dtype=torch.uint8)
    assert np.array_equal(quantize.compress_codes(codes, 4).numpy(), R.general_compress(codes.numpy(), 4))
    assert torch.equal(quantize.decompress_codes(quantize.compress_codes(codes, 4), 4), codes)
    raw = torch.randint(-128, 128, (4, 32), dtype=torch.int8)
    for nb, tgt in [(4, "float16"), (4, "int8"), (2, "int8"), (2, "float16"), (1, "int8"), (1, "float16")]:
        inter = quantize.interleave_weight(raw, nb, tgt)
        assert np.array_equal(inter.numpy(), R.interleave_weight(raw.numpy(), nb, tgt))
        assert torch.equal(quantize.deinterleave_weight(inter, nb, tgt), raw)


def test_untwiddle_fp4_gives_natural_order():
    qb = torch.randint(0, 256, (3, 32), dtype=torch.uint8)
    assert torch.equal(R.decode_fp4_e2m1(quantize.untwiddle_fp4(qb)), R.decode_fp4_twiddled(qb).float())


def test_factory_signatures_and_checks():
    k = tilelang_b200.matmul(16, 1024, 1024, "float16", "float16", "float32", num_bits=4, group_size=128)
    assert [p.name for p in k.params] == ["A", "B", "Scale", "C"] and k.out_idx == [-1]
    assert k.params[1].shape == (1024, 512) and k.params[2].shape == (1024, 8)
    with pytest.raises(ValueError):
        k(torch.zeros(16, 1024, dtype=torch.float16))          # wrong input count (tvm_ffi.py:244-246)
    kz = tilelang_b200.matmul(4, 256, 256, "bfloat16", "bfloat16", "float32", group_size=128, with_zeros=True)
    assert [p.name for p in kz.params] == ["A", "B", "Scale", "Zeros", "C"]
    kf = tilelang_b200.matmul(4, 256, 256, "bfloat16", "bfloat16", "float32", source_format="fp4", with_bias=True)
    assert [p.name for p in kf.params] == ["A", "B", "Scale", "Bias", "C"] and kf.params[2].dtype == torch.uint8
    ki = tilelang_b200.matmul(4, 256, 256, "int8", "int32", "int32")      # fine_grained.py:427-428
    assert [p.name for p in ki.params] == ["A", "B", "C"] and ki.params[2].dtype == torch.int32
    with pytest.raises(ValueError):
        tilelang_b200.matmul(4, 256, 256, "int8", "float16", "int32")
    kq = tilelang_b200.matmul(4, 256, 256, "float16", "float16", "float32", group_size=128, with_zeros=True,
                              zeros_mode="quantized")
    assert kq.params[3].name == "Zeros" and kq.params[3].dtype == torch.uint8
    with pytest.raises(ValueError):
        tilelang_b200.matmul(4, 256, 256, "float16", "float16", "float32", group_size=128, zeros_mode="other")
    gv = tilelang_b200.dequantize_gemv(1, 1024, 1024, "float16", "float16", "float16", 4, "int8", "uint", 4, 32, True)
    assert gv.out_idx is None and len(gv.params) == 3
    w8 = tilelang_b200.matmul_int8xint4(128, 256, 256, "int8", "int32", "int32")
    assert w8.params[2].shape == (256, 128)


def test_no_cpu_fallback():
    k = tilelang_b200.matmul(4, 256, 256, "float16", "float16", "float32", group_size=128)
    A = torch.zeros(4, 256, dtype=torch.float16)
    qB = torch.zeros(256, 128, dtype=torch.uint8)
    S = torch.ones(256, 2, dtype=torch.float16)
    with pytest.raises((ValueError, RuntimeError)):
        k(A, qB, S)


def test_product_does_not_import_oracle():
    pkg = os.path.join(ROOT, "tilelang_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle", src, flags=re.M), f"{f} imports the oracle"
                assert "oracle/" not in src and "oracle." not in src, f"{f} refers to the oracle"


def test_packed_weight_cache_is_keyed_by_tensor_identity_and_version():
    """A freed weight's address can be handed to the next tensor of the same shape (version 0
    again): the cache must repack for a different tensor object and after an in-place write."""
    calls = []

    def pack_fn(q):
        calls.append(q)
        return ("packed", len(calls))

    k = kernels.DequantKernel("t", [], None, None, pack_fn)
    a = torch.zeros(4, 8, dtype=torch.uint8)
    assert k._packed(a) == ("packed", 1) and k._packed(a) == ("packed", 1)
    b = torch.zeros(4, 8, dtype=torch.uint8)            # same shape, same version, another object
    assert k._packed(b) == ("packed", 2)
    assert k._packed(a) == ("packed", 1)                # still cached, source kept alive by the entry
    a.add_(1)                                           # in-place write bumps the version
    assert k._packed(a) == ("packed", 3)


def test_zero_point_modes_map_to_the_original_rule():
    from tilelang_b200 import ops
    s = (torch.rand(8, 4) * 0.015 + 0.005).to(torch.bfloat16)
    z = (torch.rand(8, 4) * 0.1 + 0.05).to(torch.bfloat16)
    assert ops.zeros_for_original_mode(s, z, "original") is z
    zr = ops.zeros_for_original_mode(s, z, "rescale")
    assert zr.dtype == torch.bfloat16 and torch.equal(zr, (z.float() / s.float()).to(torch.bfloat16))
    zq = ops.zeros_for_original_mode(s, torch.randint(0, 16, (8, 4), dtype=torch.int32), "quantized")
    assert zq.dtype == torch.bfloat16 and torch.equal(zq.float(), zq.float().round())
    with pytest.raises(ValueError):
        ops.zeros_for_original_mode(s, z, "other")


def _pack_fields(vals, bits, order=None):
    """(..., F) integer fields -> (..., F * bits / 32) int32 words, field f of a word at bit
    bits * order[f % per] (written with plain loops: the thing the adapters must undo)."""
    per = 32 // bits
    order = list(range(per)) if order is None else order
    v = vals.to(torch.int64)
    words = torch.zeros(*v.shape[:-1], v.shape[-1] // per, dtype=torch.int64)
    for f in range(v.shape[-1]):
        words[..., f // per] |= (v[..., f] & ((1 << bits) - 1)) << (bits * order[f % per])
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words)
    return words.to(torch.int32)


def test_gptq_and_awq_adapters_recover_codes_scales_and_zero_points():
    g = torch.Generator().manual_seed(5)
    K, N, group = 256, 64, 128
    q = torch.randint(0, 16, (K, N), generator=g)                       # (in, out) as the checkpoints store it
    z = torch.randint(1, 16, (K // group, N), generator=g)
    s = (torch.rand(K // group, N, generator=g) * 0.015 + 0.005).to(torch.float16)
    want_qB = torch.from_numpy(R.general_compress(q.t().contiguous().numpy().astype(np.uint8), 4))
    # AutoGPTQ: codes packed along K, zero-points along N, stored minus one
    qweight = _pack_fields(q.t().contiguous(), 4).t().contiguous()      # (K/8, N)
    qzeros = _pack_fields(z - 1, 4)                                     # (groups, N/8)
    qB, s_nk, z_nk = quantize.from_gptq(qweight, s, qzeros)
    assert torch.equal(qB, want_qB) and torch.equal(s_nk, s.t()) and torch.equal(z_nk.long(), z.t())
    # AutoAWQ GEMM: both packed along N in the order 0, 2, 4, 6, 1, 3, 5, 7
    inv = [0, 4, 1, 5, 2, 6, 3, 7]
    qB, s_nk, z_nk = quantize.from_awq(_pack_fields(q, 4, inv), s, _pack_fields(z, 4, inv))
    assert torch.equal(qB, want_qB) and torch.equal(s_nk, s.t()) and torch.equal(z_nk.long(), z.t())
    # and the weight they stand for, by the oracle's "quantized" rule
    W = R.dequant_w4_group(qB, s_nk, z_nk, group, torch.float16, "quantized")
    want = ((q.t().float() - z.t().repeat_interleave(group, 1).float()) * s.t().float().repeat_interleave(group, 1)).half()
    assert torch.equal(W, want)


def test_bitlinear_is_a_module_with_the_reference_quantisers():
    import torch.nn as nn
    assert issubclass(kernels.BitLinear, nn.Module)
    w = torch.randn(16, 32)
    s = 1.0 / w.abs().mean().clamp(min=1e-5)
    W_t = (w * s).round().clamp(-1, 1)
    q, scale = R.bitnet_weight_quant(w)
    assert torch.equal(W_t.to(torch.int8), q.to(torch.int8)) and abs(float(scale) - float(s)) < 1e-6


def test_scalar_decode_rules():
    """The per-element helpers: fp8 against torch's own float8 dtypes (every byte), integer fields
    against plain arithmetic."""
    every = torch.arange(256, dtype=torch.uint8)
    want = every.view(torch.float8_e4m3fn).to(torch.float16)
    got = quantize.u8_to_f8_e4m3_to_f16(every)
    nan = torch.isnan(want)
    assert torch.equal(torch.isnan(got), nan) and torch.equal(got[~nan], want[~nan])
    want = every.view(torch.float8_e5m2).to(torch.float16)
    got = quantize.u8_to_f8_e5m2_to_f16(every)
    nan = torch.isnan(want)
    assert torch.equal(torch.isnan(got), nan) and torch.equal(got[~nan], want[~nan])
    word = torch.tensor([0b11100100], dtype=torch.uint8)                    # fields 0, 1, 2, 3 of 2 bits
    pos = torch.arange(4)
    assert quantize.packed_to_unsigned(word, 2, pos, torch.int32).tolist() == [0, 1, 2, 3]
    assert quantize.packed_to_signed(word, 2, pos, torch.int32).tolist() == [-2, -1, 0, 1]
    assert quantize.packed_int_to_int(word, 2, pos, torch.int32).tolist() == [0, 1, -2, -1]
    assert quantize.packed_to_unsigned_with_zeros(word, 2, pos, 1, torch.int32).tolist() == [-1, 0, 1, 2]
    w32 = torch.tensor([0x76543210 - (1 << 32) if 0x76543210 >= 1 << 31 else 0x76543210], dtype=torch.int32)
    assert quantize.packed_to_unsigned(w32, 4, torch.arange(8), torch.int32).tolist() == list(range(8))
    assert quantize.packed_int_to_int(torch.tensor([-1], dtype=torch.int32), 4, torch.arange(8), torch.int32).tolist() == [-1] * 8
    codes = torch.tensor([0x0F], dtype=torch.uint8)                          # low nibble s=1 e=7, high nibble 0
    assert quantize.packed_to_fp4_e3m0_to_f16(codes, torch.arange(2)).tolist() == [-1.0, 0.0]
    assert quantize.packed_to_fp4_e3m0_to_f16(torch.tensor([0x01], dtype=torch.uint8), 0).item() == 2.0 ** -6

