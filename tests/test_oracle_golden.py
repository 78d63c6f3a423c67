"""CPU: the oracle restatements against fixtures generated from the reference's own
helpers (tests/golden/make_golden.py) and against the known-answer vectors its
tests hold."""
import os

import numpy as np
import pytest
import torch

from oracle import ref_programs as R

G = os.path.join(os.path.dirname(__file__), "golden")


def load(name):
    return np.load(os.path.join(G, name))


def test_general_compress_matches_reference():
    g = load("codecs.npz")
    assert np.array_equal(R.general_compress(g["codes4"], 4), g["compress4"].view(np.uint8))
    assert np.array_equal(R.general_compress(g["codes2"], 2), g["compress2"].view(np.uint8))
    assert np.array_equal(R.general_decompress(g["compress4"], 4), g["codes4"].astype(np.uint8))
    assert np.array_equal(R.general_decompress(g["compress2"], 2), g["codes2"].astype(np.uint8))


@pytest.mark.parametrize("nbits,target", [(4, "float16"), (4, "int8"), (2, "int8")])
def test_interleave_weight_matches_reference(nbits, target):
    g = load("codecs.npz")
    assert np.array_equal(R.interleave_weight(g["raw"], nbits, target), g[f"interleave_{nbits}_{target}"])


def test_interleave_weight_rule_for_fp16_target():
    # element e of a word -> bit (e % 2) * 16 + (e // 2) * 4   (quantize/utils.py:92-100)
    for e in range(8):
        w = np.array([0xF << (4 * e)], dtype=np.uint32).view(np.int8).reshape(1, 4)
        out = R.interleave_weight(w, 4, "float16").view(np.uint32)[0]
        assert out == 0xF << ((e % 2) * 16 + (e // 2) * 4)


def test_gen_quant4_symmetric_rule():
    # ref = (q - 8) * s per group, in fp16 (quantize/utils.py:29-30)
    g = load("gen_quant4.npz")
    s, qm8, ref_kn = g["s"], g["q_minus_8"], g["ref_kn"]
    k, n = qm8.shape
    groups = s.shape[0]
    gs = k // groups
    q = torch.from_numpy(qm8.T.astype(np.int64) + 8)                     # (n, k) codes 0..16
    q_ok = q.clamp(max=15)
    qB = torch.from_numpy(R.general_compress(q_ok.numpy(), 4))
    scales = torch.from_numpy(s.T.copy()).to(torch.float16)               # (n, groups)
    W = R.dequant_w4_group(qB, scales, None, gs, torch.float16)           # (n, k)
    same = (q == q_ok)
    assert torch.equal(W[same], torch.from_numpy(ref_kn.T.copy()).to(torch.float16)[same])


def test_fp4_simple_decoder_matches_reference():
    g = load("fp4_decode.npz")
    qb, scale = torch.from_numpy(g["qb"]), torch.from_numpy(g["scale"])
    assert np.array_equal(R.decode_fp4_simple(qb).view(torch.int16).numpy(), g["simple"])
    assert np.array_equal(R.decode_fp4_simple(qb, 32, scale).view(torch.int16).numpy(), g["simple_scaled"])
    allb = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    assert np.array_equal(R.decode_fp4_simple(allb).view(torch.int16).numpy(), g["simple_all"])


def test_fp4_simple_decoder_has_no_zero():
    # codes 0..7 -> 0.5, 0.75, 1, 1.5, 2, 3, 4, 6 (no zero, no subnormal)
    codes = torch.tensor([[0x10, 0x32, 0x54, 0x76]], dtype=torch.uint8)
    vals = R.decode_fp4_simple(codes).float().tolist()[0]
    assert vals == [0.5, 0.75, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0]


def test_fp4_twiddled_decoder_matches_reference_and_is_true_e2m1():
    g = load("fp4_decode.npz")
    qb = torch.from_numpy(g["qb"])
    assert np.array_equal(R.decode_fp4_twiddled(qb).view(torch.int16).numpy(), g["twiddled"])
    allb = torch.arange(256, dtype=torch.uint8).reshape(1, 256)
    tw = R.decode_fp4_twiddled(allb)
    assert np.array_equal(tw.view(torch.int16).numpy(), g["twiddled_all"])
    assert set(tw.float().abs().unique().tolist()) <= {0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0}


def test_e2m1_encode_pack_decode_match_reference():
    g = load("e2m1.npz")
    assert np.array_equal(R.E2M1_VALUES, g["lut"])
    codes = R.encode_fp4_e2m1(g["vals"])
    assert np.array_equal(codes, g["codes"])
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).astype(np.uint8)
    assert np.array_equal(packed, g["packed"].view(np.uint8))
    assert np.array_equal(R.decode_fp4_e2m1(torch.from_numpy(packed)).numpy(), g["decoded"])


def test_e2m1_known_codes():
    # testing/python/quantize/test_tilelang_quantize_nvfp4_scale_layout.py:881-888
    vals = np.array([[0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0, -0.5, -1.0]], dtype=np.float32)
    assert R.encode_fp4_e2m1(vals).tolist() == [[0x0, 0x1, 0x2, 0x3, 0x4, 0x5, 0x6, 0x7, 0x9, 0xA]]


@pytest.mark.parametrize("nbit,values", [(2, [-2, -1, 0, 1]), (4, list(range(-8, 8))), (8, [-128, -17, -1, 0, 1, 42, 127])])
def test_signed_subword_decode_known_values(nbit, values):
    # testing/python/issue/test_tilelang_u32_signed_decode.py:23-49: fields of a
    # uint32 word, little-endian, two's-complement sign extension
    if nbit == 8:
        return  # byte fields need no decoder
    packed = R.general_compress(np.array([v & ((1 << nbit) - 1) for v in values]).reshape(1, -1), nbit)
    codes = R.general_decompress(packed, nbit).astype(np.int64)[0]
    signed = ((codes ^ (1 << (nbit - 1))) - (1 << (nbit - 1))).tolist()
    assert signed == values
    if nbit == 4:
        assert R.sext4(torch.from_numpy(codes.astype(np.uint8))).tolist() == values


def test_int_oracles_are_exact_beyond_float32():
    # the reference checks its integer kernels through a float32 matmul; the oracle
    # must stay exact where float32 is not (|sum| >= 2^24)
    K = 4096
    A = torch.full((1, K), 127, dtype=torch.int8)
    q = torch.from_numpy(R.general_compress(np.full((1, K), 7), 4))
    out = R.ref_w4a8(A, q)
    assert out.item() == 127 * 7 * K


def test_bitnet_quantisers():
    x = torch.tensor([[0.5, -1.0, 0.25, 2.0]], dtype=torch.bfloat16)
    q, s = R.bitnet_activation_quant(x)
    assert s.item() == pytest.approx(127 / 2.0)
    assert q.tolist() == [[32, -64, 16, 127]]
    w = torch.tensor([[0.2, -0.9, 0.05, 1.5]])
    wt, sw = R.bitnet_weight_quant(w)
    assert sw.item() == pytest.approx(1 / w.abs().mean().item())
    assert wt.tolist() == [[0, -1, 0, 1]]


def test_w4a16_reference_shapes_and_rule():
    torch.manual_seed(0)
    M, N, K, g = 4, 8, 256, 128
    A = torch.randn(M, K, dtype=torch.bfloat16)
    q = torch.randint(0, 16, (N, K))
    qB = torch.from_numpy(R.general_compress(q.numpy(), 4))
    s = (torch.rand(N, K // g) * 0.015 + 0.005).to(torch.bfloat16)
    z = (torch.rand(N, K // g) * 4 + 6).to(torch.bfloat16)
    W = ((q.float() - z.float().repeat_interleave(g, 1)) * s.float().repeat_interleave(g, 1)).to(torch.bfloat16)
    ref = (A.float() @ W.float().T).to(torch.bfloat16)
    assert torch.equal(R.ref_w4a16(A, qB, s, z, g, torch.bfloat16), ref)


def test_moe_oracle_routes_top_k():
    torch.manual_seed(0)
    w, idx = R.moe_route(torch.randn(5, 8), 2)
    assert idx.shape == (5, 2) and torch.all(w > 0) and torch.all(w.sum(-1) <= 1.0 + 1e-6)


def test_mxfp4_activation_quantiser_matches_reference_outputs():
    """``fp4_act_quant_ref`` of examples/deepseek_v4/act_quant.py:249-268 run on seeded inputs
    (scales over five decades) when the fixtures were made."""
    g = load("blockscale.npz")
    x = torch.from_numpy(g["xm"]).view(torch.bfloat16)
    codes, scale = R.mxfp4_act_quant(x, 32, ties="down")
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).numpy()
    assert np.array_equal(packed, g["mx32_packed"])
    assert np.array_equal(scale.numpy(), g["mx32_scale"])
    # the hardware tie rule differs from the reference's argmin only on exact midpoints
    even, _ = R.mxfp4_act_quant(x, 32, ties="even")
    assert (even != codes).float().mean() < 0.02

