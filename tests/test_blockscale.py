"""CPU: the block-scaled 4-bit formats (``tilelang_b200.blockscale``) against outputs of the
reference's own helpers stored in ``tests/golden/blockscale.npz`` and ``e2m1.npz`` (written by
``tests/golden/make_golden.py`` from examples/dequantize_gemm/quantize/nvfp4.py,
examples/deepseek_v4/act_quant.py and examples/deepseek_v4/fp8_fp4_gemm_1d1d_sm100.py), plus the
known answers of testing/python/quantize/test_tilelang_quantize_nvfp4_scale_layout.py."""
import os

import numpy as np
import pytest
import torch

from tilelang_b200 import blockscale as B

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


@pytest.fixture(scope="module")
def gold():
    return np.load(os.path.join(GOLD, "blockscale.npz"))


def u32(a):
    return torch.from_numpy(a).view(torch.uint32)


def test_e2m1_codes_match_the_reference_encoder_and_decoder():
    g = np.load(os.path.join(GOLD, "e2m1.npz"))
    vals = torch.from_numpy(g["vals"])
    codes = B.e2m1_encode(vals, "up")
    assert np.array_equal(codes.numpy(), g["codes"])                      # thresholds included
    packed = B.e2m1_pack(codes)
    assert np.array_equal(packed.view(torch.int8).numpy(), g["packed"])
    assert np.array_equal(B.e2m1_decode(B.e2m1_unpack(packed)).numpy(), g["decoded"])
    assert np.array_equal(np.array(B.E2M1_MAGNITUDES, dtype=np.float32), g["lut"][:8])


def test_e2m1_tie_rules():
    mids = torch.tensor([0.25, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0])
    assert B.e2m1_encode(mids, "up").tolist() == [1, 2, 3, 4, 5, 6, 7]
    assert B.e2m1_encode(mids, "down").tolist() == [0, 1, 2, 3, 4, 5, 6]
    assert B.e2m1_encode(mids, "even").tolist() == [0, 2, 2, 4, 4, 6, 6]
    assert B.e2m1_encode(-mids, "even").tolist() == [0, 10, 10, 12, 12, 14, 14]
    assert B.e2m1_encode(torch.tensor([-0.1]), "even", signed_zero=True).tolist() == [8]
    assert B.e2m1_encode(torch.tensor([7.0, -100.0, float("nan")])).tolist() == [7, 15, 0]


def test_ue4m3_codec_matches_the_reference(gold):
    allb = torch.arange(256, dtype=torch.uint8)
    got, want = B.ue4m3_decode(allb).numpy(), gold["ue4m3_decode_all"]
    assert np.array_equal(np.isnan(got), np.isnan(want)) and np.array_equal(got[~np.isnan(got)], want[~np.isnan(want)])
    x = torch.from_numpy(gold["sweep"])
    assert np.array_equal(B.ue4m3_encode(x).numpy(), gold["ue4m3_nearest"])
    assert np.array_equal(B.ue4m3_encode(x, "ceil").numpy(), gold["ue4m3_ceil"])
    assert np.array_equal(B.ue4m3_encode(x, "ceil", min_positive=True).numpy(), gold["ue4m3_ceil_minpos"])
    codes = torch.arange(127, dtype=torch.uint8)                          # every finite code is a fixed point
    assert torch.equal(B.ue4m3_encode(B.ue4m3_decode(codes)), codes)
    assert torch.equal(B.ue4m3_encode(B.ue4m3_decode(codes), "ceil"), codes)


def test_scale_word_swizzle_matches_the_reference_and_its_known_answers(gold):
    words = u32(gold["words"])
    sw = B.sf_swizzle_128x4(words)
    assert torch.equal(sw.view(torch.int32), torch.from_numpy(gold["swizzled"]))
    assert torch.equal(B.sf_unswizzle_128x4(sw).view(torch.int32), words.view(torch.int32))
    # test_tilelang_quantize_nvfp4_scale_layout.py: word (row, k64) of a 128 x 4 tile sits at flat
    # word (k64 * 32 + row % 32) * 4 + row // 32, i.e. byte offsets 0 -> 0, 32 -> 4, 64 -> 8,
    # 96 -> 12, 127 -> 508 for k64 = 0
    tile = torch.arange(128 * 4, dtype=torch.int64).reshape(128, 4).to(torch.uint32)
    flat = B.sf_swizzle_128x4(tile).reshape(-1).to(torch.int64)
    for row, byte_off in ((0, 0), (32, 4), (64, 8), (96, 12), (127, 508)):
        assert int(flat[byte_off // 4]) == row * 4
    # rows are padded to whole 128-row blocks with zeros
    assert B.sf_swizzle_128x4(torch.ones(5, 4, dtype=torch.int32).view(torch.uint32)).shape == (128, 4)


def test_nvfp4_quantiser_matches_the_reference(gold):
    x = torch.from_numpy(gold["xa"]).view(torch.bfloat16)
    packed, words, sb = B.quantize_nvfp4(x, return_scale_bytes=True)
    assert np.array_equal(sb.numpy(), gold["nv_bytes"])
    assert np.array_equal(packed.numpy(), gold["nv_packed"])
    assert np.array_equal(words.view(torch.int32).numpy(), gold["nv_words"])
    assert int(sb[5, 0]) == 0 and not packed[5, :8].any()                 # the all-zero block
    with pytest.raises(ValueError):
        B.quantize_nvfp4(torch.zeros(100, 256))


def test_mxfp4_quantisers_match_the_reference(gold):
    x = torch.from_numpy(gold["xm"]).view(torch.bfloat16)
    # block 32, the activation quantiser's torch reference: nearest by argmin (ties down)
    packed, sbytes, scale = B.quantize_mxfp4(x, 32, ties="down")
    assert np.array_equal(scale.numpy(), gold["mx32_scale"])
    assert np.array_equal(packed.numpy(), gold["mx32_packed"])
    assert torch.equal(torch.pow(2.0, sbytes.float() - 127.0), scale)
    # block 128 with group-major packed e8m0 words
    packed, sbytes, _ = B.quantize_mxfp4(x.float(), 128, ties="down", signed_zero=False)
    assert np.array_equal(sbytes.numpy(), gold["mx128_sf"])
    assert np.array_equal(packed.numpy(), gold["mx128_packed"])
    pad = torch.full((x.shape[0], 4), 127, dtype=torch.uint8)
    pad[:, :sbytes.shape[1]] = sbytes
    assert np.array_equal(B.sf_pack_group_major(pad).view(torch.int32).numpy(), gold["mx128_words"])
    # a round trip stays within half a step of the block's grid
    deq = B.dequantize_mxfp4(*B.quantize_mxfp4(x, 32)[:2])
    assert ((deq - x.float()).abs() <= B.quantize_mxfp4(x, 32)[2].repeat_interleave(32, 1) * 1.0 + 1e-30).all()


def test_pow2_ceil():
    x = torch.tensor([1.0, 1.0001, 0.75, 3.0, 2.0 ** -20, 6 * 2.0 ** -126 / 6])
    assert B.pow2_ceil(x).tolist() == [1.0, 2.0, 1.0, 4.0, 2.0 ** -20, 2.0 ** -126]
