import numpy as np
import pytest
import torch

from mary_b200.nn import fp4
from mary_b200.ops import reference as ref


def test_e4m3_roundtrip_all_bytes_and_torch_agreement():
    b = np.arange(0x7F, dtype=np.uint8)
    assert np.array_equal(fp4.e4m3_encode(fp4.e4m3_decode(b)), b)
    x = np.minimum(np.abs(np.random.default_rng(0).standard_normal(20000).astype(np.float32)) * 60, 448)
    t = torch.from_numpy(x).to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    assert np.array_equal(t, fp4.e4m3_encode(x))
    # exact ties go to the even mantissa
    assert fp4.e4m3_encode(np.float32([1.0625, 1.1875]))[0] == 0x38 and fp4.e4m3_encode(np.float32([1.1875]))[0] == 0x3A


def test_e2m1_thresholds_ties_away_and_signed_zero():
    y = np.float32([0.0, 0.25, -0.25, 0.2499, 0.75, 1.25, 1.75, 2.5, 3.5, 5.0, 100.0, -0.1, -0.0])
    c = fp4.encode_e2m1(y)
    assert c.tolist() == [0, 1, 9, 0, 2, 3, 4, 5, 6, 7, 7, 8, 8]
    packed = fp4.pack_codes(np.array([[1, 2, 3, 12]], dtype=np.uint8))
    assert packed.tolist() == [[0x21, 0xC3]]                     # low nibble = lower index
    assert fp4.decode_codes(packed).tolist() == [[0.5, 1.0, 1.5, -2.0]]


def test_activation_quantiser_rules_and_torch_twin():
    rng = np.random.default_rng(1)
    x = rng.standard_normal((6, 64)).astype(np.float32) * 3
    x[0, :16] = 0                                                # zero block
    x[1, :16] = 1e6                                              # clamps at 448
    x[2, 0] = -1e-9                                              # negative that rounds to zero
    codes, scales = fp4.quantize_act_nvfp4(x)
    assert scales[0, 0] == 0 and np.all(codes[0, :8] == 0)
    assert scales[1, 0] == 0x7E
    assert (codes[2, 0] & 0xF) == 8
    tc, ts = ref.quantize_nvfp4(torch.from_numpy(x))
    assert np.array_equal(tc.numpy(), codes) and np.array_equal(ts.numpy(), scales)
    d = fp4.decode_nvfp4(codes, scales)
    assert np.allclose(ref.dequantize_nvfp4(tc, ts).numpy(), d)
    rel = np.abs(d[3:] - x[3:]).max() / np.abs(x[3:]).max()
    assert rel < 0.2


def test_mxfp4_relabel_exact_and_span_refused():
    rng = np.random.default_rng(2)
    w = rng.standard_normal((4, 128)).astype(np.float32)
    w[1] *= 2.0 ** 10
    c, s = fp4.quantize_mxfp4(w)
    ref_dec = fp4.decode_mxfp4(c, s)
    c2, s2, g = fp4.transcode_mxfp4_to_nvfp4(c, s)
    assert np.array_equal(fp4.decode_nvfp4(c2, s2, g), ref_dec)        # bit exact
    w[2] *= 2.0 ** -30                                                 # span beyond 17 octaves
    c, s = fp4.quantize_mxfp4(w)
    with pytest.raises(fp4.SpanError):
        fp4.transcode_mxfp4_to_nvfp4(c, s)


def test_scale_swizzle_layout():
    s = np.arange(128 * 8, dtype=np.uint32).reshape(128, 8).astype(np.uint8)
    t = fp4.swizzle_scales_128x4(s)
    assert t.shape == (1, 2, 512)
    for r, k in ((0, 0), (31, 3), (32, 0), (97, 5), (127, 7)):
        assert t[0, k // 4, (r % 32) * 16 + (r // 32) * 4 + k % 4] == s[r, k]
