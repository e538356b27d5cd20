"""Dense W8A16 quantiser and truncating dequant on the GPU, bit for bit against the oracle.

NaN results (0 * inf on a column whose scale overflowed) are compared as NaNs: the sign and payload
of a NaN a multiply produces differ between x86 (0xFFC0 after truncation) and CUDA (0x7FFF), and
neither the reference's kernel nor its CPU code defines one.  Every other value is compared by bits.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def assert_bf16_bits_equal(got_u16, ref_u16):
    """Bit equality of bf16 patterns, with any NaN equal to any NaN."""
    got_u16 = np.asarray(got_u16, dtype=np.uint16)
    ref_u16 = np.asarray(ref_u16, dtype=np.uint16)
    nan_got = ((got_u16 & 0x7F80) == 0x7F80) & ((got_u16 & 0x007F) != 0)
    nan_ref = ((ref_u16 & 0x7F80) == 0x7F80) & ((ref_u16 & 0x007F) != 0)
    np.testing.assert_array_equal(nan_got, nan_ref)
    np.testing.assert_array_equal(got_u16[~nan_ref], ref_u16[~nan_ref])


@pytest.mark.parametrize("K,N,g", [(4, 1, 0), (8, 3, 0), (256, 7, 128), (200, 7, 128), (77, 19, 32),
                                   (512, 256, 0), (1000, 384, 128), (4096, 1024, 128), (300, 130, 7),
                                   (5120, 2048, 0)])
def test_quantiser_and_dequant_match_oracle(K, N, g):
    import torch
    from ateniaengine_b200 import int8_to_bf16_per_group, quantize_per_group_i8
    from oracle import oracle as orc
    gen = torch.Generator(device="cpu").manual_seed(K * 31 + N)
    w = torch.randn((K, N), generator=gen, dtype=torch.float32) * 0.02
    if K >= 8 and N >= 3:
        w[:, 1] = 0.0                       # zero column: floor scale
        w[2, 2] = float("nan")
        w[5, 0] = float("inf")
        w[6, 2] = 3.0                       # outlier
    q, s = quantize_per_group_i8(w.cuda(), g)
    q_ref, s_ref = orc.absmax_per_group_symmetric(w.numpy(), g)
    np.testing.assert_array_equal(s.cpu().numpy().view(np.uint32), s_ref.view(np.uint32))
    np.testing.assert_array_equal(q.cpu().numpy(), q_ref)
    out = int8_to_bf16_per_group(q, s, g)
    ref = orc.int8_to_bf16_per_group(q_ref, s_ref, g)
    assert_bf16_bits_equal(out.view(torch.int16).cpu().numpy().view(np.uint16), ref)
    if K >= 8 and N >= 3:
        assert np.isnan(w.numpy()).any() and np.isinf(w.numpy()).any()  # the special values stay in the case


def test_misaligned_views_take_the_scalar_path():
    import torch
    from ateniaengine_b200 import _lib
    from oracle import oracle as orc
    import ctypes as C
    K, N, g = 64, 24, 16
    gen = torch.Generator(device="cpu").manual_seed(9)
    w = torch.randn((K * N + 1,), generator=gen, dtype=torch.float32)
    wd = w.cuda()
    q = torch.zeros(K * N + 1, dtype=torch.int8, device="cuda")
    s = torch.zeros((K // g) * N + 1, dtype=torch.float32, device="cuda")
    out = torch.zeros(K * N + 1, dtype=torch.int16, device="cuda")
    st = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    lib = _lib.lib()
    # every buffer starts one element past an aligned address
    _lib.check(lib.atenia_quantize_per_group_i8(wd.data_ptr() + 4, K, N, g, q.data_ptr() + 1, s.data_ptr() + 4, st), "q")
    _lib.check(lib.atenia_int8_to_bf16_per_group(q.data_ptr() + 1, s.data_ptr() + 4, K, N, g, out.data_ptr() + 2, st), "d")
    torch.cuda.synchronize()
    q_ref, s_ref = orc.absmax_per_group_symmetric(w[1:].numpy().reshape(K, N), g)
    np.testing.assert_array_equal(q[1:].cpu().numpy().reshape(K, N), q_ref)
    np.testing.assert_array_equal(s[1:].cpu().numpy().reshape(-1, N), s_ref)
    assert_bf16_bits_equal(out[1:].cpu().numpy().view(np.uint16).reshape(K, N),
                           orc.int8_to_bf16_per_group(q_ref, s_ref, g))


def test_argument_errors_and_empty():
    # -1 = ATENIA_ERR_NULL, -2 = ATENIA_ERR_SHAPE
    import torch
    from ateniaengine_b200 import _lib
    lib = _lib.lib()
    buf = torch.zeros(64, dtype=torch.float32, device="cuda")
    assert lib.atenia_quantize_per_group_i8(buf.data_ptr(), 0, 8, 0, buf.data_ptr(), buf.data_ptr(), None) == 0
    assert lib.atenia_quantize_per_group_i8(buf.data_ptr(), -1, 8, 0, buf.data_ptr(), buf.data_ptr(), None) == -2
    assert lib.atenia_quantize_per_group_i8(None, 2, 8, 0, buf.data_ptr(), buf.data_ptr(), None) == -1
    assert lib.atenia_int8_to_bf16_per_group(buf.data_ptr(), buf.data_ptr(), 2, 8, -3, buf.data_ptr(), None) == -2
    assert lib.atenia_int8_to_bf16_per_group(buf.data_ptr(), None, 2, 8, 0, buf.data_ptr(), None) == -1
