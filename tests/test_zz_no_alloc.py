"""zc_dmmv_q4k_static_scratch (scratch in a __device__ array, no context, no allocation) against
zc_dmmv on the same inputs. The file name sorts last so the shared scratch is exercised after
every other test has run; it also passes on its own."""
import ctypes as C

import numpy as np
import pytest

import zinc_b200 as zb
from zinc_b200 import _lib, synth
from helpers import canary_intact, dev, out_with_canary, rel_l2

pytestmark = pytest.mark.gpu

TOL = 1e-4


def static_call(torch, w, x, y, M, K, status, acc_mode=0, a_offset=0, stream=None):
    L = _lib.lib()
    err = C.create_string_buffer(256)
    s = torch.cuda.current_stream().cuda_stream if stream is None else stream
    rc = L.zc_dmmv_q4k_static_scratch(
        C.c_void_p(s), C.c_void_p(w.data_ptr()), w.numel() * w.element_size(),
        C.c_void_p(x.data_ptr()), x.numel() * 4, C.c_void_p(y.data_ptr()), y.numel() * 4,
        M, K, a_offset, 0, 0, acc_mode, C.c_void_p(status.data_ptr()), err, 256)
    return rc, err.value.decode()


@pytest.mark.parametrize("M,K", [(4096, 4096), (67, 2048), (12288, 4096), (1000, 12288)])
def test_matches_zc_dmmv_twice_in_a_row(gpu, oracle, M, K):
    torch, ctx, dd = gpu
    g = synth.rng(120, M * 31 + K)
    w = synth.quant_matrix(g, zb.Q4_K, M, K)
    x1, x2 = synth.activations(g, K), synth.activations(g, K) * np.float32(0.25)
    wd = dev(torch, w)
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    for x in (x1, x2):  # two calls in a row on one stream share the scratch
        xd = dev(torch, x)
        y_ref = out_with_canary(torch, M)
        y_new = out_with_canary(torch, M)
        dd.recordDispatch(zb.Q4_K, wd, xd, y_ref, M, K)
        rc, msg = static_call(torch, wd, xd, y_new, M, K, status)
        assert rc == _lib.OK, msg
        rc, msg = static_call(torch, wd, xd, y_new, M, K, status, acc_mode=1)  # y_new = 2 W x
        assert rc == _lib.OK, msg
        ctx.submit_and_wait()
        assert status.cpu().tolist() == [0, 0]
        assert canary_intact(y_new, M) and canary_intact(y_ref, M)
        ref = y_ref[:M].cpu().numpy()
        got = y_new[:M].cpu().numpy()
        if M * (K // 256) * 144 >= (2 << 20):
            assert np.array_equal(got, ref + ref)  # zc_dmmv streams too: same kernel, same worker split, same bits
        else:  # zc_dmmv runs small matrices one warp per row: same value, different summation order
            assert rel_l2(got, ref + ref) <= 1e-5
        assert rel_l2(ref, oracle.dmmv_f64(w, zb.Q4_K, M, K, x)) <= TOL


def test_weight_offset(gpu, oracle):
    torch, ctx, dd = gpu
    M, K = 257, 2048
    g = synth.rng(121, 0)
    w = synth.quant_matrix(g, zb.Q4_K, M, K)
    x = synth.activations(g, K)
    buf = np.full(w.size + 96, 0xCD, dtype=np.uint8)
    buf[32:32 + w.size] = w.reshape(-1)
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    y = out_with_canary(torch, M)
    rc, msg = static_call(torch, dev(torch, buf), dev(torch, x), y, M, K, status, a_offset=32)
    assert rc == _lib.OK, msg
    torch.cuda.synchronize()
    assert status.cpu().tolist() == [0, 0]
    assert canary_intact(y, M)
    assert rel_l2(y[:M].cpu().numpy(), oracle.dmmv_f64(w, zb.Q4_K, M, K, x)) <= TOL


def test_refusals(gpu):
    torch, ctx, dd = gpu
    status = torch.zeros(2, dtype=torch.int32, device="cuda")
    w = torch.zeros(64 * 64 * 144, dtype=torch.uint8, device="cuda")
    x = torch.zeros(16384, dtype=torch.float32, device="cuda")
    y = torch.zeros(64, dtype=torch.float32, device="cuda")
    rc, msg = static_call(torch, w, x, y, 64, 16384, status)  # K beyond the maximum
    assert rc == _lib.ERR_INVALID_ARG and "maximum" in msg
    rc, msg = static_call(torch, w, x, y, 16, 512, status)  # too few units
    assert rc == _lib.ERR_INVALID_ARG and "too small" in msg
    rc, msg = static_call(torch, w, x, y, 64, 1000, status)  # K not a multiple of 256
    assert rc == _lib.ERR_INVALID_ARG
    rc, msg = static_call(torch, w, x, y, 4096, 4096, status)  # weights larger than the buffer
    assert rc == _lib.ERR_INVALID_ARG and "exceeds" in msg
    rc, msg = static_call(torch, w, x, y, 64, 2048, status, a_offset=4)  # misaligned weights
    assert rc == _lib.ERR_INVALID_ARG and "aligned" in msg
    L = _lib.lib()
    rc = L.zc_dmmv_q4k_static_scratch(None, C.c_void_p(w.data_ptr()), w.numel(), C.c_void_p(x.data_ptr()),
                                      x.numel() * 4, C.c_void_p(y.data_ptr()), 256, 64, 2048, 0, 0, 0, 0, None, None, 0)
    assert rc == _lib.ERR_INVALID_ARG  # status words are mandatory
    torch.cuda.synchronize()
    assert float(y.abs().sum()) == 0.0
