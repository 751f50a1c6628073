"""Dense node update and softmax (through the C ABI) against the fp64 CPU oracle."""
import numpy as np
import pytest
import torch

import mgg_osdi23_b200 as mgg
from mgg_osdi23_b200 import graphgen as gg
from gpu_util import RTOL, ATOL

pytestmark = pytest.mark.gpu

SHAPES = [(1000, 602, 16), (777, 16, 41), (513, 100, 64), (300, 64, 64), (301, 64, 47), (129, 128, 172),
          (1, 3, 1), (65, 7, 5), (4096, 128, 16)]


@pytest.mark.parametrize("n,k,m", SHAPES)
def test_dense_matches_oracle(oracle, n, k, m):
    dev = torch.device("cuda")
    x = gg.features(n, k, seed=n).numpy()
    w = gg.glorot_uniform(k, m, seed=k).numpy()
    out = torch.empty(n, m, device=dev)
    mgg.dense_forward(out, torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev))
    # precision: fp32-equivalent (default path), compared with the double-accumulated product
    np.testing.assert_allclose(out.cpu().numpy(), oracle.dense(x, w), rtol=RTOL, atol=ATOL)


def test_dense_epilogues(oracle):
    dev = torch.device("cuda")
    x = gg.features(500, 33, seed=1).numpy()
    w = gg.glorot_uniform(33, 16, seed=2).numpy()
    s = np.random.default_rng(0).uniform(0.1, 2, 500).astype(np.float32)
    out = torch.empty(500, 16, device=dev)
    mgg.dense_forward(out, torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev),
                      row_scale_=torch.from_numpy(s).to(dev), relu=True)
    np.testing.assert_allclose(out.cpu().numpy(), oracle.dense(x, w, row_scale=s, relu=True), rtol=RTOL, atol=ATOL)


def test_reference_all_ones_weights():
    """The reference fills W (and its inputs) with 1.0: every output equals dim1 exactly."""
    dev = torch.device("cuda")
    d_in = torch.ones(100, 602, device=dev)
    d_out = torch.zeros(100, 16, device=dev)
    dp = mgg.dense_param_new_beg("d-1", d_in, d_out, 100, 602, 16)
    mgg.dense_beg_new_forward(dp)
    assert torch.equal(d_out, torch.full_like(d_out, 602.0))


@pytest.mark.parametrize("n,c", [(1000, 41), (333, 47), (64, 172), (5, 1), (17, 33)])
def test_softmax_matches_oracle(oracle, n, c):
    dev = torch.device("cuda")
    z = (gg.features(n, c, seed=c).numpy() * 30).astype(np.float32)    # large logits: needs the max subtraction
    d_in = torch.from_numpy(z).to(dev)
    smx = mgg.softmax_new_param("smx", d_in, d_in, n, c)                # in place, as the reference's GCN driver does
    mgg.softmax_new_forward(smx)
    got = d_in.cpu().numpy()
    np.testing.assert_allclose(got, oracle.softmax(z), rtol=1e-5, atol=1e-7)
    np.testing.assert_allclose(got.sum(1), 1.0, rtol=1e-5)


def test_tensor_core_kernel_reports_clean_status_and_matches_cuda_core_kernel(oracle):
    """The default path (row-streaming kernel for outputs of at most 16 columns, tcgen05 kernel otherwise),
    the tensor-core kernel forced (DENSE_TENSOR) and the CUDA-core kernels forced (DENSE_SIMT), including
    rows that do not fill a 128-row tile and a K tail that does not fill a 32-float slab."""
    import ctypes as C
    from mgg_osdi23_b200 import _lib
    dev = torch.device("cuda")
    for n, k, m in [(128, 32, 16), (129, 602, 16), (1000, 100, 64), (5000, 64, 47), (77, 16, 41), (40000, 602, 16),
                    (3001, 128, 16), (1001, 130, 12), (333, 602, 9), (7, 64, 1), (2050, 100, 128)]:
        x = gg.features(n, k, seed=n).numpy()
        w = gg.glorot_uniform(k, m, seed=k).numpy()
        xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
        a, b, c = (torch.full((n, m), 9.0, device=dev) for _ in range(3))
        mgg.dense_forward(a, xd, wd)
        mgg.dense_forward(b, xd, wd, flags=_lib.DENSE_SIMT)
        mgg.dense_forward(c, xd, wd, flags=_lib.DENSE_TENSOR)
        torch.cuda.synchronize()
        status = C.c_int(-1)
        _lib.check(_lib.lib.mggb_dense_device_status(C.byref(status), 1))
        assert status.value == 0, f"a bounded wait expired in the tensor-core kernel (code {status.value}) for {(n, k, m)}"
        want = oracle.dense(x, w)
        np.testing.assert_allclose(a.cpu().numpy(), want, rtol=RTOL, atol=ATOL, err_msg=str((n, k, m)))
        np.testing.assert_allclose(b.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
        np.testing.assert_allclose(c.cpu().numpy(), want, rtol=RTOL, atol=ATOL, err_msg=str((n, k, m)))
        np.testing.assert_allclose(a.cpu().numpy(), b.cpu().numpy(), rtol=RTOL, atol=2e-5)


@pytest.mark.parametrize("n,k,m", [(1003, 16, 172), (777, 16, 41), (301, 64, 47), (65, 7, 5), (1, 3, 1), (8, 4, 256),
                                   (4099, 128, 33), (5000, 64, 128), (130, 100, 47), (127, 36, 16), (20000, 64, 47)])
def test_fused_dense_softmax_matches_oracle(oracle, n, k, m):
    dev = torch.device("cuda")
    x = (gg.features(n, k, seed=n).numpy() * 4).astype(np.float32)
    w = gg.glorot_uniform(k, m, seed=k).numpy()
    xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    out = torch.empty(n, m, device=dev)
    logits = torch.empty(n, m, device=dev)
    mgg.dense_softmax_forward(out, xd, wd, logits)
    want_logits = oracle.dense(x, w)
    np.testing.assert_allclose(logits.cpu().numpy(), want_logits, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(out.cpu().numpy(), oracle.softmax(want_logits.astype(np.float32)), rtol=2e-5, atol=1e-7)
    # without the logits: the same bits from the same kernel, or, for wide inputs (a multiple of 4 above 32 floats, at
    # most 128 classes), the tensor-core kernel with the softmax in its epilogue, held to the same tolerance
    out2 = torch.full((n, m), -1.0, device=dev)
    mgg.dense_softmax_forward(out2, xd, wd)
    if k % 4 == 0 and k > 32 and m <= 128:
        np.testing.assert_allclose(out2.cpu().numpy(), oracle.softmax(want_logits.astype(np.float32)), rtol=2e-5, atol=1e-7)
        np.testing.assert_allclose(out2.sum(1).cpu().numpy(), 1.0, rtol=1e-5)
    else:
        assert torch.equal(out, out2)
    # and the reference's two calls agree with the single one through the parameter structs
    dp = mgg.dense_param_new_hidden("d-2", xd, torch.zeros(n, m, device=dev), n, k, m)
    dp.set_weight(wd)
    dp.flags = 4                                                        # CUDA-core dense: the same fp32 FMA chain
    probs = torch.zeros(n, m, device=dev)
    smx = mgg.softmax_new_param("smx", dp.d_out, probs, n, m)
    mgg.dense_hidden_new_forward(dp)
    mgg.softmax_new_forward(smx)
    np.testing.assert_allclose(out.cpu().numpy(), probs.cpu().numpy(), rtol=2e-5, atol=1e-7)


def test_fused_dense_softmax_refuses_what_it_cannot_hold():
    dev = torch.device("cuda")
    assert not mgg.dense_softmax_fits(16, 300) and not mgg.dense_softmax_fits(602, 172)
    with pytest.raises(mgg.MggbError):
        mgg.dense_softmax_forward(torch.empty(4, 300, device=dev), torch.ones(4, 16, device=dev), torch.ones(16, 300, device=dev))
    # the struct-level call falls back to the two kernels for such a shape
    d_in = torch.ones(4, 16, device=dev)
    dp = mgg.dense_param_new_hidden("d", d_in, torch.zeros(4, 300, device=dev), 4, 16, 300)
    probs = torch.zeros(4, 300, device=dev)
    mgg.dense_hidden_softmax_new_forward(dp, mgg.softmax_new_param("s", dp.d_out, probs, 4, 300))
    np.testing.assert_allclose(probs.cpu().numpy(), 1.0 / 300, rtol=1e-6)


@pytest.mark.parametrize("n,k,m", [(700, 64, 64), (600, 602, 16), (300, 100, 47)])
def test_dense_output_and_publish_views_at_odd_float_offsets(oracle, n, k, m):
    """out and the publish destinations only have to be 4-byte aligned: a view that starts one float
    into an allocation takes the element-wise store path instead of 128-bit stores (which would fault)."""
    dev = torch.device("cuda")
    x = gg.features(n, k, seed=n).numpy()
    w = gg.glorot_uniform(k, m, seed=k).numpy()
    want = oracle.dense(x, w)
    xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    for off_out, off_pub in ((1, 0), (0, 3), (2, 1), (0, 0)):
        raw_o = torch.zeros(n * m + 8, device=dev)
        raw_p = torch.zeros(n * m + 8, device=dev)
        out = raw_o[off_out:off_out + n * m].view(n, m)
        pub = raw_p[off_pub:off_pub + n * m].view(n, m)
        assert out.data_ptr() % 16 == (4 * off_out) % 16
        for flags in (0, mgg._lib.DENSE_TENSOR):
            out.zero_(); pub.zero_()
            mgg.dense_forward(out, xd, wd, publish=[pub], flags=flags)
            torch.cuda.synchronize()
            np.testing.assert_allclose(out.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
            assert torch.equal(out, pub)
        assert float(raw_o[:off_out].abs().sum()) == 0.0 and float(raw_o[off_out + n * m:].abs().sum()) == 0.0
    st = mgg._lib.C.c_int(-1)
    mgg._lib.check(mgg._lib.lib.mggb_dense_device_status(mgg._lib.C.byref(st), 0))
    assert st.value == 0


@pytest.mark.parametrize("n,k,m", [(2000, 602, 16), (1500, 64, 64), (900, 100, 47)])
def test_single_pass_tf32_mode(oracle, n, k, m):
    """MGGB_DENSE_TF32: one tensor-core pass with both operands truncated to TF32 (10 mantissa bits), what
    cublasSgemm gives under its TF32 math mode.  Tolerance: 2e-3 of sum_k |x_ik| |w_kj| per element (each
    product is off by at most 2 * 2^-10 of its magnitude).  The default mode on the same inputs stays within
    the fp32 tolerance, so the flag is what made the difference."""
    dev = torch.device("cuda")
    x = gg.features(n, k, seed=n).numpy()
    w = gg.glorot_uniform(k, m, seed=k).numpy()
    want = oracle.dense(x, w)
    mag = oracle.dense(np.abs(x), np.abs(w))
    xd, wd = torch.from_numpy(x).to(dev), torch.from_numpy(w).to(dev)
    fast = torch.empty(n, m, device=dev)
    mgg.dense_forward(fast, xd, wd, flags=mgg._lib.DENSE_TF32)
    full = torch.empty(n, m, device=dev)
    mgg.dense_forward(full, xd, wd, flags=mgg._lib.DENSE_TENSOR)
    torch.cuda.synchronize()
    err_fast = np.abs(fast.cpu().numpy() - want)
    assert np.all(err_fast <= 2e-3 * mag + 1e-6)
    np.testing.assert_allclose(full.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    assert err_fast.max() > 10 * np.abs(full.cpu().numpy() - want).max()
