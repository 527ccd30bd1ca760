"""The allocation-free backward entry point (b200rl_dense_backward_static_scratch) against the regular one.

Some callers of the library cannot provide scratch memory and must not allocate it: code that sits behind the
reference's own `backward(device, layer, input, d_output, buffer)` signature has no parameter for scratch, and a
cudaMalloc in the middle of a training step would synchronise the device. For them the split-batch partial sums live in
a static device array inside the library. This file is collected last on purpose: if it fails, every other test has
already run. It passes alone in a fresh process and after the other tests."""
import ctypes as C

import numpy as np
import pytest

import make_golden as mg

pytestmark = pytest.mark.gpu


def _backward(lib, torch, entry, W, x, pre, d_out, act, with_scratch):
    B, I = x.shape
    O = W.shape[0]
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    dW, db, d_in, dd = t(np.zeros((O, I), np.float32)), t(np.zeros(O, np.float32)), torch.empty((B, I), device="cuda"), t(d_out)
    Wd, xd, pd = t(W), t(x), t(pre)
    p = lambda z: C.c_void_p(z.data_ptr())
    L = lib.lib()
    if with_scratch:
        n = L.b200rl_dense_backward_scratch_bytes(B, I, O)
        scratch = torch.empty(max(n, 4), dtype=torch.uint8, device="cuda")
        rc = L.b200rl_dense_backward(p(Wd), p(xd), I, p(pd), O, p(dd), O, p(dW), p(db), p(d_in), I, B, I, O, lib.ACT[act], p(scratch), n, None)
    else:
        rc = entry(p(Wd), p(xd), I, p(pd), O, p(dd), O, p(dW), p(db), p(d_in), I, B, I, O, lib.ACT[act], None)
    lib.check(rc, "dense backward")
    torch.cuda.synchronize()
    return [z.cpu().numpy() for z in (dW, db, d_in, dd)]


@pytest.mark.parametrize("B,I,O,act", [(4096, 64, 256, "relu"), (2048, 27, 64, "tanh"), (300, 10, 7, "identity")])
def test_static_scratch_backward_equals_regular_backward_twice_in_a_row(lib, B, I, O, act):
    import torch
    L = lib.lib()
    W = (mg.det_uniform(B + O, O * I) / np.float32(np.sqrt(I))).reshape(O, I)
    ref = None
    for call in range(2):        # second call reuses the static array with the first call's contents still in it
        x = mg.det_normal(B + call, B * I, stream=1).reshape(B, I)
        pre = mg.det_normal(B + call, B * O, stream=2).reshape(B, O)
        d_out = mg.det_normal(B + call, B * O, stream=3).reshape(B, O)
        want = _backward(lib, torch, None, W, x, pre, d_out, act, with_scratch=True)
        got = _backward(lib, torch, L.b200rl_dense_backward_static_scratch, W, x, pre, d_out, act, with_scratch=False)
        for a, b in zip(got, want):          # same kernels, same fixed-order reduction: identical bits
            assert np.array_equal(a, b)


def test_large_batch_is_split_within_the_static_array(lib):
    """A training-sized layer (256 x 256 at batch 8192) would take 32 splits = exactly 8 MiB of weight-gradient partial sums plus the bias
    partial sums with caller scratch: more than the static array holds. The static entry point plans with fewer splits instead of refusing;
    the result differs from the caller-scratch one only by the summation order of the batch split, i.e. within the sums' bound
    1e-6 + 1e-5 * sum|terms|; d_pre and d_in do not depend on the split and are identical."""
    import torch
    L = lib.lib()
    B, I, O = 8192, 256, 256
    assert L.b200rl_dense_backward_scratch_bytes(B, I, O) > 8 * 1024 * 1024
    W = (mg.det_uniform(77, O * I) / np.float32(np.sqrt(I))).reshape(O, I)
    for call in range(2):
        x = mg.det_normal(900 + call, B * I, stream=1).reshape(B, I)
        pre = mg.det_normal(900 + call, B * O, stream=2).reshape(B, O)
        d_out = mg.det_normal(900 + call, B * O, stream=3).reshape(B, O)
        want = _backward(lib, torch, None, W, x, pre, d_out, "relu", with_scratch=True)
        got = _backward(lib, torch, L.b200rl_dense_backward_static_scratch, W, x, pre, d_out, "relu", with_scratch=False)
        d_pre = want[3].astype(np.float64)
        assert np.all(np.abs(got[0] - want[0]) <= 1e-6 + 1e-5 * (np.abs(d_pre).T @ np.abs(x.astype(np.float64))))
        assert np.all(np.abs(got[1] - want[1]) <= 1e-6 + 1e-5 * np.abs(d_pre).sum(0))
        assert np.array_equal(got[2], want[2]) and np.array_equal(got[3], want[3])


def test_static_scratch_limit_is_reported_before_any_launch(lib):
    """What the static array cannot serve at all is a layer so wide that two partial sums of its weight gradient do not fit
    (input_dim * output_dim > 2^20): refused with a clear status before anything is launched; without gradients nothing is refused."""
    L = lib.lib()
    B, I, O = 4096, 2048, 1024
    one = C.c_void_p(16)                      # never dereferenced: the size check comes first
    rc = L.b200rl_dense_backward_static_scratch(one, one, I, one, O, one, O, one, one, None, 0, B, I, O, 0, None)
    assert rc == 5 and b"static buffer" in L.b200rl_status_string(5)
