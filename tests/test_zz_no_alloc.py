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


def test_static_scratch_limit_is_reported_before_any_launch(lib):
    L = lib.lib()
    B, I, O = 1 << 20, 1024, 1024            # split-batch partials would need far more than 8 MiB
    assert L.b200rl_dense_backward_scratch_bytes(B, I, O) > 8 * 1024 * 1024
    one = C.c_void_p(16)                      # never dereferenced: the size check comes first
    rc = L.b200rl_dense_backward_static_scratch(one, one, I, one, O, one, O, one, one, None, 0, B, I, O, 0, None)
    assert rc == 5 and b"static buffer" in L.b200rl_status_string(5)
