"""GPU parity of the dense layer, MSE gradient and Adam (through the C ABI) against the CPU oracle and the golden
fixtures of the real reference. Tolerance: |x - ref| <= 1e-6 + 1e-5 |ref| per element (fp32 path)."""
import glob
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu
RTOL, ATOL = 1e-5, 1e-6


def close(got, want, rtol=RTOL, atol=ATOL):
    got = got.detach().cpu().numpy() if hasattr(got, "detach") else np.asarray(got)
    err = np.abs(got.reshape(-1).astype(np.float64) - want.reshape(-1).astype(np.float64))
    bound = atol + rtol * np.abs(want.reshape(-1).astype(np.float64))
    worst = int(np.argmax(err - bound))
    assert np.all(err <= bound), f"max excess at {worst}: got {got.reshape(-1)[worst]} want {want.reshape(-1)[worst]} err {err[worst]:.3e}"


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


SHAPES = [  # (batch, in, out, act): the reference's CUDA test sweep plus awkward sizes
    (1, 3, 64, "relu"), (256, 3, 64, "relu"), (256, 64, 2, "identity"), (2, 256, 10, "relu"), (9, 256, 60, "tanh"), (10, 200, 100, "relu"),
    (32, 10, 100, "sigmoid"), (200, 11, 256, "fast_tanh"), (1024, 256, 10, "relu"), (64, 50, 101, "tanh"), (256, 256, 256, "relu"),
    (2048, 27, 64, "tanh"), (300, 64, 8, "identity"), (4099, 65, 17, "relu"), (256, 4, 256, "relu"), (256, 256, 1, "identity"),
    # >= 2^27 multiply-adds: these take the tensor-core kernel (ragged rows, ragged k, narrow and non-multiple-of-8 columns)
    (4099, 256, 200, "relu"), (8192, 130, 257, "tanh"), (70001, 64, 40, "relu"), (16384, 256, 256, "relu"),
    # few outputs at a large batch: the backward pass takes the one-pass kernel (ragged rows, one and two columns per thread, every output count class)
    (8192, 256, 16, "identity"), (10007, 200, 5, "tanh"), (9001, 100, 1, "relu"), (33000, 256, 16, "sigmoid"),
]


@pytest.mark.parametrize("B,I,O,act", SHAPES)
def test_dense_forward_backward_vs_oracle(lib, orc, torch, B, I, O, act):
    seed = B * 7 + I * 3 + O
    W = (mg.det_uniform(seed, O * I, stream=1) / np.float32(np.sqrt(I))).reshape(O, I)
    b = mg.det_uniform(seed, O, stream=2) / np.float32(np.sqrt(I))
    x = mg.det_normal(seed, B * I, stream=3).reshape(B, I)
    d_out = mg.det_normal(seed, B * O, stream=4).reshape(B, O)
    pre_ref, y_ref = orc.dense_forward(W, b, x, act)
    pre, y = lib.dense_forward(dev(torch, W), dev(torch, b), dev(torch, x), act)
    close(pre, pre_ref)
    close(y, y_ref)
    if lib.lib().b200rl_dense_forward_workspace_bytes(B, I, O) > 0:       # tensor-core shapes: the workspace form (weights split once) gives the same bits
        pre_ws, y_ws = lib.dense_forward(dev(torch, W), dev(torch, b), dev(torch, x), act, workspace=True)
        assert torch.equal(pre_ws, pre) and torch.equal(y_ws, y)
    dW0 = mg.det_normal(seed, O * I, stream=5).reshape(O, I)   # gradients accumulate on top of existing values
    db0 = mg.det_normal(seed, O, stream=6)
    dW_ref, db_ref, din_ref, dpre_ref = orc.dense_backward(W, x, pre_ref, d_out, act, dW=dW0, db=db0)
    d_out_dev = dev(torch, d_out)
    dW, db, d_in = lib.dense_backward(dev(torch, W), dev(torch, x), dev(torch, pre_ref), d_out_dev, act, dW=dev(torch, dW0), db=dev(torch, db0))
    close(d_out_dev, dpre_ref)                                  # d_out is overwritten with d_pre, as in the reference
    # sums over the batch: tolerance scales with the number of summed terms' magnitude
    scale_w = np.abs(dpre_ref).T @ np.abs(x) + np.abs(dW0)
    assert np.all(np.abs(dW.cpu().numpy() - dW_ref) <= ATOL + RTOL * scale_w)
    scale_b = np.abs(dpre_ref).sum(0) + np.abs(db0)
    assert np.all(np.abs(db.cpu().numpy() - db_ref) <= ATOL + RTOL * scale_b)
    scale_i = np.abs(dpre_ref) @ np.abs(W)
    assert np.all(np.abs(d_in.cpu().numpy() - din_ref) <= ATOL + RTOL * scale_i)


def test_dense_forward_row_pitch_views(lib, orc, torch):
    """Inputs/outputs that are column views of a wider table (dataset rows are 13 floats wide in the on-policy runner)."""
    B, I, O = 77, 3, 5
    table = mg.det_normal(1, B * 13).reshape(B, 13)
    W = mg.det_uniform(2, O * I).reshape(O, I)
    b = mg.det_uniform(3, O)
    t = dev(torch, table)
    x_view = t[:, 2:5]
    out_table = torch.zeros((B, 11), device="cuda")
    y_view = out_table[:, 4:9]
    lib.dense_forward(dev(torch, W), dev(torch, b), x_view, "tanh", want_pre=False, y=y_view)
    _, y_ref = orc.dense_forward(W, b, np.ascontiguousarray(table[:, 2:5]), "tanh", want_pre=False)
    close(y_view, y_ref)
    assert float(out_table[:, :4].abs().max()) == 0.0 and float(out_table[:, 9:].abs().max()) == 0.0


def test_backward_input_only(lib, orc, torch):
    B, I, O = 130, 20, 33
    W = mg.det_uniform(5, O * I).reshape(O, I)
    x = mg.det_normal(5, B * I, stream=1).reshape(B, I)
    pre = mg.det_normal(5, B * O, stream=2).reshape(B, O)
    d_out = mg.det_normal(5, B * O, stream=3).reshape(B, O)
    _, _, din_ref, _ = orc.dense_backward(W, x, pre, d_out, "relu", want_grads=False)
    _, _, d_in = lib.dense_backward(dev(torch, W), dev(torch, x), dev(torch, pre), dev(torch, d_out), "relu", want_grads=False)
    close(d_in, din_ref)


def test_backward_input_only_few_outputs_large_batch(lib, orc, torch):
    """backward_input of a last layer (few outputs, large batch: the one-pass kernel without its gradient half)."""
    B, I, O = 9003, 256, 4
    W = mg.det_uniform(6, O * I).reshape(O, I)
    x = mg.det_normal(6, B * I, stream=1).reshape(B, I)
    pre = mg.det_normal(6, B * O, stream=2).reshape(B, O)
    d_out = mg.det_normal(6, B * O, stream=3).reshape(B, O)
    _, _, din_ref, dpre_ref = orc.dense_backward(W, x, pre, d_out, "tanh", want_grads=False)
    d_out_dev = dev(torch, d_out)
    _, _, d_in = lib.dense_backward(dev(torch, W), dev(torch, x), dev(torch, pre), d_out_dev, "tanh", want_grads=False)
    close(d_in, din_ref)
    close(d_out_dev, dpre_ref)


def test_mse_gradient(lib, orc, torch):
    a = mg.det_normal(9, 256 * 3).reshape(256, 3)
    b = mg.det_normal(9, 256 * 3, stream=1).reshape(256, 3)
    got = lib.mse_gradient(dev(torch, a), dev(torch, b), 0.5)
    assert np.array_equal(got.cpu().numpy(), orc.mse_gradient(a, b, 0.5))      # element-wise: bit-exact


@pytest.mark.parametrize("n", [1, 5, 1023, 67329, 152336])
def test_adam_step_bit_exact_over_several_steps(lib, orc, torch, n):
    p = mg.det_normal(n, n)
    m = np.zeros(n, np.float32)
    v = np.zeros(n, np.float32)
    dp, dm, dv = dev(torch, p), dev(torch, m), dev(torch, v)
    state = torch.zeros(4, dtype=torch.int32, device="cuda")
    import ctypes as C
    L = lib.lib()
    lib.check(L.b200rl_adam_reset(C.c_void_p(state.data_ptr()), None))
    age = 1
    hyper = lib.AdamHyper()
    for step in range(5):
        g = mg.det_normal(n + step, n, stream=7) * np.float32(0.1 if step % 2 else 3.0)
        c1, c2, age = orc.adam_bias_correction(0.9, 0.999, age)
        p, m, v = orc.adam_update(p, g, m, v, 1e-3, 0.9, 0.999, 1e-7, 1e-7, c1, c2)
        dg = dev(torch, g)
        lib.check(L.b200rl_adam_step(C.c_void_p(dp.data_ptr()), C.c_void_p(dg.data_ptr()), C.c_void_p(dm.data_ptr()), C.c_void_p(dv.data_ptr()), n, hyper,
                                     C.c_void_p(state.data_ptr()), None))
        torch.cuda.synchronize()
        st = state.cpu().numpy()
        assert int(st[0]) == age and int(st[1]) == 0                      # integer optimizer state: exact
        assert np.array_equal(dm.cpu().numpy(), m) and np.array_equal(dv.cpu().numpy(), v)
        close(dp, p, rtol=1e-6, atol=1e-7)
    assert np.array_equal(dp.cpu().numpy(), p), "Adam update differs in the last bit from the reference rounding sequence"


MLP_FIXTURES = sorted(glob.glob(os.path.join(GOLDEN, "mlp_*.npz")))


@pytest.mark.parametrize("path", MLP_FIXTURES, ids=[os.path.basename(p)[4:-4] for p in MLP_FIXTURES])
def test_mlp_train_steps_vs_reference_golden(lib, torch, path):
    """evaluate / forward / backward / Adam through the flat-arena MLP against the REAL reference's outputs."""
    fix = np.load(path)
    name = os.path.basename(path)[4:-4]
    d = fix["dims"]
    c = dict(batch=int(d[0]), input_dim=int(d[1]), hidden_dim=int(d[2]), output_dim=int(d[3]), num_layers=int(d[4]), hidden_act=int(d[5]), output_act=int(d[6]))
    dims = [c["hidden_dim"]] * (c["num_layers"] - 1) + [c["output_dim"]]
    acts = [c["hidden_act"]] * (c["num_layers"] - 1) + [c["output_act"]]
    params, x, target = mg.mlp_inputs(c, mg.case_seed(name))
    net = lib.Mlp(c["input_dim"], dims, acts, c["batch"])
    net.params.copy_(dev(torch, params))
    xd, td = dev(torch, x), dev(torch, target)

    def check(key, t, rtol=RTOL, atol=ATOL, tensor_scale=0.0):
        # tensor_scale > 0 adds tensor_scale * max|reference| to the absolute tolerance: sums over the batch are
        # compared relative to the scale of the tensor (their summation order differs from the reference's)
        s, _ = mg.sample(t.detach().cpu().numpy())
        close(s, fix[key], rtol, atol + tensor_scale * float(np.abs(fix[key]).max()))

    check("eval_out", net.evaluate(xd))
    net.zero_gradient()
    y = net.forward(xd)
    check("fwd_pre", net.pre)
    check("fwd_out", net.out)
    d_out = lib.mse_gradient(y, td, 1.0)
    net.backward(xd, d_out)
    # gradient sums run over batch x fan-in products: allow a few extra ulps of the largest term
    check("bwd_grads", net.grads, tensor_scale=1e-5)
    net.zero_gradient()
    net.reset_optimizer_state()
    for _ in range(mg.MLP_STEPS):
        net.zero_gradient()
        y = net.forward(xd)
        d_out = lib.mse_gradient(y, td, 1.0)
        net.backward(xd, d_out)
        net.step()
    check("train_m", net.m, tensor_scale=1e-5)
    # Adam normalises the step to ~alpha regardless of gradient scale, so parameter error is bounded by alpha * relative gradient error
    check("train_params", net.params)
    # full backward with d_input, from the initial parameters again
    net.params.copy_(dev(torch, params))
    net.zero_gradient()
    net.forward(xd)
    d_in = torch.empty((c["batch"], c["input_dim"]), device="cuda")
    net.backward(xd, td.clone(), d_input=d_in)
    check("full_grads", net.grads, tensor_scale=1e-5)
    check("full_d_input", d_in, tensor_scale=1e-5)


def test_sharded_train_step_matches_oracle_full_batch(lib, orc, torch):
    """Two chunks accumulated with the chunk loss weight + one Adam step == the oracle's full-batch step (world size 1)."""
    from rl_tools_b200 import parallel
    dims, acts = [32, 32, 4], ["relu", "relu", "identity"]
    shape = oracle.MlpShape.make(8, dims, acts)
    total, chunk = 512, 256
    params = mg.det_uniform(41, shape.num_params()) * np.float32(0.3)
    x = mg.det_normal(42, total * 8).reshape(total, 8)
    y = mg.det_normal(43, total * 4).reshape(total, 4)
    net = lib.Mlp(8, dims, acts, chunk)
    net.params.copy_(dev(torch, params))
    parallel.sharded_train_step(lib, net, dev(torch, x), dev(torch, y), total)
    p_ref, g_ref, m_ref, v_ref, _, _ = orc.mlp_train_steps(shape, params, x, y, 1)
    scale = float(np.abs(g_ref).max())
    close(net.grads, g_ref)
    close(net.params, p_ref)


@pytest.mark.parametrize("hidden_act,out_dim", [("tanh", 8), ("sigmoid", 40)])
def test_mlp_backward_large_batch_against_the_oracle(lib, orc, torch, hidden_act, out_dim):
    """The whole backward pass at a large batch -- the tensor-core products for the wide layers, the one-pass kernel for an output layer of
    <= 16 units (out_dim 8) or the tiled path for a wider one (out_dim 40) -- against the oracle's per-layer recursion: parameter gradients on
    top of existing values and the input gradient, for activations whose derivative is not 0 / 1, ragged rows and a ragged width; also the
    input-gradient-only pass (no parameter gradients)."""
    B, I, dims = 9001, 40, [256, 200, out_dim]
    acts = [hidden_act, hidden_act, "identity"]
    shape = oracle.MlpShape.make(I, dims, acts)
    params = mg.det_uniform(77, shape.num_params()) * np.float32(0.08)
    x = mg.det_normal(78, B * I).reshape(B, I)
    d_out = mg.det_normal(79, B * out_dim).reshape(B, out_dim) / np.float32(B)
    g0 = mg.det_normal(80, shape.num_params()) * np.float32(0.01)
    pre, out = orc.mlp_forward(shape, params, x)
    g_ref, din_ref = orc.mlp_backward(shape, params, g0, x, pre, out, d_out, want_d_input=True)
    net = lib.Mlp(I, dims, acts, B)
    net.params.copy_(dev(torch, params)); net.grads.copy_(dev(torch, g0))
    xd = dev(torch, x)
    net.forward(xd)
    close(net.pre, pre); close(net.out, out)
    d_in = torch.empty((B, I), device="cuda")
    net.backward(xd, dev(torch, d_out), d_input=d_in)
    # sums of B products of magnitude ~|d_out| * |activation|: the tolerance scales with the summed magnitudes (here <= ~1e-3 per entry)
    g = net.grads.cpu().numpy()
    assert np.all(np.abs(g - g_ref) <= 1e-6 + 1e-5 * np.maximum(np.abs(g_ref), 1e-2)), float(np.abs(g - g_ref).max())
    close(d_in, din_ref, rtol=1e-5, atol=1e-8)
    d_in_only = torch.empty((B, I), device="cuda")
    net.grads.fill_(0.25)
    net.backward(xd, dev(torch, d_out), d_input=d_in_only, accumulate_gradients=False)
    assert bool((net.grads == 0.25).all()) and torch.equal(d_in_only, d_in)


@pytest.mark.gpu
@pytest.mark.parametrize("B,I,dims,acts", [
    (256, 4, [256, 256, 1], ["relu", "relu", "identity"]),          # the critic of the off-policy algorithms
    (256, 3, [256, 256, 2], ["relu", "relu", "tanh"]),              # their actor: an odd input width, an activation on the output
    (200, 17, [300, 270, 133, 5], ["tanh", "sigmoid", "relu", "identity"]),   # four layers, nothing a multiple of the tile
    (512, 300, [512, 260], ["fast_tanh", "identity"]),              # two chunks of the summed index, the largest batch and width
])
def test_mlp_backward_in_one_cooperative_launch(lib, orc, torch, B, I, dims, acts):
    """Wide networks at small batches take the backward pass as one cooperative launch (phases with grid-wide barriers): parameter
    gradients on top of existing values and the input gradient against the oracle's per-layer recursion; the input-gradient-only pass;
    two passes in a row give the same bits (the partial tiles are added in a fixed order); no barrier wait ran into its limit."""
    import ctypes
    shape = oracle.MlpShape.make(I, dims, acts)
    params = mg.det_uniform(91, shape.num_params()) * np.float32(0.1)
    x = mg.det_normal(92, B * I).reshape(B, I)
    d_out = mg.det_normal(93, B * dims[-1]).reshape(B, dims[-1]) / np.float32(B)
    g0 = mg.det_normal(94, shape.num_params()) * np.float32(0.01)
    pre, out = orc.mlp_forward(shape, params, x)
    g_ref, din_ref = orc.mlp_backward(shape, params, g0, x, pre, out, d_out, want_d_input=True)
    net = lib.Mlp(I, dims, acts, B)
    net.params.copy_(dev(torch, params))
    xd = dev(torch, x)
    net.forward(xd)
    results = []
    for _ in range(2):
        net.grads.copy_(dev(torch, g0))
        d_in = torch.empty((B, I), device="cuda")
        net.backward(xd, dev(torch, d_out), d_input=d_in)
        results.append((net.grads.clone(), d_in))
    g = results[0][0].cpu().numpy()
    assert np.all(np.abs(g - g_ref) <= 1e-6 + 1e-5 * np.maximum(np.abs(g_ref), 1e-2)), float(np.abs(g - g_ref).max())
    close(results[0][1], din_ref, rtol=1e-5, atol=1e-8)
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])
    d_in_only = torch.empty((B, I), device="cuda")
    net.grads.fill_(0.25)
    net.backward(xd, dev(torch, d_out), d_input=d_in_only, accumulate_gradients=False)
    assert bool((net.grads == 0.25).all()) and torch.equal(d_in_only, results[0][1])
    status = ctypes.c_int(-1)
    L = lib.lib()
    L.b200rl_cooperative_pass_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    assert L.b200rl_cooperative_pass_status(ctypes.byref(status)) == 0 and status.value == 0


def test_mlp_backward_without_parameter_gradients(lib, torch):
    """grads = NULL is the reference's backward_input: the same input gradient as the full backward pass, parameter gradients untouched."""
    rs = np.random.RandomState(3)
    B = 256
    net = lib.Mlp(4, [64, 64, 1], ["relu", "relu", "identity"], B)
    net.params.copy_(torch.from_numpy((rs.uniform(-1, 1, net.params.numel()) * 0.3).astype(np.float32)).cuda())
    x = torch.from_numpy(rs.randn(B, 4).astype(np.float32)).cuda()
    d_out = torch.from_numpy(rs.randn(B, 1).astype(np.float32)).cuda()
    net.forward(x)
    net.grads.fill_(0.5)
    d_in_a, d_in_b = torch.empty((B, 4), device="cuda"), torch.empty((B, 4), device="cuda")
    net.backward(x, d_out.clone(), d_input=d_in_a, accumulate_gradients=False)
    assert bool((net.grads == 0.5).all())
    net.backward(x, d_out.clone(), d_input=d_in_b)
    assert torch.equal(d_in_a, d_in_b) and not bool((net.grads == 0.5).all())


def test_init_weights_reproduces_the_reference_engine(lib, torch):
    """b200rl_dense_init_weights, layer after layer on one host engine, against the actor the reference's own init_weights produced from
    seed 0 (3 -> 64 -> 64 -> 1, legacy Kaiming-uniform; stored in rollout.npz): bias, then the row's weights, per output row -- bit-exact."""
    want = np.load(os.path.join(GOLDEN, "rollout.npz"))["actor_params"]
    rng = lib.rng_init_host(0)
    parts, fan_in = [], 3
    for d in (64, 64, 1):
        W, b = torch.empty((d, fan_in), device="cuda"), torch.empty(d, device="cuda")
        lib.dense_init_weights(rng, W, b)
        parts += [W.cpu().numpy().reshape(-1), b.cpu().numpy()]
        fan_in = d
    assert np.array_equal(np.concatenate(parts), want)


def test_randn_host_engine_and_mse_evaluate(lib, orc, torch):
    """Normals of the host engine in the reference's order (row-major, a fresh distribution per element) into a pitched device matrix, and the
    loss value against the oracle's sequential float sum: the double sum rounded once lies within that sum's rounding error, bounded here by
    rows * cols * 2^-24 relative."""
    rows, cols = 37, 5
    table = torch.zeros((rows, 9), device="cuda")
    lib.randn_host_rng(lib.rng_init_host(5), table[:, 2:7])
    assert np.array_equal(table[:, 2:7].cpu().numpy().reshape(-1), orc.normal_stream(5, rows * cols, 0.0, 1.0))
    assert float(table[:, :2].abs().sum()) == 0 and float(table[:, 7:].abs().sum()) == 0
    for B, O, w in ((256, 1, 1.0), (2048, 8, 0.5), (1, 3, 2.0), (4099, 17, 1.0)):
        a, b = mg.det_normal(B + O, B * O, stream=1).reshape(B, O), mg.det_normal(B + O, B * O, stream=2).reshape(B, O)
        got, want = lib.mse_evaluate(dev(torch, a), dev(torch, b), w), orc.mse_evaluate(a, b, w)
        assert abs(got - want) <= max(B * O * 2.0 ** -24, 1e-6) * abs(want), (B, O, got, want)


@pytest.mark.gpu
def test_device_operand_tensor_ops_of_the_sac_update(lib, torch):
    """The small operations between the network passes of train_critic / train_actor with their operands in device memory, each against the same
    float32 arithmetic in numpy: bit-exact (one multiply, one divide or a copy per element)."""
    f = np.float32
    rng = np.random.default_rng(11)
    for rows, cols in ((256, 1), (97, 3), (1, 1)):
        a, b = rng.standard_normal((rows, cols)).astype(f), rng.standard_normal((rows, cols)).astype(f)
        mask = (rng.random(rows) < 0.4)
        if rows > 1:
            mask[0], mask[1] = True, False
        mask_d = dev(torch, mask.astype(np.uint8))
        weight = torch.zeros(1, device="cuda")
        lib.mask_count(mask_d, weight)
        assert weight.item() == mask.sum()
        if mask.sum() == 0:
            continue
        lib.scale_(weight, f(rows * 0.5), reciprocal=True)                                   # the loss weight of train_critic
        w_ref = f(1) / f(mask.sum()) * f(rows * 0.5)
        assert weight.item() == w_ref
        # gradient with that device-resident weight, into a pitched view
        table = torch.full((rows, cols + 2), 7.0, device="cuda")
        lib.mse_gradient_dev_weight(dev(torch, a), dev(torch, b), weight, table[:, 1:1 + cols])
        constant = f(2) / (f(rows) * f(cols)) * w_ref
        assert np.array_equal(table[:, 1:1 + cols].cpu().numpy(), (a - b) * constant)
        assert float((table[:, 0] - 7).abs().sum()) == 0 and float((table[:, -1] - 7).abs().sum()) == 0
        # set_all from a device scalar, plain scaling
        buf = torch.empty(rows * cols, device="cuda")
        lib.fill_from_device(buf, weight)
        assert np.all(buf.cpu().numpy() == w_ref)
        lib.scale_(buf, f(-3.0))
        assert np.all(buf.cpu().numpy() == w_ref * f(-3.0))
        # masked rows: copy of the source where the (inverted) mask is set, zeros without a source
        for invert in (False, True):
            take = mask != invert
            target = dev(torch, b.copy())
            lib.mask_rows(target, mask_d, source=dev(torch, a), invert=invert)
            assert np.array_equal(target.cpu().numpy(), np.where(take[:, None], a, b))
            target = dev(torch, b.copy())
            lib.mask_rows(target, mask_d, invert=invert)
            assert np.array_equal(target.cpu().numpy(), np.where(take[:, None], f(0), b))


@pytest.mark.gpu
def test_network_trained_on_the_device_exports_in_the_reference_code_format(lib, torch):
    """Mlp.save_code: the parameters as they are on the device, in the text the reference's own writer produces for them (the writer itself
    is held byte for byte against the reference in tests/test_export.py)."""
    from rl_tools_b200 import export
    net = lib.Mlp(3, [64, 64, 1], ["relu", "relu", "tanh"], 32)
    g = torch.Generator(device="cuda"); g.manual_seed(3)
    net.params.copy_(torch.randn(net.params.numel(), device="cuda", generator=g) * 0.2)
    x, y = torch.randn((32, 3), device="cuda", generator=g), torch.randn((32, 1), device="cuda", generator=g)
    for _ in range(2):
        net.zero_gradient()
        net.backward(x, lib.mse_gradient(net.forward(x), y, 1.0))
        net.step()
    code = net.save_code("rl_tools::checkpoint::actor")
    params = net.params.cpu().numpy()
    assert code == export.save_code(params, 3, [64, 64, 1], ["relu", "relu", "tanh"], "rl_tools::checkpoint::actor", 1)
    assert export.hexfloat(params[0]) in code and export.hexfloat(params[-1]) in code and "namespace rl_tools::checkpoint::actor {" in code
