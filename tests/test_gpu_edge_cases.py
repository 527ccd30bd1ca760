"""Edge cases of the C ABI on the GPU: empty inputs are accepted and touch nothing, degenerate and ragged sizes (one environment, tile
sizes plus or minus one, more environments than one wave of the persistent kernel) agree with the oracle, zero steps of collect still
write the reset column and the final observation (as the reference's loop does)."""
import ctypes as C

import numpy as np
import pytest

import make_golden as mg
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_empty_inputs_are_accepted_and_touch_nothing(lib, torch):
    L = lib.lib()
    shape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    sentinel = torch.full((64,), 5.0, device="cuda")
    p = lambda t: C.c_void_p(t.data_ptr())
    i32, u8 = torch.zeros(4, dtype=torch.int32, device="cuda"), torch.zeros(4, dtype=torch.uint8, device="cuda")
    params = torch.zeros(4482, device="cuda")
    other = torch.full((64,), 5.0, device="cuda")
    assert L.b200rl_dense_forward(p(sentinel), p(sentinel), p(sentinel), 4, None, 0, p(other), 4, 0, 4, 4, 1, None) == 0             # batch 0
    assert L.b200rl_dense_forward(p(sentinel), p(sentinel), p(sentinel), 4, None, 0, p(sentinel), 4, 0, 4, 4, 1, None) == 1          # in-place output is refused
    assert L.b200rl_pendulum_rollout(C.byref(shape), p(params), p(sentinel), p(i32), p(u8), p(sentinel), None, 0, 0, 5, 200,
                                     p(sentinel), p(sentinel), p(sentinel), None, None) == 0                                       # no environments
    assert L.b200rl_pendulum_rollout(C.byref(shape), p(params), p(sentinel), p(i32), p(u8), p(sentinel), None, 0, 4, 0, 200,
                                     p(sentinel), p(sentinel), p(sentinel), None, None) == 0                                       # no steps
    assert L.b200rl_fill(p(sentinel), 0, 1.0, None) == 0
    assert L.b200rl_mse_gradient(p(sentinel), 4, p(sentinel), 4, p(sentinel), 4, 0, 4, 1.0, None) == 0
    assert L.b200rl_permute_rows(p(sentinel), 4, 0, p(i32), 3, None, 0, None) == 0
    assert L.b200rl_gae(p(sentinel), 1, p(sentinel), 1, p(sentinel), 1, p(sentinel), 1, p(sentinel), 1, p(sentinel), 1, 0, 8, 0.99, 0.95, 0, None) == 0
    torch.cuda.synchronize()
    assert bool((sentinel == 5.0).all()) and bool((other == 5.0).all()) and int(i32.abs().sum()) == 0


@pytest.mark.parametrize("N", [1, 3, 31, 127, 129, 593, 4 * 148 * 128 + 5])
def test_rollout_ragged_environment_counts(lib, orc, torch, N):
    """One environment, one short of / one more than a tile, more than one wave of tiles: 3 steps against the oracle; the rows
    beyond N are not written."""
    shape, oshape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"]), oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    T = 3
    params = mg.det_uniform(91, oshape.num_params()) * np.float32(0.3)
    states = orc.pendulum_initial_states(6, N)
    es, tr, er = np.full(N, 198, np.int32), np.zeros(N, np.uint8), np.zeros(N, np.float32)      # truncates after 2 steps -> one reset inside the call
    table = orc.reset_table(2, N, T, es, tr, 200, 1)
    ref = orc.pendulum_rollout(oshape, params, states, es, tr, er, table, T)
    d = [dev(torch, a) for a in (states, es, tr, er)]
    obs = torch.full((T * N + 7, 3), 9.0, device="cuda")
    act, rew = torch.full((T * N + 7, 1), 9.0, device="cuda"), torch.full((T * N + 7, 1), 9.0, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.pendulum_rollout(shape, dev(torch, params), d[0], d[1], d[2], d[3], dev(torch, table), T, obs=obs, act=act, rew=rew, error_flag=flag)
    assert int(flag.item()) == 0
    got_obs, got_act = obs.cpu().numpy(), act.cpu().numpy()
    assert np.all(got_obs[T * N:] == 9.0) and np.all(got_act[T * N:] == 9.0)
    assert np.array_equal(d[1].cpu().numpy(), ref["episode_step"]) and np.array_equal(d[2].cpu().numpy(), ref["truncated"])
    assert np.array_equal(got_obs[2 * N:3 * N, 2], table[0, :, 1])                         # the reset row copies theta_dot from the table
    for got, want, atol in ((got_obs[:T * N], ref["obs"], 1e-6), (got_act[:T * N], ref["act"], 1e-6), (rew.cpu().numpy()[:T * N], ref["rew"], 1e-6)):
        assert np.all(np.abs(got - want) <= atol + 1e-5 * np.abs(want))                       # 3 free-running steps still within the first-step tolerance


def test_collect_with_zero_steps_writes_reset_column_and_final_observation(lib, orc, torch):
    N = 37
    shape, oshape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"]), oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    params = mg.det_uniform(92, 4482) * np.float32(0.3)
    runner = dict(states=orc.pendulum_initial_states(8, N), episode_step=np.arange(N, dtype=np.int32), truncated=(np.arange(N) % 2).astype(np.uint8),
                  episode_return=np.ones(N, np.float32))
    want = orc.pendulum_collect(oshape, params, {k: v.copy() for k, v in runner.items()}, 0, 50, rng=orc.new_rng(1))
    rd = {k: dev(torch, v) for k, v in runner.items()}
    pd = dev(torch, params)
    got = lib.pendulum_collect(shape, pd, pd[4481:], rd["states"], rd["episode_step"], rd["truncated"], rd["episode_return"], None, None, 0, 50).cpu().numpy()
    assert got.shape == (N, 13)
    assert np.array_equal(got[:, 9], want[:, 9]) and np.all(np.abs(got[:, 0:3] - want[:, 0:3]) <= 2e-6)
    for k in runner:                                                                       # the runner state is unchanged
        assert np.array_equal(rd[k].cpu().numpy(), runner[k]), k
