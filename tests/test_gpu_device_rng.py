"""Device-side random numbers of the fused rollout / collect kernels (through the C ABI).

The reference's device engines (random/operations_cuda.h) are per-thread cuRAND states, so there is no bit-level oracle for a device
stream. What is checked instead: the draws equal an independent numpy statement of Philox-4x32-10 + Box-Muller on the documented counter
layout (within fp32 rounding of the transcendental functions); they do not depend on how the environments or the steps are split over
launches; the arithmetic downstream of the draws is the table-driven kernel's (exact in the noise-to-action step, within recovery rounding
elsewhere, when the draws are fed back as host tables); and the moments are those of N(0, 1) and of the Pendulum initial-state distribution."""
import numpy as np
import pytest

import oracle

pytestmark = pytest.mark.gpu

OBS, MEAN, ACTION, LOGP, REWARD, TERMINATED, TRUNCATED, RESET = slice(0, 3), 3, 4, 5, 6, 7, 8, 9
M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """counter uint32[..., 4], key (k0, k1): Salmon et al., SC'11, ten rounds."""
    c = [counter[..., i].astype(np.uint64) for i in range(4)]
    k0, k1 = np.uint64(key[0]), np.uint64(key[1])
    mask = np.uint64(0xFFFFFFFF)
    for _ in range(10):
        p0, p1 = np.uint64(M0) * c[0], np.uint64(M1) * c[2]
        c = [(p1 >> np.uint64(32)) ^ c[1] ^ k0, p1 & mask, (p0 >> np.uint64(32)) ^ c[3] ^ k1, p0 & mask]
        k0, k1 = (k0 + np.uint64(W0)) & mask, (k1 + np.uint64(W1)) & mask
    return np.stack(c, axis=-1).astype(np.uint32)


def expected_draws(seed, first_step, T, N, env_begin=0):
    """(normal [T, N], theta [T, N], theta_dot [T, N]) in float64 from the documented counter layout."""
    steps = first_step + np.arange(T, dtype=np.uint64)[:, None] + np.zeros((1, N), np.uint64)
    envs = (env_begin + np.arange(N, dtype=np.uint64))[None, :] + np.zeros((T, 1), np.uint64)
    counter = np.stack([envs, steps & np.uint64(0xFFFFFFFF), steps >> np.uint64(32), np.zeros_like(envs)], axis=-1).astype(np.uint32)
    words = philox4x32_10(counter, (seed & 0xFFFFFFFF, seed >> 32))
    u = ((words >> np.uint32(9)).astype(np.float64) + 0.5) * 2.0 ** -23
    normal = np.sqrt(-2.0 * np.log(u[..., 0])) * np.cos(2.0 * np.pi * u[..., 1])
    return normal, u[..., 2] * 2 * np.pi - np.pi, u[..., 3] * 2 - 1


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def make_actor(lib, hact=1, log_std=-0.3, seed=5):
    rs = np.random.RandomState(seed)
    params = np.concatenate([rs.uniform(-0.5, 0.5, 64 * 3 + 64), rs.uniform(-0.2, 0.2, 64 * 64 + 64), rs.uniform(-0.2, 0.2, 64 + 1),
                             [log_std]]).astype(np.float32)
    return lib.MlpShape.make(3, [64, 64, 1], [hact, hact, 0]), params


def fresh(torch, N):
    return dict(states=torch.zeros((N, 2), device="cuda"), episode_step=torch.zeros(N, dtype=torch.int32, device="cuda"),
                truncated=torch.ones(N, dtype=torch.uint8, device="cuda"), episode_return=torch.zeros(N, device="cuda"))


def collect(lib, torch, shape, params_d, runner, seed, first_step, T, limit):
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    ds = lib.pendulum_collect_device_rng(shape, params_d, params_d[4481:], runner["states"], runner["episode_step"], runner["truncated"],
                                         runner["episode_return"], seed, first_step, T, limit, error_flag=flag)
    assert int(flag.item()) == 0
    return ds.cpu().numpy()


@pytest.mark.parametrize("N,T,limit,seed,first", [(300, 23, 7, 0x1234_5678_9ABC_DEF0, 0), (4099, 12, 5, 3, (1 << 32) - 4), (128, 64, 0, 77, 1000)])
def test_draws_match_numpy_philox(lib, torch, N, T, limit, seed, first):
    shape, params = make_actor(lib)
    params_d = dev(torch, params)
    runner = fresh(torch, N)
    got = collect(lib, torch, shape, params_d, runner, seed, first, T, limit).reshape(T + 1, N, 13)[:T]
    normal, theta, theta_dot = expected_draws(seed, first, T, N)
    std = np.float32(np.exp(np.float64(params[-1])))
    eps = (got[..., ACTION].astype(np.float64) - got[..., MEAN]) / std
    assert np.abs(eps - normal).max() < 4e-6 * (1 + np.abs(normal).max())
    # every row flagged as reset starts from the drawn initial state
    reset = got[..., RESET] != 0
    assert reset[0].all() and (limit == 0 or reset.sum() > N)
    assert np.abs(got[..., 0][reset] - np.cos(theta[reset])).max() < 2e-6
    assert np.abs(got[..., 1][reset] - np.sin(theta[reset])).max() < 2e-6
    assert np.abs(got[..., 2][reset] - theta_dot[reset]).max() < 2e-6


def test_independent_of_sharding_and_call_split(lib, torch):
    """The same (seed, environment, step) gives the same draw whether the steps come from one call or two; a runner over the first
    environments alone reproduces their rows of the larger launch bit for bit."""
    N, T, limit, seed = 1000, 30, 11, 99
    shape, params = make_actor(lib, hact=2)
    params_d = dev(torch, params)
    whole = collect(lib, torch, shape, params_d, fresh(torch, N), seed, 0, T, limit).reshape(T + 1, N, 13)
    runner = fresh(torch, N)
    first = collect(lib, torch, shape, params_d, runner, seed, 0, 13, limit).reshape(14, N, 13)
    second = collect(lib, torch, shape, params_d, runner, seed, 13, T - 13, limit).reshape(T - 13 + 1, N, 13)
    assert np.array_equal(first[:13, :, :10], whole[:13, :, :10])
    assert np.array_equal(second[:, :, :3], whole[13:, :, :3]) and np.array_equal(second[:-1, :, 3:10], whole[13:T, :, 3:10])
    part = collect(lib, torch, shape, params_d, fresh(torch, 384), seed, 0, T, limit).reshape(T + 1, 384, 13)
    assert np.array_equal(part[:, :, :3], whole[:, :384, :3]) and np.array_equal(part[:T, :, 3:10], whole[:T, :384, 3:10])
    other = collect(lib, torch, shape, params_d, fresh(torch, N), seed + 1, 0, T, limit).reshape(T + 1, N, 13)
    assert not np.array_equal(other[:T, :, ACTION], whole[:T, :, ACTION])


def test_same_arithmetic_as_table_driven_collect(lib, torch):
    """Feeding the device path's own draws back through host tables reproduces the dataset: flags exact, the noise-to-action arithmetic
    exact, trajectories within the rounding of recovering theta from its observation. Only the source of the random numbers differs
    between the two entry points."""
    N, T, limit, seed = 777, 20, 6, 2024
    shape, params = make_actor(lib)
    params_d = dev(torch, params)
    got = collect(lib, torch, shape, params_d, fresh(torch, N), seed, 0, T, limit).reshape(T + 1, N, 13)
    # recover the draws in fp32 exactly as the kernel formed them is not possible from the outputs (rounded), so take them from a
    # probe collect with a zero-weight actor and log_std = 0: mean = 0, action = noise exactly; and from step-0 style resets
    probe_params = np.zeros_like(params)
    probe = collect(lib, torch, shape, dev(torch, probe_params), fresh(torch, N), seed, 0, T, limit).reshape(T + 1, N, 13)
    noise = probe[:T, :, ACTION].copy()
    assert np.all(probe[:T, :, MEAN] == 0)
    # reset states: run a 1-step-limit probe so that every step is a reset, then read theta / theta_dot back from the observation
    rp = collect(lib, torch, shape, dev(torch, probe_params), fresh(torch, N), seed, 0, T, 1).reshape(T + 1, N, 13)
    theta = np.arctan2(rp[:T, :, 1].astype(np.float64), rp[:T, :, 0].astype(np.float64)).astype(np.float32)
    theta_dot = rp[:T, :, 2]
    # rounds of the table in the order the environments consume them
    reset = got[:T, :, RESET] != 0
    rounds = int(reset.sum(axis=0).max())
    table = np.zeros((rounds, N, 2), np.float32)
    for e in range(N):
        steps = np.nonzero(reset[:, e])[0]
        table[:len(steps), e, 0] = theta[steps, e]
        table[:len(steps), e, 1] = theta_dot[steps, e]
    runner = fresh(torch, N)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    want = lib.pendulum_collect(shape, params_d, params_d[4481:], runner["states"], runner["episode_step"], runner["truncated"],
                                runner["episode_return"], dev(torch, table), dev(torch, noise), T, limit, error_flag=flag).cpu().numpy()
    want = want.reshape(T + 1, N, 13)
    assert int(flag.item()) == 0
    # flags, noise-to-action arithmetic: exact; observation columns: theta went through atan2 once, so within rounding
    assert np.array_equal(got[:T, :, 7:10], want[:T, :, 7:10])
    std = np.float32(np.exp(np.float64(params[-1])))
    assert np.array_equal(got[:T, :, ACTION], noise * std + got[:T, :, MEAN])
    assert np.abs(got[..., :3] - want[..., :3]).max() < 1e-5
    assert np.abs(got[:T, :, 3:7] - want[:T, :, 3:7]).max() < 4e-4


def test_moments(lib, torch):
    N, T, seed = 65536, 32, 12345
    shape, params = make_actor(lib)
    probe = dev(torch, np.zeros_like(params))
    ds = collect(lib, torch, shape, probe, fresh(torch, N), seed, 0, T, 1).reshape(T + 1, N, 13)[:T]
    eps = ds[..., ACTION].astype(np.float64).ravel()
    n = eps.size
    assert abs(eps.mean()) < 5 / np.sqrt(n) and abs(eps.var() - 1) < 5 * np.sqrt(2 / n)
    assert abs((eps ** 3).mean()) < 5 * np.sqrt(15 / n) and abs((eps ** 4).mean() - 3) < 5 * np.sqrt(96 / n)
    assert np.abs(eps).max() < 6.5 and np.abs(eps).max() > 4.0
    # lag-1 correlation across steps and across neighbouring environments
    e2 = ds[..., ACTION].astype(np.float64)
    assert abs((e2[1:] * e2[:-1]).mean()) < 5 / np.sqrt(n) and abs((e2[:, 1:] * e2[:, :-1]).mean()) < 5 / np.sqrt(n)
    theta = np.arctan2(ds[..., 1].astype(np.float64), ds[..., 0].astype(np.float64)).ravel()
    theta_dot = ds[..., 2].astype(np.float64).ravel()
    assert abs(theta.mean()) < 5 * np.pi / np.sqrt(3 * n) and abs(theta.var() - np.pi ** 2 / 3) < 0.01
    assert abs(theta_dot.mean()) < 5 / np.sqrt(3 * n) and abs(theta_dot.var() - 1 / 3) < 0.002
    assert theta_dot.min() > -1 and theta_dot.max() < 1 and np.abs(theta).max() <= np.pi
    assert abs(np.corrcoef(theta, theta_dot)[0, 1]) < 5 / np.sqrt(n) and abs(np.corrcoef(theta, eps)[0, 1]) < 5 / np.sqrt(n)


def test_rollout_device_rng(lib, torch):
    """The off-policy rollout with device resets: reset rows carry the drawn initial states, everything else is the table-driven kernel's
    arithmetic (checked against the oracle by handing it the drawn states as its reset table)."""
    N, T, limit, seed = 515, 40, 9, 4242
    shape, params = make_actor(lib)
    oshape = oracle.MlpShape.make(3, [64, 64, 1], [1, 1, 0])
    params_d = dev(torch, params[:4481])
    runner = fresh(torch, N)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.pendulum_rollout_device_rng(shape, params_d, runner["states"], runner["episode_step"], runner["truncated"],
                                                    runner["episode_return"], seed, 5, T, limit, error_flag=flag)
    assert int(flag.item()) == 0
    obs = obs.cpu().numpy().reshape(T, N, 3)
    _, theta, theta_dot = expected_draws(seed, 5, T, N)
    # episode_step counts 1..limit, the reset happens on the step after it reached the limit: steps 0, limit, 2 limit, ...
    reset_steps = np.arange(T) % limit == 0
    assert np.abs(obs[reset_steps, :, 0] - np.cos(theta[reset_steps])).max() < 2e-6
    assert np.abs(obs[reset_steps, :, 2] - theta_dot[reset_steps]).max() < 2e-6
    assert np.abs(obs[~reset_steps, :, 2] - theta_dot[~reset_steps]).max() > 0.1      # other steps continue the trajectory
    table = np.stack([theta[reset_steps], theta_dot[reset_steps]], axis=-1).astype(np.float32)
    want = oracle.Oracle().pendulum_rollout(oshape, params[:4481], np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8),
                                            np.zeros(N, np.float32), table, T, limit)
    first = np.arange(T) % limit < 3                       # tight right after a reset, chaotic divergence later
    assert np.abs(obs[first] - want["obs"].reshape(T, N, 3)[first]).max() < 4e-5
    assert np.abs(act.cpu().numpy().reshape(T, N)[first] - want["act"].reshape(T, N)[first]).max() < 4e-5
    assert np.array_equal(runner["episode_step"].cpu().numpy(), want["episode_step"])
    assert np.array_equal(runner["truncated"].cpu().numpy(), want["truncated"])


def test_randn_matches_numpy_philox_and_counter(lib, torch):
    """b200rl_randn_device_rng against the numpy statement of its counter layout (element / 4, call low, call high, 2 + stream id), and the
    device-resident call counter: call_index + *counter is what enters the Philox counter."""
    n, seed, stream_id, call = 1003, 0xABCDEF0123, 3, (1 << 33) + 5
    got = lib.randn_device_rng(torch.empty(n, device="cuda"), seed, stream_id=stream_id, call_index=call).cpu().numpy()
    q = np.arange((n + 3) // 4, dtype=np.uint64)
    counter = np.stack([q, np.full_like(q, call & 0xFFFFFFFF), np.full_like(q, call >> 32), np.full_like(q, 2 + stream_id)], -1).astype(np.uint32)
    words = philox4x32_10(counter, (seed & 0xFFFFFFFF, seed >> 32))
    u = ((words >> np.uint32(9)).astype(np.float64) + 0.5) * 2.0 ** -23
    want = np.empty((len(q), 4))
    for h in range(2):
        radius = np.sqrt(-2.0 * np.log(u[:, 2 * h]))
        want[:, 2 * h], want[:, 2 * h + 1] = radius * np.cos(2 * np.pi * u[:, 2 * h + 1]), radius * np.sin(2 * np.pi * u[:, 2 * h + 1])
    assert np.abs(got - want.reshape(-1)[:n]).max() < 1e-5      # fp32 Box-Muller against float64: a few ulp of sqrt(-2 log u) <= 5.6, amplified where log u is small
    counter_d = torch.tensor([call - 7], dtype=torch.int64, device="cuda")
    via_counter = lib.randn_device_rng(torch.empty(n, device="cuda"), seed, stream_id=stream_id, call_index=7, call_counter=counter_d).cpu().numpy()
    assert np.array_equal(via_counter, got)
    lib.counter_advance(counter_d, 7)
    assert int(counter_d.item()) == call
    other = lib.randn_device_rng(torch.empty(n, device="cuda"), seed, stream_id=stream_id + 1, call_index=call).cpu().numpy()
    assert abs(np.corrcoef(other, got)[0, 1]) < 0.15
    big = lib.randn_device_rng(torch.empty(1 << 21, device="cuda"), 5).cpu().numpy().astype(np.float64)
    m = big.size
    assert abs(big.mean()) < 5 / np.sqrt(m) and abs(big.var() - 1) < 5 * np.sqrt(2 / m) and abs((big ** 4).mean() - 3) < 5 * np.sqrt(96 / m)
    assert abs((big[1:] * big[:-1]).mean()) < 5 / np.sqrt(m)


def test_graph_replay_draws_fresh_numbers(lib, torch):
    """Sampling, noise and the counter advance captured once as a CUDA graph: every replay uses the next call index, and equals the
    direct calls with that index."""
    import test_gpu_gather as tg
    import make_golden as mg
    orc = oracle.Oracle()
    case = 0
    N, cap, limit, _, steps = mg.GATHER_CASES[case]
    st, _ = tg.replay_state(orc, case)
    replay, L = tg.pack_replay(lib, torch, st)
    B, seed = 64, 21
    counter = torch.zeros(1, dtype=torch.int64, device="cuda")
    out, noise = lib.new_batch(B), torch.empty((B, 1), device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def step():
        lib.gather_batch(replay, L, N, out, seed=seed, call_counter=counter, error_flag=flag)
        lib.randn_device_rng(noise, seed, stream_id=1, call_counter=counter)
        lib.counter_advance(counter, 1)

    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        step()                                                       # warm-up outside capture
    torch.cuda.current_stream().wait_stream(side)
    counter.zero_()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        step()
    seen = []
    for k in range(3):
        graph.replay()
        torch.cuda.synchronize()
        direct = lib.gather_batch(replay, L, N, lib.new_batch(B), seed=seed, call_index=k, error_flag=flag)
        direct_noise = lib.randn_device_rng(torch.empty((B, 1), device="cuda"), seed, stream_id=1, call_index=k)
        assert torch.equal(out["oa_base"], direct["oa_base"]) and torch.equal(out["rewards"], direct["rewards"]) and torch.equal(noise, direct_noise)
        seen.append(out["oa_base"].clone())
    assert int(counter.item()) == 3 and int(flag.item()) == 0
    assert not torch.equal(seen[0], seen[1]) and not torch.equal(seen[1], seen[2])
