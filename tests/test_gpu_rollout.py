"""GPU parity of the fused Pendulum rollout (through the C ABI) against the CPU oracle and the golden rollout of the
real reference: integer runner state bit-exact, floating point within 1e-6 + 1e-5|ref| per step when the state is
teacher-forced, drift reported (and loosely bounded) for free-running trajectories of this chaotic system."""
import ctypes as C
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def actor_shapes(lib, acts=("relu", "relu", "tanh")):
    return lib.MlpShape.make(3, [64, 64, 1], list(acts)), oracle.MlpShape.make(3, [64, 64, 1], list(acts))


def close(got, want, rtol=1e-5, atol=1e-6):
    got = got.detach().cpu().numpy() if hasattr(got, "detach") else got
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(err <= atol + rtol * np.abs(want)), f"max err {err.max():.3e}"


@pytest.mark.parametrize("acts", [("relu", "relu", "tanh"), ("tanh", "fast_tanh", "identity"), ("sigmoid", "relu", "tanh")])
def test_single_step_teacher_forced(lib, orc, torch, acts):
    """T == 1 (one off-policy runner step) from oracle-provided states, 60 consecutive steps: every step's obs, action,
    reward and next state within tolerance; counters and flags exact."""
    shape, oshape = actor_shapes(lib, acts)
    N = 1000
    params = mg.det_uniform(17, oshape.num_params()) * np.float32(0.35)
    states = orc.pendulum_initial_states(4, N)
    es = (np.arange(N) * 11 % 200).astype(np.int32)
    tr = (np.arange(N) % 7 == 0).astype(np.uint8)
    er = mg.det_normal(3, N)
    table = orc.reset_table(21, N, 60, es, tr, 200, 2)
    counts = np.zeros(N, np.int64)
    dparams = dev(torch, params)
    for t in range(60):
        # the k-th reset of env e takes table[k][e]; with one step per call the caller hands over the right round
        round_table = np.stack([table[counts[e], e] for e in range(N)])[None]
        ref = orc.pendulum_rollout(oshape, params, states, es, tr, er, np.ascontiguousarray(round_table), 1)
        d_states, d_es, d_tr, d_er = dev(torch, states), dev(torch, es), dev(torch, tr), dev(torch, er)
        flag = torch.zeros(1, dtype=torch.int32, device="cuda")
        obs, act, rew = lib.pendulum_rollout(shape, dparams, d_states, d_es, d_tr, d_er, dev(torch, round_table), 1, error_flag=flag)
        assert int(flag.item()) == 0
        close(obs, ref["obs"])
        close(act, ref["act"])
        close(rew, ref["rew"])
        close(d_states, ref["states"])
        assert np.array_equal(d_es.cpu().numpy(), ref["episode_step"])
        assert np.array_equal(d_tr.cpu().numpy(), ref["truncated"])
        close(d_er, ref["episode_return"])
        counts += tr.astype(np.int64)
        states, es, tr, er = ref["states"], ref["episode_step"], ref["truncated"], ref["episode_return"]


def test_rollout_vs_reference_golden(lib, torch):
    """410 steps x 128 envs with resets at t = 0, 200, 400 against the REAL reference's trajectory. Integers and the
    RNG-driven reset rows are exact; floats are compared over the first steps after each reset (before chaotic
    divergence can amplify last-bit differences of sinf/tanhf) and the drift over the whole horizon is bounded."""
    fix = np.load(os.path.join(GOLDEN, "rollout.npz"))
    N, T, limit = int(fix["N"]), int(fix["T"]), int(fix["step_limit"])
    shape, _ = actor_shapes(lib)
    table, used = lib.reset_table_host(int(fix["reset_seed"]), N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), limit, 3)
    assert used == 3 and np.array_equal(table, fix["reset_table"])          # product-side RNG == reference engine
    st, es, tr, er = dev(torch, np.zeros((N, 2), np.float32)), dev(torch, np.zeros(N, np.int32)), dev(torch, np.ones(N, np.uint8)), dev(torch, np.zeros(N, np.float32))
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.pendulum_rollout(shape, dev(torch, fix["actor_params"]), st, es, tr, er, dev(torch, table), T, limit, error_flag=flag)
    assert int(flag.item()) == 0
    assert np.array_equal(es.cpu().numpy(), fix["episode_step"])
    assert np.array_equal(tr.cpu().numpy(), fix["truncated"])
    obs, act, rew = obs.cpu().numpy().reshape(T, N, 3), act.cpu().numpy().reshape(T, N), rew.cpu().numpy().reshape(T, N)
    gobs, gact, grew = fix["obs"].reshape(T, N, 3), fix["act"].reshape(T, N), fix["rew"].reshape(T, N)
    for t0 in (0, 200, 400):
        # reset rows: theta_dot is copied from the table, cos/sin computed from the exact same theta
        assert np.array_equal(obs[t0, :, 2], fix["reset_table"][t0 // 200, :, 1])
        for t in range(t0, t0 + 5):
            close(obs[t], gobs[t])
            close(act[t], gact[t])
    drift = np.abs(obs - gobs).reshape(T, -1).max(1)
    print("max |obs - reference| at t=1,10,50,199:", drift[1], drift[10], drift[50], drift[199])
    assert drift[:200].max() < 1e-2
    close(rew[:3], grew[:3])


def test_error_flag_when_reset_table_is_too_small(lib, torch):
    shape, oshape = actor_shapes(lib)
    N = 64
    params = dev(torch, mg.det_uniform(1, oshape.num_params()) * np.float32(0.2))
    st, es, tr, er = dev(torch, np.zeros((N, 2), np.float32)), dev(torch, np.full(N, 198, np.int32)), dev(torch, np.zeros(N, np.uint8)), dev(torch, np.zeros(N, np.float32))
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.pendulum_rollout(shape, params, st, es, tr, er, None, 5, error_flag=flag)     # env truncates after 2 steps, no table given
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert np.array_equal(es.cpu().numpy(), np.full(N, 3, np.int32))


def test_host_buffer_rollout_equals_device_rollout(lib, torch):
    """The host-buffer entry point (slabbed, overlapped copies) returns bit-identical trajectories to the device call."""
    shape, oshape = actor_shapes(lib)
    N, T, limit = 8192 + 384, 130, 50            # > 2^20 rows: the call runs as 8 slabs of steps; resets fall inside slabs
    params = mg.det_uniform(2, oshape.num_params()) * np.float32(0.3)
    table, _ = lib.reset_table_host(3, N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), limit, 3)
    st, es, tr, er = np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32)
    obs_h, act_h, rew_h = np.zeros((T * N, 3), np.float32), np.zeros((T * N, 1), np.float32), np.zeros((T * N, 1), np.float32)
    lib.pendulum_rollout_host(shape, params, st, es, tr, er, table, T, obs_h, act_h, rew_h, limit)
    d = [dev(torch, a) for a in (np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32))]
    obs, act, rew = lib.pendulum_rollout(shape, dev(torch, params), d[0], d[1], d[2], d[3], dev(torch, table), T, limit)
    assert np.array_equal(obs.cpu().numpy(), obs_h) and np.array_equal(act.cpu().numpy(), act_h) and np.array_equal(rew.cpu().numpy(), rew_h)
    assert np.array_equal(d[0].cpu().numpy(), st) and np.array_equal(d[1].cpu().numpy(), es) and np.array_equal(d[2].cpu().numpy(), tr)


def test_full_size_properties(lib, torch):
    """65,536 envs x 200 steps (the benchmark workload): size-independent properties -- every env ends the call
    truncated with episode_step == 200, cos^2 + sin^2 == 1, |theta_dot| <= 8, |action| <= 1, reward <= 0, the episode
    return equals the sum of rewards, and the first 512 envs equal a separate 512-env launch bit for bit (sharding
    by environment does not change results)."""
    shape, oshape = actor_shapes(lib)
    N, T = 65536, 200
    params = dev(torch, mg.det_uniform(5, oshape.num_params()) * np.float32(0.3))
    table, _ = lib.reset_table_host(1, N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), 200, 1)
    d = [dev(torch, a) for a in (np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32))]
    obs, act, rew = lib.pendulum_rollout(shape, params, d[0], d[1], d[2], d[3], dev(torch, table), T)
    assert bool((d[1] == 200).all()) and bool((d[2] == 1).all())
    o = obs.view(T, N, 3)
    assert float(((o[..., 0] ** 2 + o[..., 1] ** 2) - 1).abs().max()) < 1e-5
    assert float(o[..., 2].abs().max()) <= 8.0 and float(act.abs().max()) <= 1.0 and float(rew.max()) <= 0.0
    ret = rew.view(T, N).double().sum(0)
    # the device adds 200 rewards in fp32 at |sum| <= 2000: at most 200 * 2^-24 * 2000 = 2.4e-2 from the exact sum, ~sqrt(200) of an ulp typically
    assert float((ret - d[3].double()).abs().max()) < 1e-2
    M = 512
    ds = [dev(torch, a) for a in (np.zeros((M, 2), np.float32), np.zeros(M, np.int32), np.ones(M, np.uint8), np.zeros(M, np.float32))]
    obs_s, act_s, rew_s = lib.pendulum_rollout(shape, params, ds[0], ds[1], ds[2], ds[3], dev(torch, np.ascontiguousarray(table[:, :M])), T)
    assert torch.equal(obs_s.view(T, M, 3), o[:, :M]) and torch.equal(act_s.view(T, M), act.view(T, N)[:, :M])


@pytest.mark.parametrize("case", range(len(mg.OFFPOLICY_CASES)))
def test_offpolicy_step_with_replay_buffers_vs_reference_golden(lib, orc, torch, case):
    """step() of the off-policy runner with per-environment replay buffers, one call per step, teacher-forced from the oracle's runner
    state every step (so no trajectory drift enters): replay rows written this step within 1e-5 |ref| + 2e-6, the bookkeeping
    (episode_start, position, full, current_episode_start, the truncation mark on the previous transition) exact; after the last step
    the whole replay buffer equals the reference's fixture within the same tolerance."""
    fix = np.load(os.path.join(GOLDEN, "offpolicy.npz"))
    N, cap, limit, steps = mg.OFFPOLICY_CASES[case]
    shape, oshape = actor_shapes(lib)
    params = mg.offpolicy_params(case)
    st = orc.new_offpolicy_state(N, cap)
    rng_o, rng_g = orc.new_rng(mg.OFFPOLICY_SEED), lib.rng_init_host(mg.OFFPOLICY_SEED)
    L = lib.ReplayLayout.packed(cap)
    replay = torch.zeros(N * L.env_stride, dtype=torch.uint8, device="cuda")
    params_d = dev(torch, params)
    bounds = np.cumsum([0, 192, 64, 4096, 64, 64, 1])
    layers = [params_d[bounds[i]:bounds[i + 1]].clone() for i in range(6)]
    obs, act, nobs = torch.zeros((N, 3), device="cuda"), torch.zeros((N, 1), device="cuda"), torch.zeros((N, 3), device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")

    def unpack():
        raw = replay.cpu().numpy().reshape(N, L.env_stride)
        data = raw[:, :40 * cap].copy().view(np.float32).reshape(N, cap, 10)
        es = raw[:, 40 * cap:44 * cap].copy().view(np.uint32).reshape(N, cap)
        pos = raw[:, 44 * cap:44 * cap + 4].copy().view(np.uint32)[:, 0]
        ces = raw[:, 44 * cap + 4:44 * cap + 8].copy().view(np.uint32)[:, 0]
        return data, es, pos, raw[:, 44 * cap + 8], ces

    for t in range(steps):
        table = np.zeros((1, N, 2), np.float32)                 # this step's reset draws, from the product-side engine in environment order
        lib.check(lib.lib().b200rl_reset_table_host(C.c_void_p(rng_g.ctypes.data), N, 1, C.c_void_p(st["episode_step"].ctypes.data),
                                                    C.c_void_p(st["truncated"].ctypes.data), limit, C.c_void_p(table.ctypes.data), 1, None), "b200rl_reset_table_host")
        d = [dev(torch, st[k]) for k in ("states", "episode_step", "truncated", "episode_return")]
        before = st["counters"].copy()
        lib.pendulum_offpolicy_step(shape, params_d, d[0], d[1], d[2], d[3], dev(torch, table), limit, obs, act, nobs, replay, L, error_flag=flag,
                                    layers=layers if t % 2 else None)
        orc.offpolicy_steps(oshape, params, st, limit, 1, rng_o)            # advances `st`
        data, es, pos, full, ces = unpack()
        assert int(flag.item()) == 0
        assert np.array_equal(pos, st["counters"][:, 0]) and np.array_equal(full, st["counters"][:, 1]) and np.array_equal(ces, st["counters"][:, 2])
        assert np.array_equal(d[1].cpu().numpy(), st["episode_step"]) and np.array_equal(d[2].cpu().numpy(), st["truncated"])
        rows = before[:, 0]
        got_rows, want_rows = data[np.arange(N), rows], st["replay_data"][np.arange(N), rows]
        assert np.array_equal(got_rows[:, 8:], want_rows[:, 8:])
        close(got_rows[:, :8], want_rows[:, :8])
        assert np.array_equal(es[np.arange(N), rows], st["episode_start"][np.arange(N), rows])
        close(nobs, st["buf_next_obs"])
        close(d[0], st["states"])
    data, es, pos, full, ces = unpack()
    w = min(steps, cap)
    assert np.array_equal(data[:, :w, 8:], fix[f"replay_data_{case}"][:, :, 8:])          # terminated / truncated flags incl. the marks set at resets
    close(data[:, :w, :8], fix[f"replay_data_{case}"][:, :, :8])
    assert np.array_equal(es[:, :w], fix[f"episode_start_{case}"]) and np.array_equal(np.stack([pos, full, ces], 1), fix[f"counters_{case}"])


@pytest.mark.parametrize("N", [443, 130, 1, 33, 80004, 75777])
def test_environment_counts_that_fill_tiles_unevenly(lib, orc, torch, N):
    """Environment counts that leave tiles partly filled (443 per SM-sized launch, 130, 1, 33) and that need several tiles per group (80,004
    and 75,777: beyond 4 x 128 environments per SM; 75,777 is odd, i.e. the per-thread-store form). Three steps from given states, with
    resets of the truncated environments, against the oracle's runner loop: every environment is stepped exactly once per step."""
    shape, oshape = actor_shapes(lib)
    T = 3
    params = mg.det_uniform(23, oshape.num_params()) * np.float32(0.3)
    rs = np.random.RandomState(N)
    states = np.stack([rs.uniform(-3, 3, N), rs.uniform(-2, 2, N)], 1).astype(np.float32)
    es = rs.randint(0, 199, N).astype(np.int32)
    tr = (rs.uniform(size=N) < 0.3).astype(np.uint8)
    er = rs.randn(N).astype(np.float32)
    table = np.stack([rs.uniform(-np.pi, np.pi, (2, N)), rs.uniform(-1, 1, (2, N))], 2).astype(np.float32)
    ref = orc.pendulum_rollout(oshape, params, states, es, tr, er, table, T)
    d_states, d_es, d_tr, d_er = dev(torch, states), dev(torch, es), dev(torch, tr), dev(torch, er)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    obs, act, rew = lib.pendulum_rollout(shape, dev(torch, params), d_states, d_es, d_tr, d_er, dev(torch, table), T, error_flag=flag)
    assert int(flag.item()) == 0
    close(obs.cpu().numpy()[:N], ref["obs"][:N])                      # first step: exact inputs
    close(act.cpu().numpy()[:N], ref["act"][:N])
    assert np.array_equal(d_es.cpu().numpy(), ref["episode_step"]) and np.array_equal(d_tr.cpu().numpy(), ref["truncated"])
    # later steps: the oracle's MLP on the kernel's own observations (one rounding difference in a state must not be held against the next step)
    close(act.cpu().numpy().reshape(-1), orc.mlp_evaluate(oshape, params, obs.cpu().numpy()).reshape(-1))
    close(d_states, ref["states"], rtol=1e-4, atol=1e-5)
