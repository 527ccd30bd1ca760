"""GPU parity of the on-policy collect (through the C ABI) against the golden datasets of the real reference's
OnPolicyRunner::collect and against the CPU oracle: flags, counters and the noise-to-action arithmetic bit-exact, the
floating-point columns within 1e-5 relative / 2e-6 absolute per step when the state is teacher-forced."""
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu

OBS, MEAN, ACTION, LOGP, REWARD, TERMINATED, TRUNCATED, RESET, VALUE = slice(0, 3), 3, 4, 5, 6, 7, 8, 9, slice(10, 13)


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def shapes(lib, hact):
    return lib.MlpShape.make(3, [64, 64, 1], [hact, hact, 0]), oracle.MlpShape.make(3, [64, 64, 1], [hact, hact, 0])


def fresh_runner(N):
    return dict(states=np.zeros((N, 2), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8),
                episode_return=np.zeros(N, np.float32))


def to_dev(torch, runner):
    return {k: dev(torch, v) for k, v in runner.items()}


def gpu_collect(lib, torch, shape, params_d, runner_d, table, noise, T, limit, dataset=None, flag=None, layers=None):
    return lib.pendulum_collect(shape, params_d, params_d[4481:], runner_d["states"], runner_d["episode_step"], runner_d["truncated"],
                                runner_d["episode_return"], dev(torch, table) if len(table) else None, dev(torch, noise), T, limit,
                                dataset=dataset, error_flag=flag, layers=layers)


def close(got, want, rtol=1e-5, atol=1e-6, what=""):
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert np.all(err <= atol + rtol * np.abs(want)), f"{what}: max err {err.max():.3e}"


@pytest.mark.parametrize("case", range(len(mg.COLLECT_CASES)))
def test_collect_vs_reference_golden(lib, torch, case):
    """Consecutive collect calls on one runner, free-running, against the reference's datasets: the flag columns, the counters and the
    engine-driven reset rows are exact; float columns are tight on the first steps after a reset and bounded over the horizon."""
    fix = np.load(os.path.join(GOLDEN, "collect.npz"))
    N, T, limit, hact, n_collects = mg.COLLECT_CASES[case]
    shape, _ = shapes(lib, hact)
    params = mg.collect_params(case)
    params_d = dev(torch, params)
    runner = to_dev(torch, fresh_runner(N))
    rng = lib.rng_init_host(mg.COLLECT_SEED)
    ds = torch.full(((T + 1) * N, 13), 7.0, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    for c in range(n_collects):
        table, noise, _ = lib.collect_tables_host(rng, N, T, runner["episode_step"].cpu().numpy(), runner["truncated"].cpu().numpy(), limit, 8)
        gpu_collect(lib, torch, shape, params_d, runner, table, noise, T, limit, dataset=ds, flag=flag)
        got, want = ds.cpu().numpy(), fix[f"dataset_{case}"][c]
        assert int(flag.item()) == 0
        for col in (TERMINATED, TRUNCATED):
            assert np.array_equal(got[:T * N, col], want[:T * N, col]), col
        assert np.array_equal(got[:, RESET], want[:, RESET])
        assert np.all(got[:, VALUE] == 7.0) and np.all(got[T * N:, 3:9] == 7.0)    # not collect's: value / advantage / target, final rows beyond the observation
        # action = noise * std + mean with the reference's two roundings, on the GPU's own mean
        std = np.float32(np.exp(np.float64(params[-1])))          # correctly rounded, like the host's expf
        assert np.array_equal(got[:T * N, ACTION], noise.reshape(-1) * std + got[:T * N, MEAN])
        g, w = got[:T * N].reshape(T, N, 13), want[:T * N].reshape(T, N, 13)
        first = 0 if c == 0 else None                                # step 0 of the first call starts from exactly reset states
        if first is not None:
            for col in (OBS, MEAN, ACTION, LOGP, REWARD):
                close(g[0][:, col], w[0][:, col], what=f"step 0 col {col}")
        drift = np.abs(g[:, :, :7] - w[:, :, :7]).reshape(T, -1).max(1)
        print(f"case {case} collect {c}: max |dataset - reference| at step 0, {T // 2}, {T - 1}: {drift[0]:.2e} {drift[T // 2]:.2e} {drift[-1]:.2e}")
        assert drift.max() < 1e-3
    assert np.array_equal(runner["episode_step"].cpu().numpy(), fix[f"episode_step_{case}"])
    assert np.array_equal(runner["truncated"].cpu().numpy(), fix[f"truncated_{case}"])
    close(runner["states"].cpu().numpy(), fix[f"states_{case}"], what="final states")


@pytest.mark.parametrize("hact", ["relu", "tanh"])
def test_collect_single_step_teacher_forced(lib, orc, torch, hact):
    """One step at a time from the oracle's exact runner state, so no trajectory drift enters: every float column within
    1e-5 |ref| + 2e-6 (log-prob and reward 1e-5 absolute: they square the action difference), flags and counters exact."""
    N, steps, limit = 300, 40, 17
    shape, oshape = shapes(lib, hact)
    params = mg.det_uniform(71, 4482) * np.float32(0.35)
    params[-1] = np.float32(-0.8)
    params_d = dev(torch, params)
    runner = fresh_runner(N)
    rng_o, rng_g = orc.new_rng(23), lib.rng_init_host(23)
    for t in range(steps):
        table, noise, _ = lib.collect_tables_host(rng_g, N, 1, runner["episode_step"], runner["truncated"], limit, 1)
        want_table, want_noise = orc.collect_tables(rng_o, N, 1, runner["episode_step"], runner["truncated"], limit, 1)
        assert np.array_equal(table, want_table) and np.array_equal(noise, want_noise)
        runner_d = to_dev(torch, runner)
        got = gpu_collect(lib, torch, shape, params_d, runner_d, table, noise, 1, limit).cpu().numpy()
        want = orc.pendulum_collect(oshape, params, runner, 1, limit, reset_states=want_table, noise=want_noise)     # advances `runner`
        for col in (TERMINATED, TRUNCATED, RESET):
            assert np.array_equal(got[:, col], want[:, col]), (t, col)              # both datasets start from zeros here
        assert np.array_equal(got[:N, OBS], want[:N, OBS]) or np.abs(got[:N, OBS] - want[:N, OBS]).max() <= 2e-6
        close(got[:N, MEAN], want[:N, MEAN], what=f"mean t={t}")
        close(got[:N, ACTION], want[:N, ACTION], what=f"action t={t}")
        close(got[:N, LOGP], want[:N, LOGP], what=f"log_prob t={t}")
        close(got[:N, REWARD], want[:N, REWARD], what=f"reward t={t}")
        close(got[N:, OBS], want[N:, OBS], what=f"final observation t={t}")
        assert np.array_equal(runner_d["episode_step"].cpu().numpy(), runner["episode_step"])
        assert np.array_equal(runner_d["truncated"].cpu().numpy(), runner["truncated"])
        close(runner_d["states"].cpu().numpy(), runner["states"], what=f"states t={t}")
        close(runner_d["episode_return"].cpu().numpy(), runner["episode_return"], what=f"return t={t}")


def test_collect_layers_variant_pitch_and_error_flag(lib, torch):
    """Separately allocated layer tensors give the same bits as the flat arena; a wider row pitch leaves the padding alone; an
    exhausted reset table raises the device flag instead of reading past the table."""
    N, T, limit = 1000, 30, 12
    shape, _ = shapes(lib, "relu")
    params = mg.det_uniform(72, 4482) * np.float32(0.3)
    params_d = dev(torch, params)
    rng = lib.rng_init_host(3)
    r0 = fresh_runner(N)
    table, noise, used = lib.collect_tables_host(rng, N, T, r0["episode_step"], r0["truncated"], limit, 4)
    assert used == 3
    ra, rb, rc_ = to_dev(torch, r0), to_dev(torch, r0), to_dev(torch, r0)
    flat = gpu_collect(lib, torch, shape, params_d, ra, table, noise, T, limit)
    bounds = np.cumsum([0, 192, 64, 4096, 64, 64, 1])
    layers = [params_d[bounds[i]:bounds[i + 1]].clone() for i in range(6)]
    split = gpu_collect(lib, torch, shape, params_d, rb, table, noise, T, limit, layers=layers)
    assert torch.equal(flat, split)
    wide = torch.full(((T + 1) * N, 16), -3.0, device="cuda")
    gpu_collect(lib, torch, shape, params_d, rc_, table, noise, T, limit, dataset=wide)
    assert torch.equal(wide[:T * N, :10], flat[:T * N, :10]) and bool((wide[:, 10:] == -3.0).all())
    assert torch.equal(wide[T * N:, :3], flat[T * N:, :3]) and torch.equal(wide[:, 9], flat[:, 9]) and bool((wide[T * N:, 3:9] == -3.0).all())
    for k in ra:
        assert torch.equal(ra[k], rb[k]) and torch.equal(ra[k], rc_[k]), k
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    gpu_collect(lib, torch, shape, params_d, to_dev(torch, r0), table[:1], noise, T, limit, flag=flag)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1


def test_collect_full_size_properties(lib, torch):
    """65,536 environments x 64 steps (the PPO configuration's step count at the rollout benchmark's width): size-independent
    properties of the dataset -- reset is truncated delayed by one step, truncation exactly every step_limit steps, action and
    log-prob follow from mean / noise / log_std with the reference's arithmetic, cos^2 + sin^2 = 1, reward <= 0, the episode return
    is the sum of the rewards since the last reset, and a separate launch on the first 512 environments gives the same bits."""
    N, T, limit = 65536, 64, 25
    shape, _ = shapes(lib, "relu")
    params = mg.det_uniform(73, 4482) * np.float32(0.3)
    params[-1] = np.float32(-0.25)
    params_d = dev(torch, params)
    r0 = fresh_runner(N)
    table, noise, used = lib.collect_tables_host(lib.rng_init_host(9), N, T, r0["episode_step"], r0["truncated"], limit, 3)
    runner = to_dev(torch, r0)
    ds = gpu_collect(lib, torch, shape, params_d, runner, table, noise, T, limit).cpu().numpy()
    body = ds[:T * N].reshape(T, N, 13)
    trunc = body[:, :, TRUNCATED]
    want_trunc = ((np.arange(T) + 1) % limit == 0).astype(np.float32)[:, None].repeat(N, 1)
    assert np.array_equal(trunc, want_trunc)
    assert np.array_equal(ds[N:, RESET].reshape(T, N), trunc) and np.all(ds[:N, RESET] == 1.0)
    assert np.all(body[:, :, TERMINATED] == 0)
    std = np.float32(np.exp(np.float64(params[-1])))          # correctly rounded, like the host's expf
    assert np.array_equal(body[:, :, ACTION], noise * std + body[:, :, MEAN])
    ps = (body[:, :, ACTION] - body[:, :, MEAN]) / std
    c0 = np.float32(-0.5 * np.float32(np.log(np.float64(np.float32(2 * np.float32(np.pi))))))      # the host's logf, correctly rounded
    lp = (c0 - params[-1]).astype(np.float64) - 0.5 * ps.astype(np.float64) * ps.astype(np.float64)
    # the kernel carries the square as an exact float pair and rounds the difference once, where the reference rounds to double and then to
    # float: the two agree except where the double result lies next to a float rounding boundary, and then they are neighbouring floats
    got_lp, want_lp = body[:, :, LOGP], lp.astype(np.float32)
    differs = got_lp != want_lp
    assert differs.mean() < 1e-5 and np.all(np.abs(got_lp - want_lp)[differs] <= np.spacing(np.abs(want_lp[differs])))
    obs = ds[:, OBS]
    assert np.abs(obs[:, 0].astype(np.float64) ** 2 + obs[:, 1].astype(np.float64) ** 2 - 1).max() < 1e-6
    assert np.abs(obs[:, 2]).max() <= 8.0 and body[:, :, REWARD].max() <= 0
    since = (T // limit) * limit
    close(runner["episode_return"].cpu().numpy(), body[since:, :, REWARD].astype(np.float64).sum(0).astype(np.float32), what="episode return")
    assert np.array_equal(runner["episode_step"].cpu().numpy(), np.full(N, T - since, np.int32))
    # environment sharding does not change results: the first 512 environments alone
    M = 512
    sub = to_dev(torch, fresh_runner(M))
    ds_sub = gpu_collect(lib, torch, shape, params_d, sub, table[:, :M], noise[:, :M], T, limit).cpu().numpy()
    assert np.array_equal(ds_sub[:T * M].reshape(T, M, 13)[:, :, :10], body[:, :M, :10])
