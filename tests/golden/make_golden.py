"""Generate the golden fixtures in this directory from the REAL reference.

Runs only where the reference tree is available: it loads oracle/_ref/libref_strict.so, which oracle/Makefile
builds from the unmodified RLtools headers (generic CPU device, -O2 -fno-fast-math -ffp-contract=off), feeds it
seeded inputs and stores inputs and outputs as .npz files. The fixtures travel; the reference does not.

    python tests/golden/make_golden.py

Large output arrays are stored as a strided sample (every k-th element, at most MAX_KEEP elements) plus their
float64 sum; `sample()` below is the one definition of that subsampling and the tests import it.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

MAX_KEEP = 4096
MLP_STEPS = 2  # Adam steps recorded per MLP case


def _hash_u64(seed, n, stream):
    """splitmix64 of (seed, stream, index): integer-only, so identical bits on every platform and numpy version."""
    with np.errstate(over="ignore"):
        z = (np.arange(n, dtype=np.uint64) + np.uint64(1)) * np.uint64(0x9E3779B97F4A7C15)
        z = z + np.uint64(seed) * np.uint64(0xD1B54A32D192ED03) + np.uint64(stream) * np.uint64(0x8CB92BA72F3D8DD7)
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def det_uniform(seed, n, lo=-1.0, hi=1.0, stream=0):
    """Deterministic U[lo, hi) float32 from 24 hash bits (exact integer -> float conversion)."""
    u = (_hash_u64(seed, n, stream) >> np.uint64(40)).astype(np.float32) / np.float32(16777216.0)
    return (u * np.float32(hi - lo) + np.float32(lo)).astype(np.float32)


def det_normal(seed, n, stream=0):
    """Deterministic approximately-N(0,1) float32: sum of 12 twenty-bit uniforms minus 6 (Irwin-Hall), all integer
    arithmetic up to one exact float conversion, so no libm call is involved."""
    acc = np.zeros(n, np.uint64)
    for k in range(12):
        acc += _hash_u64(seed, n, stream * 16 + k + 1) >> np.uint64(44)
    return (acc.astype(np.float32) / np.float32(1048576.0) - np.float32(6.0)).astype(np.float32)


def sample(a):
    """Strided subsample used for large arrays: returns (values, float64 sum)."""
    flat = np.ascontiguousarray(a).reshape(-1)
    k = max(1, -(-flat.size // MAX_KEEP))
    return flat[::k].copy(), np.float64(flat.astype(np.float64).sum())


def mlp_inputs(case, seed):
    """Seeded synthetic inputs of one MLP case (regenerated identically by the tests; not stored)."""
    dims = [case["hidden_dim"]] * (case["num_layers"] - 1) + [case["output_dim"]]
    chunks, fan_in = [], case["input_dim"]
    for l, d in enumerate(dims):  # U(+-1/sqrt(fan_in)): the bound of the reference's default initialiser
        cnt = d * fan_in + d
        chunks.append(det_uniform(seed, cnt, stream=100 + l) / np.float32(np.sqrt(np.float32(fan_in))))
        fan_in = d
    params = np.concatenate(chunks).astype(np.float32)
    x = det_normal(seed, case["batch"] * case["input_dim"], stream=1).reshape(case["batch"], case["input_dim"])
    target = det_normal(seed, case["batch"] * case["output_dim"], stream=2).reshape(case["batch"], case["output_dim"])
    return params, x, target


def case_seed(name):
    return sum(map(ord, name))


def main():
    import oracle
    ref = oracle.Reference("strict")
    # ---- RNG streams (libstdc++ mt19937 + distributions as the reference drives them) ----
    rng_fix = {}
    for seed in (0, 1, 12345):
        rng_fix[f"uniform_{seed}"] = ref.uniform_stream(seed, 1024, -np.float32(np.pi), np.float32(np.pi))
        rng_fix[f"normal_{seed}"] = ref.normal_stream(seed, 1024, 0.25, 1.5)
        kinds = (np.arange(1024) % 3 == 0).astype(np.uint8)
        a = np.where(kinds == 0, -1.0, 0.0).astype(np.float32)
        b = np.where(kinds == 0, 1.0, 0.5).astype(np.float32)
        rng_fix[f"mixed_{seed}"] = ref.mixed_stream(seed, kinds, a, b)
        rng_fix[f"initial_states_{seed}"] = ref.pendulum_initial_states(seed, 1024)
    np.savez(os.path.join(HERE, "rng.npz"), **rng_fix)

    # ---- Pendulum step / reward / observe on independent samples ----
    states = np.stack([det_uniform(2, 4096, -12, 12, stream=0), det_uniform(2, 4096, -8, 8, stream=1)], 1).astype(np.float32)
    actions = det_uniform(2, 4096, -1.6, 1.6, stream=2)
    ns, r, obs, nobs = ref.pendulum_step(states, actions)
    np.savez(os.path.join(HERE, "pendulum_step.npz"), states=states, actions=actions, next_states=ns, rewards=r, obs=obs, next_obs=nobs)

    # ---- MLP cases: forward / backward / Adam ----
    cases = ref.cases()
    for name, c in cases.items():
        params, x, target = mlp_inputs(c, seed=case_seed(name))
        ev = ref.mlp_run(name, params, x, target, 0)
        one = ref.mlp_run(name, params, x, target, 1)
        tr = ref.mlp_run(name, params, x, target, 2, MLP_STEPS)
        full = ref.mlp_run(name, params, x, target, 3)
        fix = dict(dims=np.array([c[k] for k in ("batch", "input_dim", "hidden_dim", "output_dim", "num_layers", "hidden_act", "output_act")]))
        for key, arr in (("eval_out", ev["out"]), ("fwd_pre", one["pre"]), ("fwd_out", one["out"]), ("bwd_grads", one["grads"]),
                         ("train_params", tr["params"]), ("train_grads", tr["grads"]), ("train_m", tr["m"]), ("train_v", tr["v"]),
                         ("full_grads", full["grads"]), ("full_d_input", full["d_input"])):
            s, tot = sample(arr)
            fix[key] = s
            fix[key + "_sum"] = tot
        np.savez(os.path.join(HERE, f"mlp_{name}.npz"), **fix)

    # ---- Kaiming (legacy default) init_weights from the reference RNG, config-2 actor ----
    init = ref.mlp_run("c2_actor_b256", None, None, None, 0, init_seed=0)
    actor = init["params"]

    # ---- rollout with resets: 128 envs x 410 steps (resets at t=0, 200, 400), reference evaluate() per env ----
    N, T, LIMIT = 128, 410, 200
    st0 = np.zeros((N, 2), np.float32)
    es0 = np.zeros(N, np.int32)
    tr0 = np.ones(N, np.uint8)
    er0 = np.zeros(N, np.float32)
    # reset table drawn by the reference engine in the runner's order: per reset round, envs ascending, (theta, theta_dot)
    R = 3
    table = ref.pendulum_initial_states(5, R * N).reshape(R, N, 2)
    ro = ref.pendulum_rollout(actor, st0, es0, tr0, er0, table, T, LIMIT, chunk=1)
    np.savez(os.path.join(HERE, "rollout.npz"), actor_params=actor, reset_table=table, N=N, T=T, step_limit=LIMIT, reset_seed=5,
             obs=ro["obs"], act=ro["act"], rew=ro["rew"], states=ro["states"], episode_step=ro["episode_step"],
             truncated=ro["truncated"], episode_return=ro["episode_return"])
    # staggered start: counters differ per env, so resets fall at different steps
    es1 = (np.arange(N) * 7 % LIMIT).astype(np.int32)
    tr1 = (np.arange(N) % 5 == 0).astype(np.uint8)
    st1 = ref.pendulum_initial_states(9, N)
    ro1 = ref.pendulum_rollout(actor, st1, es1, tr1, er0, table, 300, LIMIT, chunk=1)
    np.savez(os.path.join(HERE, "rollout_staggered.npz"), states0=st1, episode_step0=es1, truncated0=tr1, T=300,
             obs=ro1["obs"][::7].copy(), act=ro1["act"][::7].copy(), rew=ro1["rew"][::7].copy(), states=ro1["states"],
             episode_step=ro1["episode_step"], truncated=ro1["truncated"], episode_return=ro1["episode_return"])
    # ---- GAE (reference Dataset + estimate_generalized_advantages) and the Gaussian policy head ----
    ppo = {}
    for N, steps in ((64, 1024), (5, 37)):
        n = N * steps
        rewards = det_normal(31, n, stream=N)
        all_values = det_normal(32, n + N, stream=N)
        truncated = (_hash_u64(33, n, N) % np.uint64(97) == 0).astype(np.uint8)
        terminated = (truncated & (_hash_u64(34, n, N) % np.uint64(2) == 0)).astype(np.uint8)     # termination implies truncation
        adv, tgt = ref.gae(rewards, all_values, terminated, truncated, N, steps)
        ppo[f"gae_{N}x{steps}_adv"], ppo[f"gae_{N}x{steps}_tgt"] = adv, tgt
    mean, log_std, value = det_normal(35, 4096), det_uniform(36, 4096, -2.0, 0.5), det_normal(37, 4096) * np.float32(1.5)
    lp, dm, dl = ref.normal_functions(mean, log_std, value)
    ppo.update(normal_log_prob=lp, normal_d_mean=dm, normal_d_log_std=dl)
    np.savez(os.path.join(HERE, "ppo.npz"), **ppo)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
