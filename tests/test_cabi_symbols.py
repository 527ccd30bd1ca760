"""CPU-side checks of the C-ABI library: it loads without a GPU, exports every symbol include/b200rl.h declares,
validates arguments before touching the device, and its host-only entry points (reference-compatible reset table)
agree with the oracle bit for bit."""
import ctypes as C
import os
import re

import numpy as np

from conftest import ROOT


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "b200rl.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(b200rl_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported(lib):
    L = lib.lib()
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(L, n), f"{n} declared in include/b200rl.h but not exported"


def test_version_and_status_strings(lib):
    L = lib.lib()
    assert L.b200rl_version() >= 100
    assert L.b200rl_status_string(0) == b"ok"
    assert b"invalid" in L.b200rl_status_string(1)


def test_argument_validation_happens_before_any_cuda_call(lib):
    L = lib.lib()
    assert L.b200rl_dense_forward(None, None, None, 0, None, 0, None, 0, 4, 4, 4, 0, None) == 1
    assert L.b200rl_adam_step(None, None, None, None, 10, lib.AdamHyper(), None, None) == 1
    shape = lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    assert L.b200rl_pendulum_rollout(C.byref(shape), None, None, None, None, None, None, 0, 4, 4, 200, None, None, None, None, None) == 1
    bad = lib.MlpShape.make(3, [48, 48, 1], ["relu", "relu", "tanh"])
    assert L.b200rl_pendulum_rollout(C.byref(bad), None, None, None, None, None, None, 0, 4, 4, 200, None, None, None, None, None) == 2
    assert L.b200rl_mlp_num_params(C.byref(shape)) == 3 * 64 + 64 + 64 * 64 + 64 + 64 + 1


def test_reset_table_matches_oracle_stream(lib, orc):
    """Product-side mt19937 / uniform_real (host code of the library) vs the oracle's independent restatement."""
    N, T, limit = 300, 450, 200
    es = (np.arange(N) * 13 % limit).astype(np.int32)
    tr = (np.arange(N) % 3 == 0).astype(np.uint8)
    table, used = lib.reset_table_host(7, N, T, es, tr, limit, 4)
    want = orc.reset_table(7, N, T, es, tr, limit, 4)
    assert used == 3
    assert np.array_equal(table, want)
    # too few rounds is an error, not an overrun
    state = np.zeros(625, np.uint32)
    lib.lib().b200rl_rng_init_host(C.c_void_p(state.ctypes.data), 7)
    small = np.zeros((1, N, 2), np.float32)
    rc = lib.lib().b200rl_reset_table_host(C.c_void_p(state.ctypes.data), N, T, C.c_void_p(es.ctypes.data), C.c_void_p(tr.ctypes.data), limit,
                                           C.c_void_p(small.ctypes.data), 1, None)
    assert rc == 1


def test_collect_tables_match_oracle_stream(lib, orc):
    """Product-side normal_distribution / uniform_real draw order of on-policy collect vs the oracle's restatement, across two
    consecutive calls on one engine state."""
    N, T, limit = 131, 77, 30
    es = (np.arange(N) * 7 % limit).astype(np.int32)
    tr = (np.arange(N) % 4 == 0).astype(np.uint8)
    state, rng = lib.rng_init_host(11), orc.new_rng(11)
    for _ in range(2):
        table, noise, used = lib.collect_tables_host(state, N, T, es, tr, limit, 4)
        want_table, want_noise = orc.collect_tables(rng, N, T, es, tr, limit, 4)
        assert used == 3
        assert np.array_equal(table, want_table) and np.array_equal(noise, want_noise)
    # step_limit 0 = never truncated: only the initially flagged environments draw a state
    table, noise, used = lib.collect_tables_host(state, N, T, es, tr, 0, 1)
    want_table, want_noise = orc.collect_tables(rng, N, T, es, tr, 0, 1)
    assert used == 1 and np.array_equal(table, want_table) and np.array_equal(noise, want_noise)


def test_shuffle_permutation_matches_oracle_stream(lib, orc):
    """Product-side uniform_int_distribution / Fisher-Yates order of the PPO epoch shuffle vs the oracle's restatement, two epochs on one
    engine; every result is a permutation."""
    state, rng = lib.rng_init_host(21), orc.new_rng(21)
    for n in (4096, 185, 1):
        for _ in range(2):
            perm = lib.shuffle_permutation_host(state, n)
            assert np.array_equal(perm, orc.shuffle_permutation(rng, n))
            assert np.array_equal(np.sort(perm), np.arange(n))


def test_product_does_not_reference_the_oracle():
    """The shipped package must never import or link the CPU oracle."""
    pkg = os.path.join(ROOT, "rl-tools_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".h", ".hpp", ".cpp")):
                text = open(os.path.join(dirpath, f), errors="ignore").read()
                assert "import oracle" not in text and "liboracle" not in text and "oracle/" not in text, f


def test_argument_validation_of_the_later_entry_points(lib):
    """The entry points of the sampling / SAC / normalisation / generic-rollout rows reject null pointers and impossible sizes with
    B200RL_ERR_INVALID_ARGUMENT (1) or B200RL_ERR_UNSUPPORTED (2) before any CUDA call (this machine has no GPU)."""
    L = lib.lib()
    layout = lib.ReplayLayout.packed(16)
    assert L.b200rl_replay_counters(None, C.byref(layout), 4, None, None, None) == 1
    assert L.b200rl_gather_batch(None, C.byref(layout), 4, 200, 3, 1, None, None, 8, None, 4, None, None, None, None, None, None, None, None) == 1
    assert L.b200rl_gather_batch_device_rng(None, C.byref(layout), 4, 200, 3, 1, 1, 0, 8, None, 4, None, None, None, None, None, None, None, None) == 1
    assert L.b200rl_gather_batch_device_counter(None, C.byref(layout), 4, 200, 3, 1, 1, None, 8, None, 4, None, None, None, None, None, None, None, None) == 1
    assert L.b200rl_polyak_update(None, 4, None, 4, 2, 4, 0.5, 0, None) == 1
    assert L.b200rl_sample_and_squash_forward(None, 2, None, 1, 8, 1, None, None, 1, None, None) == 1
    assert L.b200rl_sample_and_squash_backward(None, 2, None, 1, None, None, 1, None, 1, None, -1.0, 8, 1, None, 2, None, None, None) == 1
    assert L.b200rl_sac_target_action_values(None, 1, None, 1, None, None, None, None, 0.99, 0, 1, 1, None, 1, 8, None) == 1
    assert L.b200rl_sac_min_value_d_output(None, 1, None, 1, None, None, 4, 3, 1, None, 1, 8, None) == 1
    assert L.b200rl_running_normalizer_update(None, 3, 10, 3, None, None, 1, None) == 1
    assert L.b200rl_standardize_set_statistics(None, None, 3, None, None, None) == 1
    assert L.b200rl_standardize_forward(None, 3, None, None, None, 3, 10, 3, None) == 1
    assert L.b200rl_counter_advance(None, 1, None) == 1
    assert L.b200rl_randn_device_rng(None, 16, 1, 0, 0, None, None) == 1
    shape6, shape3 = lib.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"]), lib.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    assert L.b200rl_env_rollout(7, C.byref(shape6), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None) == 1       # no such environment
    assert L.b200rl_env_rollout(lib.ENV_ACROBOT_SWINGUP, C.byref(shape3), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None) == 2
    assert L.b200rl_env_rollout(lib.ENV_ACROBOT_SWINGUP, C.byref(shape6), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None) == 1
    assert (L.b200rl_env_observation_dim(0), L.b200rl_env_state_dim(0), L.b200rl_env_observation_dim(1), L.b200rl_env_state_dim(1)) == (3, 2, 6, 4)
    # the L2F entry points: missing parameter blocks, an actor that is not 18 -> H -> H -> 4 with H in {16, 32, 64}, missing outputs
    p = lib.L2fParameters.make(np.zeros(85, np.float32), 0.01)
    mdp, init = (C.c_float * 18)(), (C.c_float * 12)()
    good, wide = lib.MlpShape.make(18, [32, 32, 4], ["relu", "relu", "tanh"]), lib.MlpShape.make(18, [48, 48, 4], ["relu", "relu", "tanh"])
    assert L.b200rl_l2f_steps(None, None, None, 4, 1, None) == 1 and L.b200rl_l2f_steps(C.byref(p), None, None, 4, 1, None) == 1
    assert L.b200rl_l2f_steps(C.byref(p), None, None, 0, 1, None) == 0                                          # nothing to do
    assert L.b200rl_l2f_rollout(C.byref(p), None, C.byref(good), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None, None) == 1
    assert L.b200rl_l2f_rollout(C.byref(p), mdp, C.byref(wide), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None, None) == 2
    assert L.b200rl_l2f_rollout(C.byref(p), mdp, C.byref(good), None, None, None, None, None, None, 0, 4, 4, 10, None, None, None, None, None, None) == 1
    assert L.b200rl_l2f_rollout_device_rng(C.byref(p), mdp, None, C.byref(good), None, None, None, None, None, 1, 0, 4, 4, 10, None, None, None, None, None) == 1
    assert L.b200rl_l2f_rollout_device_rng(C.byref(p), mdp, init, C.byref(wide), None, None, None, None, None, 1, 0, 4, 4, 10, None, None, None, None, None) == 2
    assert L.b200rl_l2f_rollout_device_rng(C.byref(p), mdp, init, C.byref(good), None, None, None, None, None, 1, 0, 4, 0, 10, None, None, None, None, None) == 0
    assert L.b200rl_l2f_initial_states_from_draws(C.byref(p), None, None, None, None, 4, None) == 1
    assert L.b200rl_l2f_initial_states_from_draws(C.byref(p), init, None, None, None, 4, None) == 1
    assert L.b200rl_l2f_initial_states_from_draws(C.byref(p), init, None, None, None, 0, None) == 0
    lay43, lay10 = lib.ReplayLayout.packed(8, 18, 4), lib.ReplayLayout.packed(8)
    assert (lay43.ld_data, lay10.ld_data, lay10.env_stride) == (43, 10, 44 * 8 + 12)
    assert L.b200rl_l2f_offpolicy_prologue(C.byref(p), None, None, None, None, None, None, 0, 0, None, 4, None, None, None) == 1
    assert L.b200rl_l2f_offpolicy_prologue(C.byref(p), init, None, None, None, None, None, 0, 0, None, 4, None, None, None) == 1
    assert L.b200rl_l2f_offpolicy_epilogue(C.byref(p), None, None, None, None, None, 4, 10, None, None, None, C.byref(lay43), None, None) == 1
    assert L.b200rl_l2f_offpolicy_epilogue(C.byref(p), mdp, None, None, None, None, 4, 10, None, None, None, C.byref(lay43), None, None) == 1
    L.b200rl_cooperative_pass_status.argtypes = [C.POINTER(C.c_int)]
    assert L.b200rl_cooperative_pass_status(None) == 1
    # host-side draws of gather_batch: an empty replay buffer is refused, like the reference's assertion
    state = lib.rng_init_host(3)
    out = np.zeros(4, np.int32)
    pos, full = np.zeros(2, np.int32), np.zeros(2, np.uint8)
    rc = L.b200rl_gather_draws_host(C.c_void_p(state.ctypes.data), 2, 4, C.c_void_p(pos.ctypes.data), C.c_void_p(full.ctypes.data), 16, C.c_void_p(out.ctypes.data), C.c_void_p(out.ctypes.data))
    assert rc == 1


def test_gather_draws_match_oracle_stream(lib, orc):
    """Product-side draws of gather_batch (environment, then offset below that environment's eligible count) vs the oracle's
    restatement of the reference's order, on buffers with different fill levels."""
    N, cap, batch = 7, 50, 200
    counters = np.zeros((N, 3), np.int64)
    counters[:, 0] = [1, 13, 49, 0, 25, 7, 3]
    counters[3, 1] = 1                                           # one full buffer (position 0)
    st = dict(replay_data=np.arange(N * cap * 10, dtype=np.float32).reshape(N, cap, 10), counters=counters)
    state, rng = lib.rng_init_host(5), orc.new_rng(5)
    for _ in range(2):
        env_index, offset = lib.gather_draws_host(state, N, batch, counters[:, 0], counters[:, 1], cap)
        want = orc.gather_batch(st, batch, rng)
        assert np.array_equal(env_index, want["env_index"])
        full = counters[env_index, 1] != 0
        index = np.where(full, (counters[env_index, 0] + 200 + offset) % cap, offset)
        assert np.array_equal(index, want["sample_index"])
