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
