"""GPU parity of the replay-buffer sampling (gather_batch, sequence length 1) through the C ABI: with the draws made on the
reference-compatible host engine every batch tensor equals the golden batches of the real reference bit for bit (the kernel only moves
data and applies the reference's index arithmetic); with the draws made inside the kernel the batch is checked against the oracle's
replay state row by row, and the index distribution against its uniform expectation."""
import ctypes as C
import os

import numpy as np
import pytest

import make_golden as mg
from conftest import GOLDEN
import oracle

pytestmark = pytest.mark.gpu
KEYS = ("oa_base", "rewards", "terminated", "reset", "next_reset_base", "final_step_mask", "next_final_step_mask_base")


@pytest.fixture(scope="module")
def torch():
    import torch
    assert torch.cuda.is_available()
    return torch


def pack_replay(lib, torch, st):
    """The oracle's replay state in the packed device layout (ReplayLayout.packed)."""
    N, cap = st["replay_data"].shape[:2]
    L = lib.ReplayLayout.packed(cap)
    raw = np.zeros((N, L.env_stride), np.uint8)
    raw[:, :40 * cap] = st["replay_data"].reshape(N, -1).view(np.uint8)
    raw[:, 40 * cap:44 * cap] = st["episode_start"].astype(np.uint32).view(np.uint8).reshape(N, -1)
    raw[:, 44 * cap:44 * cap + 4] = st["counters"][:, 0].astype(np.uint32).view(np.uint8).reshape(N, 4)
    raw[:, 44 * cap + 4:44 * cap + 8] = st["counters"][:, 2].astype(np.uint32).view(np.uint8).reshape(N, 4)
    raw[:, 44 * cap + 8] = st["counters"][:, 1].astype(np.uint8)
    return torch.from_numpy(raw.reshape(-1)).cuda(), L


def replay_state(orc, case):
    """(replay state after the case's runner steps, the oracle engine as those steps left it)"""
    N, cap, limit, batch, steps = mg.GATHER_CASES[case]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rng = orc.new_rng(mg.GATHER_SEED)
    return orc.offpolicy_steps(shape, mg.gather_params(case), orc.new_offpolicy_state(N, cap), limit, steps, rng), rng


def product_engine_after_steps(lib, N, steps, limit):
    """The product-side host engine advanced over the runner steps' reset draws, exactly as the reference's engine was."""
    rng = lib.rng_init_host(mg.GATHER_SEED)
    es, tr = np.zeros(N, np.int32), np.ones(N, np.uint8)
    rounds = steps // limit + 2
    table, used = np.zeros((rounds, N, 2), np.float32), C.c_int(0)
    lib.check(lib.lib().b200rl_reset_table_host(C.c_void_p(rng.ctypes.data), N, steps, C.c_void_p(es.ctypes.data), C.c_void_p(tr.ctypes.data), limit,
                                                C.c_void_p(table.ctypes.data), rounds, C.byref(used)), "b200rl_reset_table_host")
    return rng


@pytest.mark.parametrize("case", range(len(mg.GATHER_CASES)))
def test_gather_batch_vs_reference_golden(lib, orc, torch, case):
    fix = np.load(os.path.join(GOLDEN, "gather.npz"))
    N, cap, limit, batch, steps = mg.GATHER_CASES[case]
    st, orng = replay_state(orc, case)
    replay, L = pack_replay(lib, torch, st)
    rng = product_engine_after_steps(lib, N, steps, limit)
    position, full = lib.replay_counters(replay, L, N)
    assert np.array_equal(position.cpu().numpy(), st["counters"][:, 0]) and np.array_equal(full.cpu().numpy(), st["counters"][:, 1])
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    for g in range(mg.N_GATHERS + 1):                             # one more than the fixture holds: the engines must still agree afterwards
        env_index, offset = lib.gather_draws_host(rng, N, batch, position.cpu().numpy(), full.cpu().numpy(), cap)
        want = orc.gather_batch(st, batch, orng)
        assert np.array_equal(env_index, want["env_index"])
        out = lib.new_batch(batch)
        for v in out.values():
            v.fill_(3)                                            # every element must be written
        lib.gather_batch(replay, L, N, out, env_index=torch.from_numpy(env_index).cuda(), sample_offset=torch.from_numpy(offset).cuda(), error_flag=flag)
        assert int(flag.item()) == 0
        for k in KEYS:
            assert np.array_equal(out[k].cpu().numpy(), want[k]), (g, k)
            if g < mg.N_GATHERS:
                assert np.array_equal(out[k].cpu().numpy(), fix[f"{k}_{case}"][g]), (g, k)


def test_gather_batch_rejects_bad_indices(lib, orc, torch):
    """An environment index or a sample offset outside its range sets the error flag and leaves that element alone; nothing is read out
    of bounds."""
    case = 2                                                      # partly filled buffer: position 47 of 300
    N, cap, limit, batch, steps = mg.GATHER_CASES[case]
    st, _ = replay_state(orc, case)
    replay, L = pack_replay(lib, torch, st)
    env_index = np.array([0, N, 1, -1, 2], np.int32)
    offset = np.array([3, 0, steps, 0, steps - 1], np.int32)      # steps == position: first offset beyond the eligible range
    out = lib.new_batch(5)
    for v in out.values():
        v.fill_(3)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.gather_batch(replay, L, N, out, env_index=torch.from_numpy(env_index).cuda(), sample_offset=torch.from_numpy(offset).cuda(), error_flag=flag)
    assert int(flag.item()) == 2
    oa = out["oa_base"].cpu().numpy()
    assert np.array_equal(oa[0, 0], st["replay_data"][0, 3, :4]) and np.array_equal(oa[0, 4], st["replay_data"][2, steps - 1, :4])
    assert np.all(oa[:, [1, 2, 3]] == 3) and np.all(out["rewards"].cpu().numpy()[[1, 2, 3]] == 3)


@pytest.mark.parametrize("case", [0, 2])
def test_gather_batch_device_rng(lib, orc, torch, case):
    """Indices drawn inside the kernel: every batch element is a transition of the replay buffers (found by matching its row), inside the
    eligible range, step 1 carries that transition's next observation; calls with different call indices differ, the same call index
    repeats; environments and rows are hit uniformly."""
    N, cap, limit, _, steps = mg.GATHER_CASES[case]
    st, _ = replay_state(orc, case)
    replay, L = pack_replay(lib, torch, st)
    batch = 8192
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    a = lib.gather_batch(replay, L, N, lib.new_batch(batch), seed=17, call_index=0, error_flag=flag)
    b = lib.gather_batch(replay, L, N, lib.new_batch(batch), seed=17, call_index=1, error_flag=flag)
    a2 = lib.gather_batch(replay, L, N, lib.new_batch(batch), seed=17, call_index=0, error_flag=flag)
    assert int(flag.item()) == 0
    for k in KEYS:
        assert torch.equal(a[k], a2[k])
    assert not torch.equal(a["oa_base"], b["oa_base"])
    eligible = cap if steps >= cap else steps
    position = steps % cap
    valid = (position + 200 + np.arange(eligible)) % cap if steps >= cap else np.arange(eligible)
    rows = st["replay_data"][:, valid].reshape(-1, 10)                      # every row the reference could return
    keys = {r[:5].tobytes(): i for i, r in enumerate(rows)}
    oa, rew = a["oa_base"].cpu().numpy(), a["rewards"].cpu().numpy()
    hits = np.zeros(len(rows), np.int64)
    for i in range(batch):
        j = keys.get(np.concatenate([oa[0, i], rew[i:i + 1]]).tobytes())
        assert j is not None, i
        assert np.array_equal(oa[1, i, :3], rows[j, 5:8]) and oa[1, i, 3] == 0
        hits[j] += 1
    assert a["terminated"].sum().item() == 0 and a["reset"].min().item() == 1 and a["final_step_mask"].min().item() == 1
    assert np.array_equal(a["next_reset_base"].cpu().numpy(), np.ones((2, batch), np.uint8))
    assert np.array_equal(a["next_final_step_mask_base"].cpu().numpy(), np.stack([np.zeros(batch, np.uint8), np.ones(batch, np.uint8)]))
    # uniformity: chi-square of the hit counts against the uniform expectation (mean dof, sd sqrt(2 dof))
    expect = batch / len(rows)
    chi2 = ((hits - expect) ** 2 / expect).sum()
    dof = len(rows) - 1
    assert abs(chi2 - dof) < 6 * np.sqrt(2 * dof), (chi2, dof)


def test_gather_batch_device_rng_empty_buffer_sets_flag(lib, torch):
    L = lib.ReplayLayout.packed(16)
    replay = torch.zeros(4 * L.env_stride, dtype=torch.uint8, device="cuda")
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.gather_batch(replay, L, 4, lib.new_batch(8), seed=1, call_index=0, error_flag=flag)
    assert int(flag.item()) == 2


@pytest.mark.parametrize("case", range(len(mg.POLYAK_CASES)))
def test_polyak_update_vs_reference_golden(lib, orc, torch, case):
    """Target-network update against the reference's fixture, bit for bit; then on a view with a row pitch against the oracle."""
    fix = np.load(os.path.join(GOLDEN, "polyak.npz"))
    polyak, square, n = mg.POLYAK_CASES[case]
    source, target = mg.polyak_inputs()
    s_d, t_d = torch.from_numpy(source).cuda(), torch.from_numpy(target.copy()).cuda()
    for _ in range(n):
        lib.polyak_update(s_d, t_d, np.float32(polyak), square)
    assert np.array_equal(t_d.cpu().numpy(), fix[f"target_{case}"])
    rs = np.random.RandomState(case)
    big_s, big_t = rs.randn(300, 70).astype(np.float32), rs.randn(300, 80).astype(np.float32)
    s_d, t_d = torch.from_numpy(big_s).cuda(), torch.from_numpy(big_t).cuda()
    lib.polyak_update(s_d[:, 3:60], t_d[:, 10:67], np.float32(polyak), square)
    want = big_t.copy()
    view = np.ascontiguousarray(want[:, 10:67])
    orc.polyak_update(np.ascontiguousarray(big_s[:, 3:60]), view, np.float32(polyak), square)
    want[:, 10:67] = view
    assert np.array_equal(t_d.cpu().numpy(), want)


# --- sequences longer than 1 -----------------------------------------------------------------------------------------------------------
def sequence_replay_state(orc, which, steps):
    N, cap, limit, batch, L = oracle.Reference.GATHER_SEQUENCE_CASES[which]
    shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    rng = orc.new_rng(mg.GATHER_SEQ_SEED)
    return orc.offpolicy_steps(shape, mg.gather_sequence_params(which), orc.new_offpolicy_state(N, cap), limit, steps, rng)


@pytest.mark.parametrize("run", [i for i, r in enumerate(mg.GATHER_SEQ_RUNS) if r[1] in (8, 9)])
def test_gather_batch_sequences_deterministic_vs_reference_golden(lib, orc, torch, run):
    """With the reference's DETERMINISTIC flag (environment 0, offset = batch element) and fixed sequence lengths nothing is drawn: the kernel's
    walk through the replay buffer -- sequence starts (at the episode's first step or anywhere), cuts at truncated transitions, at the newest
    transition and at the padded length, next observations behind a sequence's end, every mask -- equals the real reference's batch bit for bit."""
    fix = np.load(os.path.join(GOLDEN, "gather_sequences.npz"))
    which, mode, steps = mg.GATHER_SEQ_RUNS[run]
    N, cap, limit, batch, L = oracle.Reference.GATHER_SEQUENCE_CASES[which]
    replay, layout = pack_replay(lib, torch, sequence_replay_state(orc, which, steps))
    out = lib.new_sequence_batch(batch, L)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    flags = (mode & 1) | lib.GATHER_FIRST_STEP_TARGET | lib.GATHER_DETERMINISTIC
    lib.gather_batch_sequences(replay, layout, N, out, flags=flags, error_flag=flag)
    assert int(flag.item()) == 0
    for k in mg.GATHER_SEQ_KEYS:
        assert np.array_equal(out[k].cpu().numpy(), fix[f"{k}_{run}"][0]), k          # both consecutive golden batches are the same without draws
        assert np.array_equal(fix[f"{k}_{run}"][0], fix[f"{k}_{run}"][1]), k


@pytest.mark.parametrize("which,steps,flags", [(0, 230, 7), (0, 800, 7), (1, 950, 7), (1, 950, 6), (0, 600, 4), (1, 299, 5)])
def test_gather_batch_sequences_with_device_draws(lib, orc, torch, which, steps, flags):
    """Draws made inside the kernel: every batch element is re-walked on the host from the oracle's replay state. Each step's observation | action
    row is located in the replay buffers; inside a sequence the indices are consecutive, a sequence starts at its episode's first step when that
    flag is set, ends where the rules say it may (truncated transition, newest transition, padded length, or -- with random lengths only -- early),
    the step behind a sequence's end holds that transition's next observation with a zero action, and the masks mark exactly these places.
    Over many elements all environments are used, and with random lengths both early cuts and full-length sequences occur."""
    N, cap, limit, batch_small, L = oracle.Reference.GATHER_SEQUENCE_CASES[which]
    st = sequence_replay_state(orc, which, steps)
    replay, layout = pack_replay(lib, torch, st)
    B, P = 2048, L + 1
    out = lib.new_sequence_batch(B, L)
    flag = torch.zeros(1, dtype=torch.int32, device="cuda")
    lib.gather_batch_sequences(replay, layout, N, out, flags=flags, seed=77, call_index=3, error_flag=flag)
    assert int(flag.item()) == 0
    mg.check_sequence_batch({k: v.cpu().numpy() for k, v in out.items()}, st, L, flags)
    # another call index draws another batch; the same call index the same one
    out2 = lib.new_sequence_batch(B, L)
    lib.gather_batch_sequences(replay, layout, N, out2, flags=flags, seed=77, call_index=4)
    assert not torch.equal(out2["oa_base"], out["oa_base"])
    out3 = lib.new_sequence_batch(B, L)                      # a fresh batch: entries behind a sequence's end are left as they are, like the reference's
    lib.gather_batch_sequences(replay, layout, N, out3, flags=flags, seed=77, call_index=3)
    assert all(torch.equal(out3[k], out[k]) for k in out)
