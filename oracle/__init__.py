"""TEST INFRASTRUCTURE: ctypes bindings for the CPU oracle (oracle.c) and, where it was built, the real reference
(ref_driver.cpp compiled against the unmodified RLtools headers).

Only tests/, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline legs import this package. The product
package never does.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "_build", "liboracle.so")
REF_STRICT_SO = os.path.join(_HERE, "_ref", "libref_strict.so")
REF_FAST_SO = os.path.join(_HERE, "_ref", "libref_fast.so")
REF_CUDA_SO = os.path.join(_HERE, "_ref", "libref_cuda.so")

ACT = {"identity": 0, "relu": 1, "tanh": 2, "fast_tanh": 3, "sigmoid": 4}

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")
_u8p = np.ctypeslib.ndpointer(dtype=np.uint8, flags="C_CONTIGUOUS")


def build(ref: bool = True) -> None:
    """Compile oracle.c (always) and the reference driver (when the reference tree exists)."""
    subprocess.run(["make", "-s", "-C", _HERE, "oracle"], check=True)
    # the reference tree: named by B200RL_REFERENCE, else a checkout next to this repository; absent -> the prebuilt _ref libraries are used
    reference = os.environ.get("B200RL_REFERENCE") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference")
    if ref and os.path.isdir(os.path.join(reference, "include", "rl_tools")):
        subprocess.run(["make", "-s", "-C", _HERE, "ref", "REFERENCE=" + reference], check=True)
        if os.path.exists("/usr/local/cuda/bin/nvcc"):            # the reference's own CUDA device, as the second baseline
            subprocess.run(["make", "-s", "-C", _HERE, "ref_cuda", "REFERENCE=" + reference], check=True)


class MlpShape(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("input_dim", C.c_int), ("dims", C.c_int * 8), ("acts", C.c_int * 8)]

    @staticmethod
    def make(input_dim, dims, acts):
        s = MlpShape()
        s.n_layers = len(dims)
        s.input_dim = input_dim
        for i, (d, a) in enumerate(zip(dims, acts)):
            s.dims[i] = d
            s.acts[i] = ACT[a] if isinstance(a, str) else a
        return s

    def num_params(self):
        n, i = 0, self.input_dim
        for l in range(self.n_layers):
            n += self.dims[l] * i + self.dims[l]
            i = self.dims[l]
        return n

    def layer_dims(self):
        return [self.dims[l] for l in range(self.n_layers)]


def C5_SHAPE():
    """The training network of the sharded configuration."""
    return MlpShape.make(64, [256, 256, 256, 16], ["relu", "relu", "relu", "identity"])


def _opt(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


class Oracle:
    """Typed wrapper around liboracle.so. Arrays are float32 C-contiguous numpy arrays."""

    def __init__(self, path=ORACLE_SO):
        if not os.path.exists(path):
            build(ref=False)
        self.lib = L = C.CDLL(path)
        L.orc_rng_uniform_stream.argtypes = [C.c_uint32, C.c_int, C.c_float, C.c_float, _f32p]
        L.orc_rng_normal_stream.argtypes = [C.c_uint32, C.c_int, C.c_float, C.c_float, _f32p]
        L.orc_rng_mixed_stream.argtypes = [C.c_uint32, C.c_int, _u8p, _f32p, _f32p, _f32p]
        L.orc_dense_forward.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_void_p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_dense_backward.argtypes = [_f32p, _f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,
                                         C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.orc_mse_gradient.argtypes = [_f32p, C.c_int, _f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_mse_evaluate.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_mse_evaluate.restype = C.c_float
        L.orc_adam_bias_correction.argtypes = [C.c_float, C.c_float, C.POINTER(C.c_uint32), C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.orc_adam_update.argtypes = [_f32p, _f32p, _f32p, _f32p, C.c_size_t] + [C.c_float] * 7
        L.orc_mlp_evaluate.argtypes = [C.POINTER(MlpShape), _f32p, _f32p, C.c_int, _f32p, C.c_int, C.c_int]
        L.orc_mlp_forward.argtypes = [C.POINTER(MlpShape), _f32p, _f32p, C.c_int, _f32p, _f32p, C.c_int]
        L.orc_mlp_backward.argtypes = [C.POINTER(MlpShape), _f32p, _f32p, _f32p, C.c_int, _f32p, _f32p, _f32p, C.c_void_p, C.c_int]
        L.orc_pendulum_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.orc_pendulum_step_batch.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, C.c_void_p, C.c_void_p]
        L.orc_pendulum_rollout.argtypes = [C.POINTER(MlpShape), _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int,
                                           _f32p, _f32p, _f32p, C.c_void_p]
        L.orc_pendulum_rollout.restype = C.c_int
        L.orc_rng_init.argtypes = [C.c_void_p, C.c_uint32]
        L.orc_reset_table.argtypes = [C.c_void_p, C.c_int, C.c_int, _i32p, _u8p, C.c_int, _f32p, C.c_int]
        L.orc_reset_table.restype = C.c_int
        L.orc_gae.argtypes = [_f32p, _f32p, _u8p, _u8p, _f32p, _f32p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_int]
        _u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
        L.orc_rng_uniform_int_stream.argtypes = [C.c_uint32, C.c_int, _u64p, _u64p, _u64p]
        L.orc_shuffle_permutation.argtypes = [C.c_void_p, C.c_int, _i32p]
        _i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
        L.orc_offpolicy_steps.argtypes = [C.POINTER(MlpShape), _f32p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, _f32p, _i32p, _u8p, _f32p,
                                          _f32p, _i64p, _f32p, _f32p, _i64p, _f32p, _f32p, _f32p]
        L.orc_sample_and_squash_forward.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p]
        L.orc_sample_and_squash_backward.argtypes = [_f32p, C.c_int, _f32p, _f32p, _f32p, _f32p, C.c_float, C.c_float, C.c_int, C.c_int, _f32p, C.c_int, _f32p, _f32p]
        L.orc_running_normalizer_update.argtypes = [_f32p, C.c_int, C.c_int, C.c_int, _f32p, _f32p, C.c_void_p]
        L.orc_standardize_set_statistics.argtypes = [_f32p, _f32p, C.c_int, _f32p, _f32p]
        L.orc_standardize_forward.argtypes = [_f32p, C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int]
        L.orc_acrobot_step_batch.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.orc_acrobot_rollout.argtypes = [C.POINTER(MlpShape), _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, C.c_void_p]
        L.orc_acrobot_rollout.restype = C.c_int
        L.orc_acrobot_rollout_variant.argtypes = [C.c_int, C.POINTER(MlpShape), _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _u8p,
                                                  C.c_void_p]
        L.orc_acrobot_rollout_variant.restype = C.c_int
        L.orc_acrobot_terminating_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.orc_polyak_update.argtypes = [_f32p, C.c_int, _f32p, C.c_int, C.c_int, C.c_int, C.c_float, C.c_int]
        L.orc_l2f_functions.argtypes = [C.c_int, _f32p, C.c_float, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _u8p]
        L.orc_l2f_rollout.argtypes = [C.c_void_p, _f32p, _f32p, C.c_float, _f32p, _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _u8p]
        L.orc_l2f_steps.argtypes = [C.c_int, C.c_int, _f32p, C.c_float, _f32p, _f32p, _f32p, _f32p]
        L.orc_l2f_initial_state_from_draws.argtypes = [_f32p, C.c_float, C.c_float, _f32p, _f32p, _f32p]
        L.orc_l2f_sample_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p, C.c_float, C.c_float, _f32p]
        L.orc_gather_batch_sequences.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_float, C.c_void_p, _f32p, _i64p, _i64p, _f32p, _f32p, _u8p, _u8p, _u8p, _u8p, _u8p]
        L.orc_gather_batch.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.c_void_p, _f32p, _i64p, _f32p, _f32p, _u8p, _u8p, _u8p, _u8p, _u8p, _i32p, _i32p]
        L.orc_pendulum_collect.argtypes = [C.POINTER(MlpShape), _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, C.c_void_p, C.c_void_p, C.c_int,
                                           C.c_void_p, C.c_int, _f32p, C.c_int]
        L.orc_pendulum_collect.restype = C.c_int
        L.orc_collect_tables.argtypes = [C.c_void_p, C.c_int, C.c_int, _i32p, _u8p, C.c_int, _f32p, C.c_int, _f32p]
        L.orc_collect_tables.restype = C.c_int
        L.orc_normal_functions.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.orc_ppo_policy_gradient.argtypes = [_f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_float, C.c_float, C.c_float, C.c_int, C.c_int]

    # --- RNG -----------------------------------------------------------------------------------------------
    def uniform_stream(self, seed, n, lo, hi):
        out = np.empty(n, np.float32)
        self.lib.orc_rng_uniform_stream(seed, n, lo, hi, out)
        return out

    def normal_stream(self, seed, n, mean, std):
        out = np.empty(n, np.float32)
        self.lib.orc_rng_normal_stream(seed, n, mean, std, out)
        return out

    def mixed_stream(self, seed, kinds, a, b):
        out = np.empty(len(kinds), np.float32)
        self.lib.orc_rng_mixed_stream(seed, len(kinds), kinds, a, b, out)
        return out

    # --- dense / mlp ---------------------------------------------------------------------------------------
    def dense_forward(self, W, b, x, act, want_pre=True):
        B, I = x.shape
        O = W.shape[0]
        pre = np.empty((B, O), np.float32) if want_pre else None
        y = np.empty((B, O), np.float32)
        self.lib.orc_dense_forward(W, b, x, I, _opt(pre), O, y, O, B, I, O, ACT[act] if isinstance(act, str) else act)
        return pre, y

    def dense_backward(self, W, x, pre, d_out, act, dW=None, db=None, want_d_in=True, want_grads=True):
        B, I = x.shape
        O = W.shape[0]
        d_out = d_out.copy()
        if want_grads:
            dW = np.zeros((O, I), np.float32) if dW is None else dW.copy()
            db = np.zeros(O, np.float32) if db is None else db.copy()
        else:
            dW = db = None
        d_in = np.empty((B, I), np.float32) if want_d_in else None
        self.lib.orc_dense_backward(W, x, I, pre, O, d_out, O, _opt(dW), _opt(db), _opt(d_in), I, B, I, O,
                                    ACT[act] if isinstance(act, str) else act, 1)
        return dW, db, d_in, d_out

    def mse_gradient(self, a, b, loss_weight=1.0):
        d = np.empty_like(a)
        self.lib.orc_mse_gradient(a, a.shape[1], b, b.shape[1], d, d.shape[1], a.shape[0], a.shape[1], loss_weight)
        return d

    def mse_evaluate(self, a, b, loss_weight=1.0):
        return float(self.lib.orc_mse_evaluate(a, a.shape[1], b, b.shape[1], a.shape[0], a.shape[1], loss_weight))

    def adam_bias_correction(self, beta_1, beta_2, age):
        a = C.c_uint32(age)
        c1, c2 = C.c_float(), C.c_float()
        self.lib.orc_adam_bias_correction(beta_1, beta_2, C.byref(a), C.byref(c1), C.byref(c2))
        return c1.value, c2.value, a.value

    def adam_update(self, p, g, m, v, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2):
        p, m, v = p.copy(), m.copy(), v.copy()
        self.lib.orc_adam_update(p, g, m, v, p.size, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)
        return p, m, v

    def mlp_evaluate(self, shape, params, x):
        B = x.shape[0]
        y = np.empty((B, shape.dims[shape.n_layers - 1]), np.float32)
        self.lib.orc_mlp_evaluate(C.byref(shape), params, x, x.shape[1], y, y.shape[1], B)
        return y

    def mlp_forward(self, shape, params, x):
        B = x.shape[0]
        n = B * sum(shape.layer_dims())
        pre, out = np.empty(n, np.float32), np.empty(n, np.float32)
        self.lib.orc_mlp_forward(C.byref(shape), params, x, x.shape[1], pre, out, B)
        return pre, out

    def mlp_backward(self, shape, params, grads, x, pre, out, d_out, want_d_input=False):
        B = x.shape[0]
        grads = grads.copy()
        d_out = d_out.copy()
        d_in = np.empty((B, shape.input_dim), np.float32) if want_d_input else None
        self.lib.orc_mlp_backward(C.byref(shape), params, grads, x, x.shape[1], pre, out, d_out, _opt(d_in), B)
        return grads, d_in

    def mlp_train_steps(self, shape, params, x, target, n_steps, alpha=1e-3, beta_1=0.9, beta_2=0.999, eps=1e-7, eps_sqrt=1e-7):
        """n_steps x {zero_gradient, forward, mse gradient (weight 1), backward, Adam step}; TF-default hyper-parameters."""
        p = params.copy()
        m = np.zeros_like(p)
        v = np.zeros_like(p)
        age = 1
        g = np.zeros_like(p)
        pre = out = None
        for _ in range(n_steps):
            g = np.zeros_like(p)
            pre, out = self.mlp_forward(shape, p, x)
            O = shape.dims[shape.n_layers - 1]
            y = out[-x.shape[0] * O:].reshape(x.shape[0], O)
            d = self.mse_gradient(np.ascontiguousarray(y), target, 1.0)
            g, _ = self.mlp_backward(shape, p, g, x, pre, out, d)
            c1, c2, age = self.adam_bias_correction(beta_1, beta_2, age)
            p, m, v = self.adam_update(p, g, m, v, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)
        return p, g, m, v, pre, out

    def mlp_chunked_step(self, shape, params, x, target, chunk_rows, do_step=True, alpha=1e-3, beta_1=0.9, beta_2=0.999, eps=1e-7, eps_sqrt=1e-7):
        """One optimizer step over chunks of chunk_rows rows: per chunk forward, mse gradient weighted chunk_rows / rows, backward with the
        gradients accumulating over the chunks; then Adam (first step). Returns params, grads, m, v and the last chunk's pre / out."""
        rows = x.shape[0]
        assert rows % chunk_rows == 0
        g = np.zeros_like(params)
        O = shape.dims[shape.n_layers - 1]
        w = np.float32(np.float32(chunk_rows) / np.float32(rows))
        pre = out = None
        for c in range(0, rows, chunk_rows):
            xc, tc = np.ascontiguousarray(x[c:c + chunk_rows]), np.ascontiguousarray(target[c:c + chunk_rows])
            pre, out = self.mlp_forward(shape, params, xc)
            y = np.ascontiguousarray(out[-chunk_rows * O:].reshape(chunk_rows, O))
            g, _ = self.mlp_backward(shape, params, g, xc, pre, out, self.mse_gradient(y, tc, w))
        p, m, v = params.copy(), np.zeros_like(params), np.zeros_like(params)
        if do_step:
            c1, c2, _ = self.adam_bias_correction(beta_1, beta_2, 1)
            p, m, v = self.adam_update(p, g, m, v, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)
        return dict(params=p, grads=g, m=m, v=v, pre=pre, out=out)

    @staticmethod
    def dataset_columns(obs_dim, action_dim):
        """Column indices of the on-policy dataset matrix (rl/components/on_policy_runner/on_policy_runner.h:38-72, symmetric observations)."""
        o, a = obs_dim, action_dim
        return dict(obs=slice(0, o), mean=slice(o, o + a), action=slice(o + a, o + 2 * a), log_prob=o + 2 * a, reward=o + 2 * a + 1, terminated=o + 2 * a + 2,
                    truncated=o + 2 * a + 3, reset=o + 2 * a + 4, value=o + 2 * a + 5, advantage=o + 2 * a + 6, target=o + 2 * a + 7, dim=o + 2 * a + 8)

    def uniform_int_stream(self, seed, lo, hi):
        lo, hi = np.ascontiguousarray(lo, np.uint64), np.ascontiguousarray(hi, np.uint64)
        out = np.empty(lo.size, np.uint64)
        self.lib.orc_rng_uniform_int_stream(seed, lo.size, lo, hi, out)
        return out

    def shuffle_permutation(self, rng, n):
        """perm[i] = original row that the reference's epoch shuffle leaves at position i (engine `rng` advanced in place)."""
        perm = np.empty(n, np.int32)
        self.lib.orc_shuffle_permutation(rng, n, perm)
        return perm

    def ppo_train(self, actor_shape, critic_shape, actor_params, critic_params, dataset, n_rows, batch, epochs,
                  alpha=1e-3, beta_1=0.9, beta_2=0.999, eps=1e-7, eps_sqrt=1e-7, shuffle_rng=None):
        """The PPO update of rl/algorithms/ppo/operations_generic.h:96-336, default parameters: per minibatch zero_gradient, actor
        forward, clipped-surrogate gradient (+ log_std gradient), actor backward, critic forward, MSE gradient with weight 0.5 against
        the target values, critic backward, one Adam step each. dataset = the [rows, obs + 2 act + 8] matrix of the on-policy runner;
        actor_params = MLP arena + log_std[act]. shuffle_rng (from new_rng) switches the per-epoch row shuffle on (:127-158): observation,
        action, advantage, log-prob and target-value columns, in place. Returns (actor params, grads, first moment, critic ...)."""
        na = actor_shape.num_params()
        A = actor_shape.dims[actor_shape.n_layers - 1]
        col = self.dataset_columns(actor_shape.input_dim, A)
        shuffled = list(range(col["obs"].start, col["obs"].stop)) + list(range(col["action"].start, col["action"].stop)) + [col["log_prob"], col["advantage"], col["target"]]
        ap, cp = actor_params.copy(), critic_params.copy()
        am, av, cm, cv = np.zeros_like(ap), np.zeros_like(ap), np.zeros_like(cp), np.zeros_like(cp)
        a_age = c_age = 1
        ag, cg = np.zeros_like(ap), np.zeros_like(cp)
        for _ in range(epochs):
            if shuffle_rng is not None:
                perm = self.shuffle_permutation(shuffle_rng, n_rows)
                dataset[:n_rows, shuffled] = dataset[:n_rows][perm][:, shuffled]
            for b in range(n_rows // batch):
                rows = dataset[b * batch:(b + 1) * batch]
                obs = np.ascontiguousarray(rows[:, col["obs"]])
                pre, out = self.mlp_forward(actor_shape, ap[:na], obs)
                current = np.ascontiguousarray(out[-batch * A:].reshape(batch, A))
                d_actions, d_log_std = self.ppo_policy_gradient(current, np.ascontiguousarray(rows[:, col["action"]]), ap[na:], np.ascontiguousarray(rows[:, col["log_prob"]]),
                                                                np.ascontiguousarray(rows[:, col["advantage"]]))
                g_mlp, _ = self.mlp_backward(actor_shape, ap[:na], np.zeros(na, np.float32), obs, pre, out, d_actions)
                ag = np.concatenate([g_mlp, d_log_std]).astype(np.float32)
                pre, out = self.mlp_forward(critic_shape, cp, obs)
                values = np.ascontiguousarray(out[-batch:].reshape(batch, 1))
                d_values = self.mse_gradient(values, np.ascontiguousarray(rows[:, col["target"]:col["target"] + 1]), 0.5)
                cg, _ = self.mlp_backward(critic_shape, cp, np.zeros_like(cp), obs, pre, out, d_values)
                c1, c2, a_age = self.adam_bias_correction(beta_1, beta_2, a_age)
                ap, am, av = self.adam_update(ap, ag, am, av, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)
                c1, c2, c_age = self.adam_bias_correction(beta_1, beta_2, c_age)
                cp, cm, cv = self.adam_update(cp, cg, cm, cv, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)
        return ap, ag, am, cp, cg, cm

    # --- pendulum ------------------------------------------------------------------------------------------
    def pendulum_initial_states(self, seed, n):
        s = np.empty((n, 2), np.float32)
        self.lib.orc_pendulum_initial_states(seed, n, s)
        return s

    def pendulum_step(self, states, actions):
        n = states.shape[0]
        ns, r = np.empty((n, 2), np.float32), np.empty(n, np.float32)
        obs, nobs = np.empty((n, 3), np.float32), np.empty((n, 3), np.float32)
        self.lib.orc_pendulum_step_batch(n, states, np.ascontiguousarray(actions.reshape(-1)), ns, r, _opt(obs), _opt(nobs))
        return ns, r, obs, nobs

    def reset_table(self, seed, N, T, episode_step, truncated, step_limit, R):
        rng = C.create_string_buffer(4 * 624 + 16)
        self.lib.orc_rng_init(rng, seed)
        table = np.zeros((R, N, 2), np.float32)
        used = self.lib.orc_reset_table(rng, N, T, episode_step, truncated, step_limit, table, R)
        if used < 0:
            raise ValueError("reset table too small")
        return table

    def pendulum_rollout(self, shape, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=200,
                         teacher_states=None):
        N = states.shape[0]
        states, episode_step = states.copy(), episode_step.copy()
        truncated, episode_return = truncated.copy(), episode_return.copy()
        obs = np.empty((T * N, 3), np.float32)
        act = np.empty((T * N, 1), np.float32)
        rew = np.empty((T * N, 1), np.float32)
        rc = self.lib.orc_pendulum_rollout(C.byref(shape), params, N, T, states, episode_step, truncated, episode_return, reset_states,
                                           reset_states.shape[0], step_limit, obs, act, rew, _opt(teacher_states))
        if rc != 0:
            raise RuntimeError(f"orc_pendulum_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    # --- acrobot swing-up ------------------------------------------------------------------------------------
    def acrobot_step(self, states, actions):
        n = states.shape[0]
        ns, r, obs, nobs = np.empty((n, 4), np.float32), np.empty(n, np.float32), np.empty((n, 6), np.float32), np.empty((n, 6), np.float32)
        self.lib.orc_acrobot_step_batch(n, np.ascontiguousarray(states, np.float32), np.ascontiguousarray(actions.reshape(-1), np.float32), ns, r, obs, nobs)
        return ns, r, obs, nobs

    def acrobot_initial_states(self, seed, n):
        """sample_initial_state of AcrobotSwingup from one engine: theta_1, theta_2 ~ U(-pi, pi), velocities 0."""
        draws = self.uniform_stream(seed, 2 * n, -np.float32(np.pi), np.float32(np.pi)).reshape(n, 2)
        return np.concatenate([draws, np.zeros((n, 2), np.float32)], axis=1)

    def acrobot_terminating_initial_states(self, seed, n):
        """n initial states of the terminating Acrobot (four U(-0.1, 0.1) draws each, double bounds) from a fresh engine: [n, 4]."""
        s = np.empty((n, 4), np.float32)
        self.lib.orc_acrobot_terminating_initial_states(seed, n, s)
        return s

    def acrobot_terminating_rollout(self, shape, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=500):
        """The runner loop on the terminating Acrobot: reset_states [R, N, 4]; returns obs, act, rew, terminated and the runner state."""
        N = states.shape[0]
        states, episode_step, truncated, episode_return = (np.array(states, np.float32), np.array(episode_step, np.int32), np.array(truncated, np.uint8),
                                                           np.array(episode_return, np.float32))
        reset_states = np.ascontiguousarray(reset_states, np.float32)
        assert reset_states.shape[1:] == (N, 4)
        obs, act, rew, term = np.empty((T * N, 6), np.float32), np.empty((T * N, 1), np.float32), np.empty((T * N, 1), np.float32), np.empty(T * N, np.uint8)
        rc = self.lib.orc_acrobot_rollout_variant(1, C.byref(shape), np.ascontiguousarray(params, np.float32), N, T, states, episode_step, truncated, episode_return,
                                                  reset_states, reset_states.shape[0], step_limit, obs, act, rew, term, None)
        if rc != 0:
            raise RuntimeError(f"orc_acrobot_rollout_variant rc={rc}")
        return dict(obs=obs, act=act, rew=rew, terminated=term, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    def acrobot_rollout(self, shape, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=500, teacher_states=None):
        N = states.shape[0]
        states, episode_step = states.copy(), episode_step.copy()
        truncated, episode_return = truncated.copy(), episode_return.copy()
        obs, act, rew = np.empty((T * N, 6), np.float32), np.empty((T * N, 1), np.float32), np.empty((T * N, 1), np.float32)
        rc = self.lib.orc_acrobot_rollout(C.byref(shape), params, N, T, states, episode_step, truncated, episode_return, reset_states, reset_states.shape[0],
                                          step_limit, obs, act, rew, None if teacher_states is None else teacher_states.ctypes.data_as(C.c_void_p))
        if rc != 0:
            raise RuntimeError(f"orc_acrobot_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    # --- off-policy runner with replay buffers -------------------------------------------------------------
    @staticmethod
    def new_offpolicy_state(N, capacity):
        """Runner + replay-buffer state right after init(): every environment flagged truncated, empty buffers."""
        return dict(states=np.zeros((N, 2), np.float32), episode_step=np.zeros(N, np.int32), truncated=np.ones(N, np.uint8), episode_return=np.zeros(N, np.float32),
                    replay_data=np.zeros((N, capacity, 10), np.float32), episode_start=np.zeros((N, capacity), np.int64),
                    replay_states=np.zeros((N, capacity, 2), np.float32), replay_next_states=np.zeros((N, capacity, 2), np.float32),
                    counters=np.zeros((N, 3), np.int64), buf_obs=np.zeros((N, 3), np.float32), buf_act=np.zeros((N, 1), np.float32),
                    buf_next_obs=np.zeros((N, 3), np.float32))

    def offpolicy_steps(self, shape, params, st, step_limit, n_steps, rng):
        """n_steps x step() of the off-policy runner on the state dict `st` (updated in place); `rng` from new_rng."""
        N, capacity = st["replay_data"].shape[:2]
        self.lib.orc_offpolicy_steps(C.byref(shape), params, N, capacity, step_limit, n_steps, rng, st["states"], st["episode_step"], st["truncated"],
                                     st["episode_return"], st["replay_data"], st["episode_start"], st["replay_states"], st["replay_next_states"],
                                     st["counters"], st["buf_obs"], st["buf_act"], st["buf_next_obs"])
        return st

    def sample_and_squash(self, inp, noise, d_output, log_alpha, target_entropy=-1.0):
        """Forward (external noise) and backward of the SAC policy head on inp [B, 2A]: dict(pre_squashing, output, log_probs, d_input,
        d_log_alpha_per_sample, log_alpha_gradient)."""
        B, A = noise.shape
        inp, noise, d_output = (np.ascontiguousarray(x, np.float32) for x in (inp, noise, d_output))
        out = dict(pre_squashing=np.empty((B, A), np.float32), output=np.empty((B, A), np.float32), log_probs=np.empty(B, np.float32),
                   d_input=np.empty((B, 2 * A), np.float32), d_log_alpha_per_sample=np.empty(B, np.float32))
        self.lib.orc_sample_and_squash_forward(inp, 2 * A, noise, B, A, out["pre_squashing"], out["output"], out["log_probs"])
        grad = np.zeros(1, np.float32)
        self.lib.orc_sample_and_squash_backward(inp, 2 * A, noise, out["pre_squashing"], out["output"], d_output, log_alpha, target_entropy, B, A,
                                                out["d_input"], 2 * A, out["d_log_alpha_per_sample"], grad)
        out["log_alpha_gradient"] = grad[0]
        return out

    def normalizer(self, data):
        """RunningNormalizer updates on data [U, R, D] (fresh normalizer), then a standardize layer with the resulting statistics on the last
        batch: dict(mean [U, D], std [U, D], layer_mean, layer_precision, output [R, D])."""
        U, R, D = data.shape
        data = np.ascontiguousarray(data, np.float32)
        mean, std, age = np.zeros(D, np.float32), np.ones(D, np.float32), C.c_uint64(0)
        means, stds = np.empty((U, D), np.float32), np.empty((U, D), np.float32)
        for u in range(U):
            self.lib.orc_running_normalizer_update(data[u], D, R, D, mean, std, C.byref(age))
            means[u], stds[u] = mean, std
        lm, lp = np.empty(D, np.float32), np.empty(D, np.float32)
        self.lib.orc_standardize_set_statistics(mean, std, D, lm, lp)
        out = np.empty((R, D), np.float32)
        self.lib.orc_standardize_forward(data[-1], D, lm, lp, out, D, R, D)
        return dict(mean=means, std=stds, layer_mean=lm, layer_precision=lp, output=out)

    def sac_target_action_values(self, q1, q2, rewards, terminated, next_log_probs, log_alpha, gamma=np.float32(0.99)):
        """rl/algorithms/sac/operations_generic.h:133-163 with the default parameters (entropy bonus inside the discounted term, termination honoured)."""
        alpha = np.float32(np.exp(np.float64(np.float32(log_alpha))))          # the host libm's expf is correctly rounded
        m = np.minimum(q1, q2).astype(np.float32) + (-alpha * next_log_probs.astype(np.float32))
        future = np.where(terminated == 0, np.float32(gamma) * m, np.float32(0)).astype(np.float32)
        return (rewards.astype(np.float32) + future).astype(np.float32)

    def sac_updates(self, hidden, actor_params, log_alpha, critic_params, target_params, oa_base, rewards, terminated, noise_critic, noise_actor,
                    alpha=1e-3, beta_1=0.9, beta_2=0.999, eps=1e-7, eps_sqrt=1e-7, polyak=np.float32(1.0 - 0.005), target_entropy=-1.0):
        """n x { train_critic(critic 0), train_critic(critic 1), update_critic_targets, train_actor } of rl/algorithms/sac/operations_generic.h
        (:223-336, :486-522, :378-456), default parameters, sequence length 1, Pendulum shapes (observation 3, action 1), hidden width `hidden`.
        oa_base [U, 2, B, 4], rewards / terminated [U, B], noise_critic [U, 2, B, 1], noise_actor [U, B, 1]; critic_params / target_params [2, n].
        Returns dict(actor=(params, grads, m), log_alpha=(value, grad, m), critics=[(params, grads, m)] * 2, targets=[params] * 2, target_values)."""
        U, _, B, _ = oa_base.shape
        actor_shape = MlpShape.make(3, [hidden, hidden, 2], ["relu", "relu", "identity"])
        critic_shape = MlpShape.make(4, [hidden, hidden, 1], ["relu", "relu", "identity"])
        ap = actor_params.copy(); am, av, ag = np.zeros_like(ap), np.zeros_like(ap), np.zeros_like(ap)
        la = np.array([log_alpha], np.float32); lm, lv, lg = np.zeros(1, np.float32), np.zeros(1, np.float32), np.zeros(1, np.float32)
        cp = [critic_params[c].copy() for c in range(2)]
        cm, cv, cg = ([np.zeros_like(cp[0]) for _ in range(2)] for _ in range(3))
        tp = [target_params[c].copy() for c in range(2)]
        ages = dict(actor=1, alpha=1, c0=1, c1=1)
        adam = lambda p, g, m, v, key: self._adam(p, g, m, v, ages, key, alpha, beta_1, beta_2, eps, eps_sqrt)
        target_values = None
        for u in range(U):
            obs, nobs = np.ascontiguousarray(oa_base[u, 0, :, :3]), np.ascontiguousarray(oa_base[u, 1, :, :3])
            oa = np.ascontiguousarray(oa_base[u, 0])
            for c in range(2):
                head_in = self.mlp_evaluate(actor_shape, ap, nobs)
                head = self.sample_and_squash(head_in, noise_critic[u, c], np.zeros((B, 1), np.float32), la[0], target_entropy)
                nin = np.ascontiguousarray(np.concatenate([nobs, head["output"]], axis=1))
                q1, q2 = self.mlp_evaluate(critic_shape, tp[0], nin)[:, 0], self.mlp_evaluate(critic_shape, tp[1], nin)[:, 0]
                target_values = self.sac_target_action_values(q1, q2, rewards[u], terminated[u], head["log_probs"], la[0])
                pre, out = self.mlp_forward(critic_shape, cp[c], oa)
                values = np.ascontiguousarray(out[-B:].reshape(B, 1))
                d_values = self.mse_gradient(values, np.ascontiguousarray(target_values.reshape(B, 1)), 0.5)
                cg[c], _ = self.mlp_backward(critic_shape, cp[c], np.zeros_like(cp[c]), oa, pre, out, d_values)
                cp[c], cm[c], cv[c] = adam(cp[c], cg[c], cm[c], cv[c], f"c{c}")
            for c in range(2):                                 # update_critic_targets, layer by layer = element-wise over the flat arena
                t2 = tp[c].reshape(1, -1).copy()
                self.polyak_update(cp[c].reshape(1, -1), t2, polyak)
                tp[c] = t2.reshape(-1)
            pre_a, out_a = self.mlp_forward(actor_shape, ap, obs)
            head_in = np.ascontiguousarray(out_a[-2 * B:].reshape(B, 2))
            inp = obs
            fwd = self.sample_and_squash(head_in, noise_actor[u], np.zeros((B, 1), np.float32), la[0], target_entropy)
            cin = np.ascontiguousarray(np.concatenate([inp, fwd["output"]], axis=1))
            d_out = np.full((B, 1), np.float32(-1) / np.float32(B), np.float32)
            qs, d_ins = [], []
            for c in range(2):
                pre, out = self.mlp_forward(critic_shape, cp[c], cin)
                qs.append(out[-B:].copy())
                _, d_in = self.mlp_backward(critic_shape, cp[c], np.zeros_like(cp[c]), cin, pre, out, d_out, want_d_input=True)
                d_ins.append(d_in)
            d_action = np.where((qs[0] < qs[1])[:, None], d_ins[0][:, 3:], d_ins[1][:, 3:]).astype(np.float32)
            bwd = self.sample_and_squash(head_in, noise_actor[u], np.ascontiguousarray(d_action), la[0], target_entropy)
            ag, _ = self.mlp_backward(actor_shape, ap, np.zeros_like(ap), obs, pre_a, out_a, np.ascontiguousarray(bwd["d_input"]))
            lg = np.array([bwd["log_alpha_gradient"]], np.float32)
            ap, am, av = adam(ap, ag, am, av, "actor")
            la, lm, lv = adam(la, lg, lm, lv, "alpha")
        return dict(actor=(ap, ag, am), log_alpha=(la[0], lg[0], lm[0]), critics=[(cp[c], cg[c], cm[c]) for c in range(2)], targets=tp, target_values=target_values)

    def _adam(self, p, g, m, v, ages, key, alpha, beta_1, beta_2, eps, eps_sqrt):
        c1, c2, ages[key] = self.adam_bias_correction(beta_1, beta_2, ages[key])
        return self.adam_update(p, g, m, v, alpha, beta_1, beta_2, eps, eps_sqrt, c1, c2)

    def polyak_update(self, source, target, polyak, square=False):
        """target = polyak * target + (1 - polyak) * source [squared], in place on a 2-D float32 array."""
        rows, cols = target.shape
        self.lib.orc_polyak_update(np.ascontiguousarray(source, np.float32), cols, target, cols, rows, cols, polyak, int(square))
        return target

    @staticmethod
    def new_batch(batch):
        """Output arrays of one gather_batch with sequence length 1 (padded length 2)."""
        return dict(oa_base=np.zeros((2, batch, 4), np.float32), rewards=np.zeros(batch, np.float32), terminated=np.zeros(batch, np.uint8),
                    reset=np.zeros(batch, np.uint8), next_reset_base=np.zeros((2, batch), np.uint8), final_step_mask=np.zeros(batch, np.uint8),
                    next_final_step_mask_base=np.zeros((2, batch), np.uint8), env_index=np.zeros(batch, np.int32), sample_index=np.zeros(batch, np.int32))

    def gather_batch(self, st, batch, rng, max_episode_length=200):
        """One gather_batch on the replay buffers of the state dict `st` (engine `rng` from new_rng, advanced in place)."""
        N, capacity = st["replay_data"].shape[:2]
        out = self.new_batch(batch)
        self.lib.orc_gather_batch(N, capacity, max_episode_length, batch, rng, st["replay_data"], st["counters"], out["oa_base"], out["rewards"], out["terminated"],
                                  out["reset"], out["next_reset_base"], out["final_step_mask"], out["next_final_step_mask_base"], out["env_index"], out["sample_index"])
        return out

    # --- L2F quadrotor -------------------------------------------------------------------------------------------
    L2F_STATE_LIMITS = np.array([100000, 100000, 100000], np.float32)      # the reference harness' STATE_LIMIT_* (position, velocity, angular velocity)

    def l2f_steps(self, dynamics, dt, states, actions, n_steps=1, state_limits=None):
        """n_steps x step() of the L2F quadrotor (harness configuration) per row: states [n, 23], actions [n, 4] (normalised, constant over the
        steps), dynamics = the 85 floats of the reference's parameters.dynamics. Returns the states afterwards."""
        states, actions = np.ascontiguousarray(states, np.float32), np.ascontiguousarray(actions, np.float32)
        out = np.empty_like(states)
        limits = self.L2F_STATE_LIMITS if state_limits is None else np.ascontiguousarray(state_limits, np.float32)
        self.lib.orc_l2f_steps(states.shape[0], n_steps, np.ascontiguousarray(dynamics, np.float32), np.float32(dt), limits, states, actions, out)
        return out

    def l2f_functions(self, dynamics, dt, mdp, states, actions, next_states):
        """(observe(state) [n, 18], reward(state, action, next_state) [n], terminated(next_state) [n]) of the L2F environment, row by row."""
        n = states.shape[0]
        obs, rew, term = np.empty((n, 18), np.float32), np.empty(n, np.float32), np.empty(n, np.uint8)
        self.lib.orc_l2f_functions(n, np.ascontiguousarray(dynamics, np.float32), np.float32(dt), np.ascontiguousarray(mdp, np.float32), np.ascontiguousarray(states, np.float32),
                                   np.ascontiguousarray(actions, np.float32), np.ascontiguousarray(next_states, np.float32), obs, rew, term)
        return obs, rew, term

    def l2f_initial_states_from_draws(self, init, dynamics, u, normals):
        """sample_initial_state of the L2F environment as a function of its draws: u [n, 17] canonical uniforms, normals [n, 6] standard normals
        (see orc_l2f_initial_state_from_draws); action limits = the last two floats of the dynamics block. Returns [n, 23]."""
        u, normals = np.ascontiguousarray(u, np.float32), np.ascontiguousarray(normals, np.float32)
        init, d = np.ascontiguousarray(init, np.float32), np.ascontiguousarray(dynamics, np.float32)
        out = np.empty((u.shape[0], 23), np.float32)
        for e in range(u.shape[0]):
            self.lib.orc_l2f_initial_state_from_draws(init, d[83], d[84], u[e], normals[e], out[e])
        return out

    def l2f_sample_initial_states(self, seed, n, init, dynamics):
        """n x sample_initial_state on one engine seeded with `seed`, in the reference's draw order: [n, 23]."""
        d = np.ascontiguousarray(dynamics, np.float32)
        out = np.empty((n, 23), np.float32)
        self.lib.orc_l2f_sample_initial_states(seed, n, np.ascontiguousarray(init, np.float32), d[83], d[84], out)
        return out

    def l2f_rollout(self, shape, params, dynamics, dt, mdp, states, episode_step, truncated, episode_return, reset_states, T, step_limit=500, state_limits=None):
        """The runner loop on the L2F environment: reset_states [R, N, 23]; returns obs, act, rew, terminated and the runner state afterwards."""
        N = states.shape[0]
        states, episode_step, truncated, episode_return = (np.array(states, np.float32), np.array(episode_step, np.int32), np.array(truncated, np.uint8),
                                                           np.array(episode_return, np.float32))
        reset_states = np.ascontiguousarray(reset_states, np.float32)
        assert reset_states.shape[1:] == (N, 23)
        limits = self.L2F_STATE_LIMITS if state_limits is None else np.ascontiguousarray(state_limits, np.float32)
        obs, act, rew, term = np.empty((T * N, 18), np.float32), np.empty((T * N, 4), np.float32), np.empty(T * N, np.float32), np.empty(T * N, np.uint8)
        rc = self.lib.orc_l2f_rollout(C.byref(shape), np.ascontiguousarray(params, np.float32), np.ascontiguousarray(dynamics, np.float32), np.float32(dt), limits,
                                      np.ascontiguousarray(mdp, np.float32), N, T, states, episode_step, truncated, episode_return, reset_states, reset_states.shape[0], step_limit,
                                      obs, act, rew, term)
        if rc != 0:
            raise RuntimeError(f"orc_l2f_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, terminated=term, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    GATHER_FROM_INITIAL_STATE, GATHER_RANDOM_LENGTH, GATHER_FIRST_STEP_TARGET, GATHER_DETERMINISTIC = 1, 2, 4, 8

    @staticmethod
    def new_sequence_batch(batch, L):
        """Zeroed output arrays of one gather_batch with sequence length L (padded length L + 1)."""
        u8 = np.uint8
        return dict(oa_base=np.zeros((L + 1, batch, 4), np.float32), rewards=np.zeros((L, batch), np.float32), terminated=np.zeros((L, batch), u8),
                    reset=np.zeros((L, batch), u8), next_reset_base=np.zeros((L + 1, batch), u8), final_step_mask=np.zeros((L, batch), u8),
                    next_final_step_mask_base=np.zeros((L + 1, batch), u8))

    def gather_batch_sequences(self, st, batch, L, flags, rng, max_episode_length=200, nominal_probability=0.5):
        """One gather_batch with sequence length L on the replay buffers of the state dict `st` (engine `rng` from new_rng, advanced in place);
        flags = GATHER_* bits. max_episode_length is the ENVIRONMENT's episode step limit (off_policy_runner.h:41)."""
        N, capacity = st["replay_data"].shape[:2]
        out = self.new_sequence_batch(batch, L)
        self.lib.orc_gather_batch_sequences(N, capacity, max_episode_length, batch, L, flags, nominal_probability, rng, st["replay_data"], st["episode_start"], st["counters"],
                                            out["oa_base"], out["rewards"], out["terminated"], out["reset"], out["next_reset_base"], out["final_step_mask"],
                                            out["next_final_step_mask_base"])
        return out

    # --- on-policy collect ---------------------------------------------------------------------------------
    def new_rng(self, seed):
        rng = C.create_string_buffer(4 * 624 + 16)
        self.lib.orc_rng_init(rng, seed)
        return rng

    def collect_tables(self, rng, N, T, episode_step, truncated, step_limit, R):
        """Draws of one collect call (engine state `rng` from new_rng, advanced in place): reset table [R,N,2], noise [T,N]."""
        table, noise = np.zeros((R, N, 2), np.float32), np.empty((T, N), np.float32)
        used = self.lib.orc_collect_tables(rng, N, T, episode_step, truncated, step_limit, table, R, noise)
        if used < 0:
            raise ValueError("reset table too small")
        return table, noise

    def pendulum_collect(self, shape, params, runner, T, step_limit, rng=None, reset_states=None, noise=None, dataset=None):
        """runner = dict(states, episode_step, truncated, episode_return), updated IN PLACE. Either rng (inline draws) or the
        two tables. Returns the dataset matrix [(T+1)*N, 13]."""
        N = runner["states"].shape[0]
        ds = np.zeros(((T + 1) * N, 13), np.float32) if dataset is None else dataset
        R = 0 if reset_states is None else reset_states.shape[0]
        rc = self.lib.orc_pendulum_collect(C.byref(shape), params, N, T, runner["states"], runner["episode_step"], runner["truncated"],
                                           runner["episode_return"], rng, _opt(reset_states), R, _opt(noise), step_limit, ds, 13)
        if rc != 0:
            raise RuntimeError(f"orc_pendulum_collect rc={rc}")
        return ds

    def gae(self, rewards, all_values, terminated, truncated, N, steps, gamma=0.99, lam=0.95, ignore_termination=False):
        adv, tgt = np.empty(steps * N, np.float32), np.empty(steps * N, np.float32)
        self.lib.orc_gae(rewards, all_values, terminated, truncated, adv, tgt, N, steps, gamma, lam, int(ignore_termination))
        return adv, tgt


    def normal_functions(self, mean, log_std, value):
        n = mean.size
        lp, dm, dl = np.empty(n, np.float32), np.empty(n, np.float32), np.empty(n, np.float32)
        self.lib.orc_normal_functions(n, mean, log_std, value, lp, dm, dl)
        return lp, dm, dl

    def ppo_policy_gradient(self, current_actions, rollout_actions, log_std, rollout_log_probs, advantages, d_log_std=None,
                            epsilon_clip=0.2, entropy_coefficient=0.01, advantage_epsilon=1e-8, normalize_advantage=True, learn_action_std=True):
        B, A = current_actions.shape
        d_actions = np.empty((B, A), np.float32)
        d_log_std = np.zeros(A, np.float32) if d_log_std is None else d_log_std.copy()
        self.lib.orc_ppo_policy_gradient(current_actions, rollout_actions, log_std, rollout_log_probs, advantages, d_actions, d_log_std, B, A,
                                         epsilon_clip, entropy_coefficient, advantage_epsilon, int(normalize_advantage), int(learn_action_std))
        return d_actions, d_log_std


class ReferenceCuda:
    """The real reference on ITS OWN CUDA device (libref_cuda.so: cuBLAS SGEMM + the reference's kernels). Present only where it was built;
    needs a GPU to run. Arguments that are device memory are passed as raw addresses (torch tensors' data_ptr())."""
    CASES = {"c5_b65536": (0, 65536, 64, 16, 152336), "c5_b1024": (1, 1024, 64, 16, 152336), "c3_b256": (2, 256, 4, 1, 67329)}

    def __init__(self):
        if not os.path.exists(REF_CUDA_SO):
            raise FileNotFoundError(REF_CUDA_SO)
        self.lib = C.CDLL(REF_CUDA_SO)
        self.lib.ref_cuda_mlp_train.argtypes = [C.c_int, C.c_longlong, C.c_int, C.c_int, _f32p, C.c_void_p, C.c_void_p, C.POINTER(C.c_float), _f32p, _f32p]
        self.lib.ref_cuda_mlp_train.restype = C.c_int
        self.lib.ref_cuda_rollout.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        self.lib.ref_cuda_rollout.restype = C.c_int

    def rollout(self, case, actor_params, steps, warmup=0):
        """`steps` timed rollouts of 200 off-policy runner steps (the reference's step<0> on its CUDA device) of the deterministic actor
        3 -> 64 -> 64 -> 1 on 65,536 ("65536env") or 512 ("512env") Pendulum environments. Returns (ms per rollout, mean episode return)."""
        params = np.ascontiguousarray(actor_params, np.float32)
        assert params.size == 4481
        ms, probe = C.c_float(), C.c_float()
        rc = self.lib.ref_cuda_rollout({"65536env": 0, "512env": 1}[case], steps, warmup, params, C.byref(ms), C.byref(probe))
        if rc != 0:
            raise RuntimeError(f"ref_cuda_rollout returned {rc}")
        return ms.value, probe.value

    def mlp_train(self, case, params, x_ptr, y_ptr, rows, steps, warmup=0):
        """`steps` training steps (zero_gradient; per chunk forward, MSE gradient weighted chunk / rows, backward; Adam) after `warmup` untimed
        ones. Returns (ms per step, parameters afterwards, gradient of the last step)."""
        which, chunk, _, _, n_params = self.CASES[case]
        params = np.ascontiguousarray(params, np.float32)
        assert params.size == n_params and rows % chunk == 0
        out, grads, ms = np.empty(n_params, np.float32), np.empty(n_params, np.float32), C.c_float()
        rc = self.lib.ref_cuda_mlp_train(which, rows, steps, warmup, params, x_ptr, y_ptr, C.byref(ms), out, grads)
        if rc != 0:
            raise RuntimeError(f"ref_cuda_mlp_train returned {rc}")
        return ms.value, out, grads


class Reference:
    """Typed wrapper around the real reference (libref_strict.so / libref_fast.so). Present only where it was built."""

    def __init__(self, kind="strict"):
        path = REF_STRICT_SO if kind == "strict" else REF_FAST_SO
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.lib = L = C.CDLL(path)
        L.ref_case_name.restype = C.c_char_p
        L.ref_case_dims.argtypes = [C.c_char_p, C.POINTER(C.c_int)]
        L.ref_mlp_run.argtypes = [C.c_char_p, C.c_void_p, C.c_uint32, C.c_void_p, C.c_void_p, C.c_int, C.c_int] + [C.c_void_p] * 7 + [C.POINTER(C.c_double)]
        L.ref_rng_uniform.argtypes = [C.c_uint32, C.c_int, C.c_float, C.c_float, _f32p]
        L.ref_rng_normal.argtypes = [C.c_uint32, C.c_int, C.c_float, C.c_float, _f32p]
        L.ref_rng_mixed.argtypes = [C.c_uint32, C.c_int, _u8p, _f32p, _f32p, _f32p]
        L.ref_pendulum_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.ref_pendulum_step.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, C.c_void_p, C.c_void_p]
        L.ref_pendulum_rollout.argtypes = [C.c_int, _f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int,
                                           _f32p, _f32p, _f32p, C.c_int]
        L.ref_pendulum_rollout.restype = C.c_int
        L.ref_gae.argtypes = [C.c_int, C.c_int, _f32p, _f32p, _u8p, _u8p, _f32p, _f32p]
        L.ref_ppo_train.argtypes = [C.c_int] * 6 + [C.c_uint32] + [_f32p] * 10 + [C.POINTER(C.c_double)]
        _u64p = np.ctypeslib.ndpointer(np.uint64, flags="C_CONTIGUOUS")
        L.ref_rng_uniform_int.argtypes = [C.c_uint32, C.c_int, _u64p, _u64p, _u64p]
        _i64p = np.ctypeslib.ndpointer(np.int64, flags="C_CONTIGUOUS")
        L.ref_offpolicy_steps.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, C.c_uint32, C.c_int, _f32p, _i64p, _f32p, _f32p, _i64p, _f32p, _i32p, _u8p, _f32p, _f32p, _f32p, _f32p]
        L.ref_acrobot_rollout.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p]
        L.ref_acrobot_step.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.ref_acrobot_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.ref_acrobot_terminating_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.ref_acrobot_terminating_rollout.argtypes = [_f32p, C.c_int, C.c_int, _f32p, _i32p, _u8p, _f32p, _f32p, C.c_int, C.c_int, _f32p, _f32p, _f32p, _u8p]
        L.ref_normalizer.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.ref_sac_updates.argtypes = [C.c_int, C.c_int, C.c_int, _f32p, C.c_float, _f32p, _f32p, _f32p, _f32p, _u8p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.ref_sample_and_squash.argtypes = [C.c_int, C.c_int, _f32p, _f32p, _f32p, C.c_float, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.ref_polyak_update.argtypes = [_f32p, _f32p, C.c_float, C.c_int, C.c_int]
        L.ref_offpolicy_gather.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _f32p, C.c_uint32, C.c_int, C.c_int, _f32p, _f32p, _u8p, _u8p, _u8p, _u8p, _u8p, C.c_void_p]
        L.ref_l2f_parameters.argtypes = [_f32p, C.POINTER(C.c_float), C.POINTER(C.c_float)]
        L.ref_l2f_mdp.argtypes = [_f32p]
        L.ref_l2f_init.argtypes = [_f32p]
        L.ref_l2f_functions.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _u8p]
        L.ref_l2f_initial_states.argtypes = [C.c_uint32, C.c_int, _f32p]
        L.ref_l2f_steps.argtypes = [C.c_int, C.c_int, _f32p, _f32p, _f32p]
        L.ref_offpolicy_gather_sequences.argtypes = [C.c_int, C.c_int, _f32p, C.c_uint32, C.c_int, C.c_int, _f32p, _f32p, _u8p, _u8p, _u8p, _u8p, _u8p, C.c_void_p]
        L.ref_collect.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, _f32p, C.c_uint32, C.c_int, _f32p, _f32p, _i32p, _u8p, _f32p, C.POINTER(C.c_uint64)]
        L.ref_normal_functions.argtypes = [C.c_int, _f32p, _f32p, _f32p, _f32p, _f32p, _f32p]
        L.ref_mlp_c5_chunked.argtypes = [C.c_int, _f32p, _f32p, _f32p, C.c_int, C.c_int, C.c_int] + [_f32p] * 6

    def cases(self):
        out = {}
        for i in range(self.lib.ref_num_cases()):
            name = self.lib.ref_case_name(i).decode()
            d = (C.c_int * 7)()
            self.lib.ref_case_dims(name.encode(), d)
            out[name] = dict(batch=d[0], input_dim=d[1], hidden_dim=d[2], output_dim=d[3], num_layers=d[4], hidden_act=d[5], output_act=d[6])
        return out

    @staticmethod
    def case_shape(c):
        dims = [c["hidden_dim"]] * (c["num_layers"] - 1) + [c["output_dim"]]
        acts = [c["hidden_act"]] * (c["num_layers"] - 1) + [c["output_act"]]
        return MlpShape.make(c["input_dim"], dims, acts)

    def mlp_run(self, name, params, x, target, mode, n_steps=0, init_seed=0):
        c = self.cases()[name]
        shape = self.case_shape(c)
        n, B = shape.num_params(), c["batch"]
        acts = B * sum(shape.layer_dims())
        res = dict(params=np.empty(n, np.float32), grads=np.empty(n, np.float32), m=np.empty(n, np.float32), v=np.empty(n, np.float32),
                   pre=np.empty(acts, np.float32) if mode != 0 else None,
                   out=np.empty(acts if mode != 0 else B * c["output_dim"], np.float32),
                   d_input=np.empty((B, c["input_dim"]), np.float32) if mode == 3 else None)
        sec = C.c_double()
        rc = self.lib.ref_mlp_run(name.encode(), _opt(params), init_seed, _opt(x), _opt(target), mode, n_steps, _opt(res["params"]), _opt(res["grads"]),
                                  _opt(res["m"]), _opt(res["v"]), _opt(res["pre"]), _opt(res["out"]), _opt(res["d_input"]), C.byref(sec))
        assert rc == 0, name
        res["seconds"] = sec.value
        return res

    def mlp_c5_chunked(self, chunk_rows, params, x, target, do_step=True):
        """One optimizer step of the 64 -> 256 -> 256 -> 256 -> 16 network over x.shape[0] / chunk_rows chunks (gradients accumulate over the
        chunks, each weighted chunk_rows / rows), through the reference's own zero_gradient / forward / mse::gradient / backward / step."""
        shape = C5_SHAPE()
        n, rows = shape.num_params(), x.shape[0]
        assert rows % chunk_rows == 0
        acts = chunk_rows * sum(shape.layer_dims())
        res = dict(params=np.empty(n, np.float32), grads=np.empty(n, np.float32), m=np.empty(n, np.float32), v=np.empty(n, np.float32),
                   pre=np.empty(acts, np.float32), out=np.empty(acts, np.float32))
        rc = self.lib.ref_mlp_c5_chunked(chunk_rows, params, np.ascontiguousarray(x), np.ascontiguousarray(target), rows // chunk_rows, rows, 1 if do_step else 0,
                                         res["params"], res["grads"], res["m"], res["v"], res["pre"], res["out"])
        assert rc == 0
        return res

    COLLECT_CASES = ((64, 64, 100, 1), (5, 37, 20, 1), (7, 50, 0, 1), (33, 25, 10, 2))   # (N, steps, step_limit, hidden activation id)

    def collect(self, N, steps, step_limit, hidden_act, actor_params, seed, n_collects):
        """n_collects consecutive collect() calls of the reference's OnPolicyRunner on a fresh runner. Returns the data matrix
        after each call [n_collects, (steps+1)*N, 13] and the final runner state."""
        ds = np.empty((n_collects, (steps + 1) * N, 13), np.float32)
        runner = dict(states=np.empty((N, 2), np.float32), episode_step=np.empty(N, np.int32), truncated=np.empty(N, np.uint8),
                      episode_return=np.empty(N, np.float32))
        step = C.c_uint64(0)
        rc = self.lib.ref_collect(N, steps, step_limit, hidden_act, actor_params, seed, n_collects, ds, runner["states"], runner["episode_step"],
                                  runner["truncated"], runner["episode_return"], C.byref(step))
        if rc != 0:
            raise KeyError("no such collect case")
        runner["step"] = step.value
        return ds, runner

    PPO_TRAIN_CASES = ((64, 64, 4096, 1), (64, 64, 512, 2), (5, 37, 37, 3))      # (N, steps, minibatch, epochs)
    PPO_TRAIN_SHUFFLE_CASES = ((64, 64, 512, 2), (5, 37, 37, 3))

    PPO_TRAIN_ANT_CASES = ((64, 1024, 2048, 1, False), (64, 1024, 2048, 1, True), (64, 1024, 2048, 10, True))   # + shuffle flag; env="ant"

    OFFPOLICY_CASES = ((8, 64, 50), (33, 40, 17))      # (N, replay capacity, episode step limit)

    def offpolicy_steps(self, N, capacity, step_limit, actor_params, seed, n_steps):
        """n_steps x step<0>() of the reference's OffPolicyRunner on a fresh runner; returns a state dict like Oracle.new_offpolicy_state."""
        st = Oracle.new_offpolicy_state(N, capacity)
        rc = self.lib.ref_offpolicy_steps(N, capacity, step_limit, actor_params, seed, n_steps, st["replay_data"], st["episode_start"], st["replay_states"],
                                          st["replay_next_states"], st["counters"], st["states"], st["episode_step"], st["truncated"], st["episode_return"],
                                          st["buf_obs"], st["buf_act"], st["buf_next_obs"])
        if rc != 0:
            raise KeyError("no such off-policy runner case")
        return st

    def acrobot_step(self, states, actions):
        n = states.shape[0]
        ns, r, obs, nobs = np.empty((n, 4), np.float32), np.empty(n, np.float32), np.empty((n, 6), np.float32), np.empty((n, 6), np.float32)
        self.lib.ref_acrobot_step(n, np.ascontiguousarray(states, np.float32), np.ascontiguousarray(actions.reshape(-1), np.float32), ns, r, obs, nobs)
        return ns, r, obs, nobs

    def acrobot_initial_states(self, seed, n):
        s = np.empty((n, 4), np.float32)
        self.lib.ref_acrobot_initial_states(seed, n, s)
        return s

    def acrobot_terminating_initial_states(self, seed, n):
        s = np.empty((n, 4), np.float32)
        self.lib.ref_acrobot_terminating_initial_states(seed, n, s)
        return s

    def acrobot_terminating_rollout(self, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=500):
        """The reference's own observe / step / reward / terminated of rl::environments::Acrobot under the runner loop; reset_states [R, N, 4]."""
        N = states.shape[0]
        states, episode_step, truncated, episode_return = (np.array(states, np.float32), np.array(episode_step, np.int32), np.array(truncated, np.uint8),
                                                           np.array(episode_return, np.float32))
        reset_states = np.ascontiguousarray(reset_states, np.float32)
        obs, act, rew, term = np.empty((T * N, 6), np.float32), np.empty((T * N, 1), np.float32), np.empty((T * N, 1), np.float32), np.empty(T * N, np.uint8)
        rc = self.lib.ref_acrobot_terminating_rollout(np.ascontiguousarray(params, np.float32), N, T, states, episode_step, truncated, episode_return, reset_states,
                                                      reset_states.shape[0], step_limit, obs, act, rew, term)
        if rc != 0:
            raise RuntimeError(f"ref_acrobot_terminating_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, terminated=term, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    def acrobot_rollout(self, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=500):
        N = states.shape[0]
        states, episode_step = states.copy(), episode_step.copy()
        truncated, episode_return = truncated.copy(), episode_return.copy()
        obs, act, rew = np.empty((T * N, 6), np.float32), np.empty((T * N, 1), np.float32), np.empty((T * N, 1), np.float32)
        rc = self.lib.ref_acrobot_rollout(params, N, T, states, episode_step, truncated, episode_return, reset_states, reset_states.shape[0], step_limit, obs, act, rew)
        if rc != 0:
            raise RuntimeError(f"ref_acrobot_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)

    NORMALIZER_CASES = ((4096, 27), (333, 3), (50, 5))            # (rows, dim) instantiated in ref_driver.cpp

    def normalizer(self, data):
        """The reference's RunningNormalizer::update on data [U, R, D], then set_statistics / evaluate of its standardize layer on the last batch
        (same dict as Oracle.normalizer)."""
        U, R, D = data.shape
        means, stds = np.empty((U, D), np.float32), np.empty((U, D), np.float32)
        lm, lp, out = np.empty(D, np.float32), np.empty(D, np.float32), np.empty((R, D), np.float32)
        rc = self.lib.ref_normalizer(R, D, U, np.ascontiguousarray(data, np.float32), means, stds, lm, lp, out)
        if rc != 0:
            raise KeyError("no such normalizer case")
        return dict(mean=means, std=stds, layer_mean=lm, layer_precision=lp, output=out)

    SAC_CASES = ((256, 64), (100, 32))                          # (batch, hidden width) instantiated in ref_driver.cpp; (256, 256) too, for the timed baseline

    def sac_updates(self, batch, hidden, actor_params, log_alpha, critic_params, target_params, oa_base, rewards, terminated, noise_critic, noise_actor):
        """The reference's train_critic x 2, update_critic_targets, train_actor per update (same dict as Oracle.sac_updates)."""
        U = oa_base.shape[0]
        na, nc = actor_params.size, critic_params.shape[1]
        f = lambda a: np.ascontiguousarray(a, np.float32)
        actor_out, la_out = np.empty((3, na), np.float32), np.empty(3, np.float32)
        critic_out, target_out, tv = np.empty((2, 3, nc), np.float32), np.empty((2, nc), np.float32), np.empty(batch, np.float32)
        rc = self.lib.ref_sac_updates(batch, hidden, U, f(actor_params), log_alpha, f(critic_params), f(target_params), f(oa_base), f(rewards),
                                      np.ascontiguousarray(terminated, np.uint8), f(noise_critic), f(noise_actor), actor_out, la_out, critic_out, target_out, tv)
        if rc != 0:
            raise KeyError("no such SAC case")
        return dict(actor=tuple(actor_out), log_alpha=tuple(la_out), critics=[tuple(critic_out[c]) for c in range(2)], targets=[target_out[c] for c in range(2)],
                    target_values=tv)

    SAS_CASES = ((256, 1), (100, 8), (7, 3))                   # (batch, action dim) instantiated in ref_driver.cpp

    def sample_and_squash(self, inp, noise, d_output, log_alpha):
        """The reference's sample_and_squash LayerGradient: forward with external noise, then backward_full (same dict as Oracle.sample_and_squash)."""
        B, A = noise.shape
        inp, noise, d_output = (np.ascontiguousarray(x, np.float32) for x in (inp, noise, d_output))
        out = dict(pre_squashing=np.empty((B, A), np.float32), output=np.empty((B, A), np.float32), log_probs=np.empty(B, np.float32),
                   d_input=np.empty((B, 2 * A), np.float32), d_log_alpha_per_sample=np.empty(B, np.float32))
        grad = np.zeros(1, np.float32)
        rc = self.lib.ref_sample_and_squash(B, A, inp, noise, d_output, log_alpha, out["pre_squashing"], out["output"], out["log_probs"], out["d_input"],
                                            out["d_log_alpha_per_sample"], grad)
        if rc != 0:
            raise KeyError("no such sample_and_squash case")
        out["log_alpha_gradient"] = grad[0]
        return out

    def polyak_update(self, source, target, polyak, square=False, n_updates=1):
        """The reference's utils::polyak::update[_squared] on [41, 29] matrices, n_updates times; returns the new target."""
        assert source.shape == (41, 29) and target.shape == (41, 29)
        out = np.ascontiguousarray(target, np.float32).copy()
        self.lib.ref_polyak_update(np.ascontiguousarray(source, np.float32), out, polyak, int(square), n_updates)
        return out

    GATHER_CASES = ((8, 64, 50, 32), (33, 40, 17, 100), (5, 300, 60, 64))        # (N, capacity, step limit, batch) instantiated in ref_driver.cpp

    def offpolicy_gather(self, N, capacity, step_limit, batch, actor_params, seed, n_steps, n_gathers):
        """n_steps x step<0>() on a fresh runner, then n_gathers x gather_batch on the same engine: a list of batch dicts (Oracle.new_batch
        without the index arrays) and the engine's next raw draw afterwards."""
        outs = [Oracle.new_batch(batch) for _ in range(n_gathers)]
        stack = {k: np.zeros((n_gathers,) + outs[0][k].shape, outs[0][k].dtype) for k in outs[0] if k not in ("env_index", "sample_index")}
        next_draw = C.c_uint32(0)
        rc = self.lib.ref_offpolicy_gather(N, capacity, step_limit, batch, actor_params, seed, n_steps, n_gathers, stack["oa_base"], stack["rewards"], stack["terminated"],
                                           stack["reset"], stack["next_reset_base"], stack["final_step_mask"], stack["next_final_step_mask_base"], C.byref(next_draw))
        if rc != 0:
            raise KeyError("no such gather_batch case")
        return [{k: v[g] for k, v in stack.items()} for g in range(n_gathers)], next_draw.value

    def l2f_parameters(self):
        """(dynamics [85] floats = the reference's parameters.dynamics of the default parameter set, dt, action noise std)"""
        d, dt, noise = np.zeros(85, np.float32), C.c_float(), C.c_float()
        self.lib.ref_l2f_parameters(d, C.byref(dt), C.byref(noise))
        return d, dt.value, noise.value

    def l2f_mdp(self):
        """The 18 floats of the default parameter set's reward function and termination thresholds (see ref_l2f_mdp)."""
        m = np.zeros(18, np.float32)
        self.lib.ref_l2f_mdp(m)
        return m

    def l2f_init(self):
        """The 12 floats of the default parameter set's initial-state distribution (see ref_l2f_init)."""
        m = np.zeros(12, np.float32)
        self.lib.ref_l2f_init(m)
        return m

    def l2f_functions(self, states, actions, next_states):
        """(observe(state) [n, 18], reward(state, action, next_state) [n], terminated(next_state) [n]) through the reference's own functions."""
        n = states.shape[0]
        obs, rew, term = np.empty((n, 18), np.float32), np.empty(n, np.float32), np.empty(n, np.uint8)
        self.lib.ref_l2f_functions(n, np.ascontiguousarray(states, np.float32), np.ascontiguousarray(actions, np.float32), np.ascontiguousarray(next_states, np.float32), obs, rew, term)
        return obs, rew, term

    def l2f_initial_states(self, seed, n):
        """n x sample_initial_state of the L2F environment on one engine (nominal parameters): [n, 23]."""
        out = np.empty((n, 23), np.float32)
        self.lib.ref_l2f_initial_states(seed, n, out)
        return out

    def l2f_steps(self, states, actions, n_steps=1):
        """n_steps x the reference's step() per row of states [n, 23] with the row's constant action [n, 4]."""
        states, actions = np.ascontiguousarray(states, np.float32), np.ascontiguousarray(actions, np.float32)
        out = np.empty_like(states)
        self.lib.ref_l2f_steps(states.shape[0], n_steps, states, actions, out)
        return out

    GATHER_SEQUENCE_CASES = ((4, 256, 20, 32, 5), (3, 300, 17, 16, 8))       # N, capacity, step limit, batch, sequence length
    GATHER_SEQUENCE_MODES = (3, 0, 1, 8, 9, 2)                                # bit 0 from the initial state, bit 1 random lengths, bit 3 deterministic

    def offpolicy_gather_sequences(self, which, mode, actor_params, seed, n_steps, n_gathers):
        """n_steps x step<0>() on a fresh runner, then n_gathers x gather_batch with the sequence length of case `which` and the sampling
        parameters of `mode`: a list of batch dicts (Oracle.new_sequence_batch) and the engine's next raw draw afterwards."""
        N, capacity, limit, batch, L = self.GATHER_SEQUENCE_CASES[which]
        proto = Oracle.new_sequence_batch(batch, L)
        stack = {k: np.zeros((n_gathers,) + v.shape, v.dtype) for k, v in proto.items()}
        next_draw = C.c_uint32(0)
        rc = self.lib.ref_offpolicy_gather_sequences(which, mode, actor_params, seed, n_steps, n_gathers, stack["oa_base"], stack["rewards"], stack["terminated"],
                                                     stack["reset"], stack["next_reset_base"], stack["final_step_mask"], stack["next_final_step_mask_base"], C.byref(next_draw))
        if rc != 0:
            raise KeyError("no such sequence gather case")
        return [{k: v[g] for k, v in stack.items()} for g in range(n_gathers)], next_draw.value

    def ppo_train(self, N, steps, batch, epochs, actor_params, critic_params, dataset, shuffle_seed=None, env="pendulum", want_seconds=False):
        """The reference's train() on a given dataset matrix [(steps+1)*N, obs + 2 act + 8]; SHUFFLE_EPOCH with an engine seeded by
        shuffle_seed, or off (None). env = "pendulum" (3 / 1, ReLU) or "ant" (27 / 8, tanh). Returns the same tuple as Oracle.ppo_train plus
        the dataset matrix as train() leaves it (plus train()'s wall time if want_seconds)."""
        obs, act = (3, 1) if env == "pendulum" else (27, 8)
        n_critic = obs * 64 + 64 + 64 * 64 + 64 + 64 + 1
        n_actor = obs * 64 + 64 + 64 * 64 + 64 + 64 * act + act + act
        assert actor_params.size == n_actor and critic_params.size == n_critic and dataset.shape == ((steps + 1) * N, obs + 2 * act + 8)
        outs = [np.empty(n_actor, np.float32) for _ in range(3)] + [np.empty(n_critic, np.float32) for _ in range(3)]
        ds_out = np.empty(dataset.shape, np.float32)
        seconds = C.c_double(0)
        rc = self.lib.ref_ppo_train(0 if env == "pendulum" else 1, N, steps, batch, epochs, int(shuffle_seed is not None), shuffle_seed or 0, actor_params,
                                    critic_params, np.ascontiguousarray(dataset, np.float32), *outs, ds_out, C.byref(seconds))
        if rc != 0:
            raise KeyError("no such PPO train case")
        return tuple(outs) + (ds_out,) + ((seconds.value,) if want_seconds else ())

    def uniform_int_stream(self, seed, lo, hi):
        lo, hi = np.ascontiguousarray(lo, np.uint64), np.ascontiguousarray(hi, np.uint64)
        out = np.empty(lo.size, np.uint64)
        self.lib.ref_rng_uniform_int(seed, lo.size, lo, hi, out)
        return out

    def gae(self, rewards, all_values, terminated, truncated, N, steps):
        adv, tgt = np.empty(steps * N, np.float32), np.empty(steps * N, np.float32)
        assert self.lib.ref_gae(N, steps, rewards, all_values, terminated, truncated, adv, tgt) == 0
        return adv, tgt

    def normal_functions(self, mean, log_std, value):
        n = mean.size
        lp, dm, dl = np.empty(n, np.float32), np.empty(n, np.float32), np.empty(n, np.float32)
        self.lib.ref_normal_functions(n, mean, log_std, value, lp, dm, dl)
        return lp, dm, dl

    def uniform_stream(self, seed, n, lo, hi):
        out = np.empty(n, np.float32)
        self.lib.ref_rng_uniform(seed, n, lo, hi, out)
        return out

    def normal_stream(self, seed, n, mean, std):
        out = np.empty(n, np.float32)
        self.lib.ref_rng_normal(seed, n, mean, std, out)
        return out

    def mixed_stream(self, seed, kinds, a, b):
        out = np.empty(len(kinds), np.float32)
        self.lib.ref_rng_mixed(seed, len(kinds), kinds, a, b, out)
        return out

    def pendulum_initial_states(self, seed, n):
        s = np.empty((n, 2), np.float32)
        self.lib.ref_pendulum_initial_states(seed, n, s)
        return s

    def pendulum_step(self, states, actions):
        n = states.shape[0]
        ns, r = np.empty((n, 2), np.float32), np.empty(n, np.float32)
        obs, nobs = np.empty((n, 3), np.float32), np.empty((n, 3), np.float32)
        self.lib.ref_pendulum_step(n, states, np.ascontiguousarray(actions.reshape(-1)), ns, r, _opt(obs), _opt(nobs))
        return ns, r, obs, nobs

    def pendulum_rollout(self, params, states, episode_step, truncated, episode_return, reset_states, T, step_limit=200, chunk=1, num_threads=1):
        N = states.shape[0]
        states, episode_step = states.copy(), episode_step.copy()
        truncated, episode_return = truncated.copy(), episode_return.copy()
        obs = np.empty((T * N, 3), np.float32)
        act = np.empty((T * N, 1), np.float32)
        rew = np.empty((T * N, 1), np.float32)
        rc = self.lib.ref_pendulum_rollout(chunk, params, N, T, states, episode_step, truncated, episode_return, reset_states,
                                           reset_states.shape[0], step_limit, obs, act, rew, num_threads)
        if rc != 0:
            raise RuntimeError(f"ref_pendulum_rollout rc={rc}")
        return dict(obs=obs, act=act, rew=rew, states=states, episode_step=episode_step, truncated=truncated, episode_return=episode_return)
