"""rl_tools_b200: Python plumbing around libb200rl.so (the sm_100a kernels behind the C ABI in include/b200rl.h).

The library is the product; this module only (a) builds it with nvcc for sm_100a, (b) loads it with ctypes and
(c) offers thin wrappers that take torch CUDA tensors (device memory + streams come from torch) and pass raw
pointers through the C ABI. There is no CPU fallback: without the built library every call raises.
"""
import ctypes as C
import os
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(HERE)
CSRC = os.path.join(HERE, "csrc")
LIB_PATH = os.path.join(HERE, "libb200rl.so")
SOURCES = ["dense.cu", "dense_tc.cu", "dense_skinny.cu", "mlp_fused.cu", "mlp_coop.cu", "adam.cu", "rollout.cu", "rollout_tc.cu", "ppo.cu", "host_api.cu", "sac.cu", "normalize.cu", "rollout_env.cu", "l2f.cu"]
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17", "-Xcompiler", "-fPIC", "-shared"]
# per-source flags: the quadrotor dynamics keep the reference's association of every expression (bit-for-bit parity with its CPU step)
SOURCE_FLAGS = {"l2f.cu": ["-fmad=false"]}

ACT = {"identity": 0, "relu": 1, "tanh": 2, "fast_tanh": 3, "sigmoid": 4}
MAX_LAYERS = 8

_lib = None


class ReplayLayout(C.Structure):
    """Mirror of b200rl_replay_layout: byte offsets of one environment's replay buffer."""
    _fields_ = [("env_stride", C.c_size_t), ("off_data", C.c_size_t), ("off_episode_start", C.c_size_t), ("off_position", C.c_size_t),
                ("off_full", C.c_size_t), ("off_current_episode_start", C.c_size_t), ("capacity", C.c_int), ("ld_data", C.c_int), ("index_bytes", C.c_int)]

    @staticmethod
    def packed(capacity, obs_dim=3, action_dim=1):
        """data [capacity, 2 obs + action + 3] f32 | episode_start [capacity] u32 | position u32 | current_episode_start u32 | full u8 (+3 pad);
        the Pendulum's row of 10 floats by default."""
        L = ReplayLayout()
        ld = 2 * obs_dim + action_dim + 3
        L.capacity, L.ld_data, L.index_bytes = capacity, ld, 4
        L.off_data, L.off_episode_start = 0, 4 * ld * capacity
        base = 4 * (ld + 1) * capacity
        L.off_position, L.off_current_episode_start, L.off_full = base, base + 4, base + 8
        L.env_stride = base + 12
        return L


class B200RLError(RuntimeError):
    pass


def build(force: bool = False, verbose: bool = False) -> str:
    """Compile every CUDA source into libb200rl.so for sm_100a (nvcc cross-compiles without a GPU)."""
    srcs = [os.path.join(CSRC, s) for s in SOURCES]
    deps = srcs + [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")] + [os.path.join(ROOT, "include", "b200rl.h"), os.path.abspath(__file__)]
    if not force and os.path.exists(LIB_PATH) and all(os.path.getmtime(LIB_PATH) >= os.path.getmtime(d) for d in deps):
        return LIB_PATH
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    # one object per source, compiled in parallel (a source is recompiled when it or any header is newer than its object), then one link;
    # the library is written next to its final name and renamed into place, so that nothing ever loads or copies a half-written file
    from concurrent.futures import ThreadPoolExecutor
    objdir = os.path.join(CSRC, "build")
    os.makedirs(objdir, exist_ok=True)
    headers = [d for d in deps if not d.endswith(".cu")]
    compile_flags = [f for f in NVCC_FLAGS if f != "-shared"]

    def compile_one(src):
        obj = os.path.join(objdir, os.path.basename(src)[:-3] + ".o")
        if not force and os.path.exists(obj) and all(os.path.getmtime(obj) >= os.path.getmtime(d) for d in [src] + headers):
            return obj, None
        res = subprocess.run([nvcc] + compile_flags + (["-Xptxas", "-v"] if verbose else []) + SOURCE_FLAGS.get(os.path.basename(src), []) + ["-c", src, "-o", obj], capture_output=True, text=True)
        if res.returncode != 0:
            raise B200RLError("nvcc failed on " + src + ":\n" + res.stdout + res.stderr)
        return obj, res.stderr

    with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 4)) as pool:
        results = list(pool.map(compile_one, srcs))
    if verbose:
        print("".join(log for _, log in results if log))
    tmp = LIB_PATH + ".tmp"
    res = subprocess.run([nvcc] + NVCC_FLAGS + [obj for obj, _ in results] + ["-o", tmp], capture_output=True, text=True)
    if res.returncode != 0:
        raise B200RLError("nvcc link failed:\n" + res.stdout + res.stderr)
    os.replace(tmp, LIB_PATH)
    return LIB_PATH


class MlpShape(C.Structure):
    """Mirror of b200rl_mlp_shape."""
    _fields_ = [("n_layers", C.c_int), ("input_dim", C.c_int), ("dims", C.c_int * MAX_LAYERS), ("acts", C.c_int * MAX_LAYERS)]

    @staticmethod
    def make(input_dim, dims, acts):
        s = MlpShape()
        s.n_layers, s.input_dim = len(dims), input_dim
        for i, (d, a) in enumerate(zip(dims, acts)):
            s.dims[i] = d
            s.acts[i] = ACT[a] if isinstance(a, str) else int(a)
        return s

    def layer_dims(self):
        return [self.dims[i] for i in range(self.n_layers)]

    def num_params(self):
        n, i = 0, self.input_dim
        for d in self.layer_dims():
            n += d * i + d
            i = d
        return n


class AdamHyper(C.Structure):
    """Mirror of b200rl_adam_hyper; defaults are the reference's DEFAULT_PARAMETERS_TENSORFLOW."""
    _fields_ = [("alpha", C.c_float), ("beta_1", C.c_float), ("beta_2", C.c_float), ("epsilon", C.c_float), ("epsilon_sqrt", C.c_float)]

    def __init__(self, alpha=1e-3, beta_1=0.9, beta_2=0.999, epsilon=1e-7, epsilon_sqrt=1e-7):
        super().__init__(alpha, beta_1, beta_2, epsilon, epsilon_sqrt)


def lib():
    """The loaded C-ABI library (ctypes). Raises if it has not been built: there is no fallback path."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise B200RLError(f"{LIB_PATH} is missing: run rl_tools_b200.build() (needs nvcc); there is no CPU fallback")
        L = C.CDLL(LIB_PATH)
        vp, i, f, sz = C.c_void_p, C.c_int, C.c_float, C.c_size_t
        shape_p = C.POINTER(MlpShape)
        L.b200rl_version.restype = i
        L.b200rl_status_string.restype = C.c_char_p
        L.b200rl_status_string.argtypes = [i]
        L.b200rl_last_cuda_error.restype = C.c_char_p
        L.b200rl_dense_forward.argtypes = [vp, vp, vp, i, vp, i, vp, i, i, i, i, i, vp]
        L.b200rl_dense_backward_scratch_bytes.argtypes = [i, i, i]
        L.b200rl_dense_backward_scratch_bytes.restype = sz
        L.b200rl_dense_backward.argtypes = [vp, vp, i, vp, i, vp, i, vp, vp, vp, i, i, i, i, i, vp, sz, vp]
        L.b200rl_dense_backward_static_scratch.argtypes = [vp, vp, i, vp, i, vp, i, vp, vp, vp, i, i, i, i, i, vp]
        L.b200rl_gae.argtypes = [vp, i, vp, i, vp, i, vp, i, vp, i, vp, i, i, i, f, f, i, vp]
        L.b200rl_ppo_scratch_bytes.argtypes = [i, i]
        L.b200rl_ppo_scratch_bytes.restype = sz
        L.b200rl_ppo_policy_gradient.argtypes = [vp, i, vp, i, vp, vp, i, vp, i, vp, i, vp, i, i, f, f, f, i, i, vp, sz, vp]
        L.b200rl_mse_gradient.argtypes = [vp, i, vp, i, vp, i, i, i, f, vp]
        L.b200rl_fill.argtypes = [vp, sz, f, vp]
        L.b200rl_mlp_num_params.argtypes = [shape_p]
        L.b200rl_mlp_num_params.restype = sz
        L.b200rl_mlp_evaluate.argtypes = [shape_p, vp, vp, i, vp, i, vp, vp, i, vp]
        L.b200rl_mlp_forward.argtypes = [shape_p, vp, vp, i, vp, vp, i, vp]
        L.b200rl_dense_forward_workspace_bytes.argtypes = [i, i, i]
        L.b200rl_dense_forward_workspace_bytes.restype = sz
        L.b200rl_dense_forward_ws.argtypes = [vp, vp, vp, i, vp, i, vp, i, i, i, i, i, vp, sz, vp]
        L.b200rl_mlp_forward_workspace_bytes.argtypes = [shape_p, i]
        L.b200rl_mlp_forward_workspace_bytes.restype = sz
        L.b200rl_mlp_evaluate_ws.argtypes = [shape_p, vp, vp, i, vp, i, vp, vp, i, vp, sz, vp]
        L.b200rl_mlp_forward_ws.argtypes = [shape_p, vp, vp, i, vp, vp, i, vp, sz, vp]
        L.b200rl_mlp_backward_scratch_bytes.argtypes = [shape_p, i]
        L.b200rl_mlp_backward_scratch_bytes.restype = sz
        L.b200rl_mlp_backward.argtypes = [shape_p, vp, vp, vp, i, vp, vp, vp, vp, vp, vp, i, vp, sz, vp]
        L.b200rl_adam_reset.argtypes = [vp, vp]
        L.b200rl_adam_step.argtypes = [vp, vp, vp, vp, sz, AdamHyper, vp, vp]
        L.b200rl_pendulum_rollout.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp]
        L.b200rl_pendulum_rollout_host.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp]
        L.b200rl_release_host_staging.argtypes = []
        L.b200rl_rng_init_host.argtypes = [vp, C.c_uint32]
        L.b200rl_dense_init_weights.argtypes = [vp, f, f, i, vp, vp, i, i, vp]
        L.b200rl_randn_host_rng.argtypes = [vp, vp, i, i, i, vp]
        L.b200rl_mse_evaluate.argtypes = [vp, i, vp, i, i, i, f, vp, vp]
        L.b200rl_mse_gradient_dev_weight.argtypes = [vp, i, vp, i, vp, i, i, i, vp, vp]
        L.b200rl_mask_count.argtypes = [vp, sz, vp, vp]
        L.b200rl_scale.argtypes = [vp, sz, f, i, vp]
        L.b200rl_fill_from_device.argtypes = [vp, sz, vp, vp]
        L.b200rl_mask_rows.argtypes = [vp, i, vp, i, vp, i, i, i, vp]
        L.b200rl_reset_table_host.argtypes = [vp, i, i, vp, vp, i, vp, i, C.POINTER(i)]
        L.b200rl_shuffle_permutation_host.argtypes = [vp, i, vp]
        L.b200rl_permute_rows_scratch_bytes.argtypes = [i, C.c_uint64]
        L.b200rl_permute_rows_scratch_bytes.restype = sz
        L.b200rl_permute_rows.argtypes = [vp, i, i, vp, C.c_uint64, vp, sz, vp]
        L.b200rl_pendulum_offpolicy_step.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, vp, i, i, vp, vp, vp, vp, C.POINTER(ReplayLayout), vp, vp, vp, vp]
        L.b200rl_collect_tables_host.argtypes = [vp, i, i, vp, vp, i, vp, i, C.POINTER(i), vp]
        L.b200rl_sample_and_squash_forward.argtypes = [vp, i, vp, i, i, i, vp, vp, i, vp, vp]
        L.b200rl_sample_and_squash_backward.argtypes = [vp, i, vp, i, vp, vp, i, vp, i, vp, f, i, i, vp, i, vp, vp, vp]
        L.b200rl_sac_target_action_values.argtypes = [vp, i, vp, i, vp, vp, vp, vp, f, i, i, i, vp, i, i, vp]
        L.b200rl_sac_min_value_d_output.argtypes = [vp, i, vp, i, vp, vp, i, i, i, vp, i, i, vp]
        L.b200rl_counter_advance.argtypes = [vp, C.c_uint64, vp]
        L.b200rl_randn_device_rng.argtypes = [vp, sz, C.c_uint64, C.c_uint, C.c_uint64, vp, vp]
        L.b200rl_gather_batch_device_counter.argtypes = [vp, C.POINTER(ReplayLayout), i, i, i, i, C.c_uint64, vp, i, vp, i, vp, vp, vp, vp, vp, vp, vp, vp]
        L.b200rl_running_normalizer_update.argtypes = [vp, i, i, i, vp, vp, C.c_uint64, vp]
        L.b200rl_standardize_set_statistics.argtypes = [vp, vp, i, vp, vp, vp]
        L.b200rl_standardize_forward.argtypes = [vp, i, vp, vp, vp, i, i, i, vp]
        L.b200rl_env_observation_dim.argtypes = [i]
        L.b200rl_env_state_dim.argtypes = [i]
        L.b200rl_env_rollout.argtypes = [i, shape_p, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp]
        L.b200rl_env_rollout_flags.argtypes = [i, shape_p, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, vp]
        L.b200rl_env_reset_dim.argtypes = [i]
        L.b200rl_polyak_update.argtypes = [vp, i, vp, i, i, i, f, i, vp]
        L.b200rl_replay_counters.argtypes = [vp, C.POINTER(ReplayLayout), i, vp, vp, vp]
        L.b200rl_gather_draws_host.argtypes = [vp, i, i, vp, vp, i, vp, vp]
        L.b200rl_gather_batch.argtypes = [vp, C.POINTER(ReplayLayout), i, i, i, i, vp, vp, i, vp, i, vp, vp, vp, vp, vp, vp, vp, vp]
        L.b200rl_gather_batch_device_rng.argtypes = [vp, C.POINTER(ReplayLayout), i, i, i, i, C.c_uint64, C.c_uint64, i, vp, i, vp, vp, vp, vp, vp, vp, vp, vp]
        L.b200rl_pendulum_collect.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, vp, i, vp, i, i, i, vp, i, vp, vp]
        L.b200rl_pendulum_collect_layers.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, vp, i, vp, i, i, i, vp, i, vp, vp]
        u64 = C.c_uint64
        L.b200rl_pendulum_collect_device_rng.argtypes = [shape_p, vp, vp, vp, vp, vp, vp, u64, u64, i, i, i, vp, i, vp, vp]
        L.b200rl_l2f_rollout.argtypes = [C.POINTER(L2fParameters), C.POINTER(C.c_float * 18), shape_p, vp, vp, vp, vp, vp, vp, i, i, i, i, vp, vp, vp, vp, vp, vp]
        L.b200rl_l2f_rollout_device_rng.argtypes = [C.POINTER(L2fParameters), C.POINTER(C.c_float * 18), C.POINTER(C.c_float * 12), shape_p, vp, vp, vp, vp, vp,
                                                    C.c_ulonglong, C.c_ulonglong, i, i, i, vp, vp, vp, vp, vp]
        L.b200rl_l2f_initial_states_from_draws.argtypes = [C.POINTER(L2fParameters), C.POINTER(C.c_float * 12), vp, vp, vp, i, vp]
        L.b200rl_l2f_offpolicy_prologue.argtypes = [C.POINTER(L2fParameters), C.POINTER(C.c_float * 12), vp, vp, vp, vp, vp, C.c_ulonglong, C.c_ulonglong, vp, i, vp, vp, vp]
        L.b200rl_l2f_offpolicy_epilogue.argtypes = [C.POINTER(L2fParameters), C.POINTER(C.c_float * 18), vp, vp, vp, vp, i, i, vp, vp, vp, C.POINTER(ReplayLayout), vp, vp]
        L.b200rl_l2f_steps.argtypes = [C.POINTER(L2fParameters), vp, vp, i, i, vp]
        L.b200rl_gather_batch_sequences.argtypes = [vp, C.POINTER(ReplayLayout), i, i, i, i, i, i, f, u64, u64, vp, i, vp, i, vp, vp, vp, vp, vp, vp, vp, vp]
        L.b200rl_pendulum_offpolicy_prologue.argtypes = [vp, vp, vp, vp, vp, u64, u64, vp, i, vp, vp, vp]
        L.b200rl_pendulum_offpolicy_epilogue.argtypes = [vp, vp, vp, vp, i, i, vp, vp, vp, vp, C.POINTER(ReplayLayout), vp, vp]
        L.b200rl_pendulum_rollout_device_rng.argtypes = [shape_p, vp, vp, vp, vp, vp, u64, u64, i, i, i, vp, vp, vp, vp, vp]
        _lib = L
    return _lib


def check(status: int, what: str = ""):
    if status != 0:
        L = lib()
        msg = L.b200rl_status_string(status).decode()
        if status == 3:
            msg += ": " + L.b200rl_last_cuda_error().decode()
        raise B200RLError(f"{what} failed with status {status} ({msg})")


def _ptr(t):
    return None if t is None else C.c_void_p(t.data_ptr())


def _stream():
    import torch
    return C.c_void_p(torch.cuda.current_stream().cuda_stream)


def _act(a):
    return ACT[a] if isinstance(a, str) else int(a)


# ------------------------------------------------------------------------------------------------------------
# Thin tensor-level wrappers (torch CUDA float32 tensors in, C ABI underneath)
# ------------------------------------------------------------------------------------------------------------
def dense_forward(W, bias, x, act, want_pre=True, y=None, pre=None, workspace=False):
    """workspace=True: the b200rl_dense_forward_ws form with a workspace of the size the library asks for (weights split once per call)."""
    import torch
    B, I = x.shape
    O = W.shape[0]
    y = torch.empty((B, O), device=x.device, dtype=torch.float32) if y is None else y
    if want_pre and pre is None:
        pre = torch.empty((B, O), device=x.device, dtype=torch.float32)
    if workspace:
        n = lib().b200rl_dense_forward_workspace_bytes(B, I, O)
        ws = torch.empty(max(n, 16), device=x.device, dtype=torch.uint8)
        check(lib().b200rl_dense_forward_ws(_ptr(W), _ptr(bias), _ptr(x), x.stride(0), _ptr(pre), pre.stride(0) if pre is not None else 0,
                                            _ptr(y), y.stride(0), B, I, O, _act(act), _ptr(ws), n, _stream()), "b200rl_dense_forward_ws")
        return pre, y
    check(lib().b200rl_dense_forward(_ptr(W), _ptr(bias), _ptr(x), x.stride(0), _ptr(pre), pre.stride(0) if pre is not None else 0,
                                     _ptr(y), y.stride(0), B, I, O, _act(act), _stream()), "b200rl_dense_forward")
    return pre, y


def dense_backward(W, x, pre, d_out, act, dW=None, db=None, want_d_in=True, want_grads=True):
    """Returns (dW, db, d_in); d_out is overwritten with d_pre. dW/db accumulate when given."""
    import torch
    B, I = x.shape
    O = W.shape[0]
    if want_grads:
        dW = torch.zeros((O, I), device=x.device, dtype=torch.float32) if dW is None else dW
        db = torch.zeros((O,), device=x.device, dtype=torch.float32) if db is None else db
    else:
        dW = db = None
    d_in = torch.empty((B, I), device=x.device, dtype=torch.float32) if want_d_in else None
    nbytes = lib().b200rl_dense_backward_scratch_bytes(B, I, O)
    scratch = torch.empty((max(nbytes, 4),), device=x.device, dtype=torch.uint8)
    check(lib().b200rl_dense_backward(_ptr(W), _ptr(x), x.stride(0), _ptr(pre), pre.stride(0), _ptr(d_out), d_out.stride(0), _ptr(dW), _ptr(db),
                                      _ptr(d_in), d_in.stride(0) if d_in is not None else 0, B, I, O, _act(act), _ptr(scratch), nbytes, _stream()),
          "b200rl_dense_backward")
    return dW, db, d_in


def mse_gradient(a, b, loss_weight=1.0, d_a=None):
    import torch
    d_a = torch.empty_like(a) if d_a is None else d_a
    check(lib().b200rl_mse_gradient(_ptr(a), a.stride(0), _ptr(b), b.stride(0), _ptr(d_a), d_a.stride(0), a.shape[0], a.shape[1], loss_weight, _stream()),
          "b200rl_mse_gradient")
    return d_a


def mse_gradient_dev_weight(a, b, loss_weight, d_a=None):
    """mse_gradient with the loss weight read from the one-element device tensor `loss_weight`."""
    import torch
    d_a = torch.empty_like(a) if d_a is None else d_a
    check(lib().b200rl_mse_gradient_dev_weight(_ptr(a), a.stride(0), _ptr(b), b.stride(0), _ptr(d_a), d_a.stride(0), a.shape[0], a.shape[1], _ptr(loss_weight),
                                               _stream()), "b200rl_mse_gradient_dev_weight")
    return d_a


def mask_count(mask, result):
    """result[0] = number of set entries of the uint8 / bool device tensor `mask` (the reference's cast_reduce_sum)."""
    check(lib().b200rl_mask_count(_ptr(mask), mask.numel(), _ptr(result), _stream()), "b200rl_mask_count")


def scale_(t, scale, reciprocal=False):
    """In place: t * scale, or (1 / t) * scale."""
    check(lib().b200rl_scale(_ptr(t), t.numel(), scale, int(reciprocal), _stream()), "b200rl_scale")


def fill_from_device(dst, value):
    """dst[:] = value[0] with `value` a one-element device tensor."""
    check(lib().b200rl_fill_from_device(_ptr(dst), dst.numel(), _ptr(value), _stream()), "b200rl_fill_from_device")


def mask_rows(target, mask, source=None, invert=False):
    """Rows of `target` [rows, cols] whose mask (inverted if asked) is set receive the row of `source`, or zeros without a source."""
    check(lib().b200rl_mask_rows(_ptr(source) if source is not None else None, source.stride(0) if source is not None else 0, _ptr(target), target.stride(0),
                                 _ptr(mask), target.shape[0], target.shape[1], int(invert), _stream()), "b200rl_mask_rows")


def mse_evaluate(a, b, loss_weight=1.0):
    """The loss value loss_weight * mean((a - b)^2) as a Python float (synchronises the current stream)."""
    import ctypes
    out = ctypes.c_float()
    check(lib().b200rl_mse_evaluate(_ptr(a), a.stride(0), _ptr(b), b.stride(0), a.shape[0], a.shape[1], loss_weight, ctypes.byref(out), _stream()), "b200rl_mse_evaluate")
    return out.value


def dense_init_weights(rng_state, W, bias, legacy=True, scale=1.0):
    """The reference's Kaiming-uniform init_weights of one dense layer on the host engine `rng_state` (advanced in place), written to the device
    tensors W [O, I] and bias [O]. Bounds evaluated in float32 exactly as nn/layers/dense/operations_generic.h:61-76 does."""
    import numpy as np
    f = np.float32
    O, I = W.shape
    if legacy:
        slope = np.sqrt(f(5))
        gain = np.sqrt(f(2.0) / (f(1) + slope * slope))
    else:
        gain = np.sqrt(f(2.0)) * f(scale)
    std = f(gain) / np.sqrt(f(I))
    weight_bound = np.sqrt(f(3.0)) * f(std)
    bias_bound = f(1) / np.sqrt(f(I))
    check(lib().b200rl_dense_init_weights(C.c_void_p(rng_state.ctypes.data), float(weight_bound), float(bias_bound), int(bool(legacy)), _ptr(W), _ptr(bias), I, O, _stream()),
          "b200rl_dense_init_weights")


def randn_host_rng(rng_state, dst):
    """Fills the device matrix dst [rows, cols] (any row stride) with standard normals from the host engine, in the reference's order."""
    check(lib().b200rl_randn_host_rng(C.c_void_p(rng_state.ctypes.data), _ptr(dst), dst.stride(0), dst.shape[0], dst.shape[1], _stream()), "b200rl_randn_host_rng")
    return dst


def gae(rewards, all_values, terminated, truncated, n_envs, steps, gamma=0.99, lam=0.95, ignore_termination=False):
    """Column tensors ([rows] or [rows, 1] views with any row stride) -> (advantages, target_values), both [steps * n_envs]."""
    import torch
    adv = torch.empty(steps * n_envs, device=rewards.device, dtype=torch.float32)
    tgt = torch.empty_like(adv)
    check(lib().b200rl_gae(_ptr(rewards), rewards.stride(0), _ptr(all_values), all_values.stride(0), _ptr(terminated), terminated.stride(0),
                           _ptr(truncated), truncated.stride(0), _ptr(adv), 1, _ptr(tgt), 1, n_envs, steps, gamma, lam, int(ignore_termination), _stream()), "b200rl_gae")
    return adv, tgt


def ppo_policy_gradient(current_actions, rollout_actions, log_std, rollout_log_probs, advantages, d_log_std, epsilon_clip=0.2, entropy_coefficient=0.01,
                        advantage_epsilon=1e-8, normalize_advantage=True, learn_action_std=True, d_actions=None, scratch=None):
    """d_log_std is accumulated in place; returns d_actions [B, A]. scratch: a dict that keeps the device scratch buffer between calls
    (required under CUDA graph capture, where nothing may be allocated)."""
    import torch
    B, A = current_actions.shape
    d_actions = torch.empty((B, A), device=current_actions.device, dtype=torch.float32) if d_actions is None else d_actions
    nbytes = lib().b200rl_ppo_scratch_bytes(B, A)
    if scratch is not None:
        if scratch.get("bytes", -1) < nbytes:
            scratch["buffer"], scratch["bytes"] = torch.empty(nbytes, device=current_actions.device, dtype=torch.uint8), nbytes
        scratch = scratch["buffer"]
    else:
        scratch = torch.empty(nbytes, device=current_actions.device, dtype=torch.uint8)
    check(lib().b200rl_ppo_policy_gradient(_ptr(current_actions), current_actions.stride(0), _ptr(rollout_actions), rollout_actions.stride(0), _ptr(log_std),
                                           _ptr(rollout_log_probs), rollout_log_probs.stride(0), _ptr(advantages), advantages.stride(0), _ptr(d_actions),
                                           d_actions.stride(0), _ptr(d_log_std), B, A, epsilon_clip, entropy_coefficient, advantage_epsilon,
                                           int(normalize_advantage), int(learn_action_std), _ptr(scratch), nbytes, _stream()), "b200rl_ppo_policy_gradient")
    return d_actions


def fill(t, value):
    check(lib().b200rl_fill(_ptr(t), t.numel(), float(value), _stream()), "b200rl_fill")


class Mlp:
    """An MLP on flat arenas (params / grads / Adam moments), mirroring the verbs of nn_models::mlp in the reference:
    evaluate, forward, backward, zero_gradient, reset_optimizer_state, step."""

    def __init__(self, input_dim, dims, acts, batch, device="cuda", extra_params=0):
        import torch
        self.shape = MlpShape.make(input_dim, dims, acts)
        self.batch = batch
        self.device = device
        n = self.shape.num_params()
        assert n == lib().b200rl_mlp_num_params(C.byref(self.shape))
        z = lambda *s: torch.zeros(*s, device=device, dtype=torch.float32)
        # extra_params: further parameters optimised together with the network (e.g. the PPO actor's log_std,
        # nn_models/mlp_unconditional_stddev/network.h:11-27), stored behind the layers in the same arenas
        self.n_mlp, self.n_extra = n, extra_params
        n = n + extra_params
        self.params, self.grads, self.m, self.v = z(n), z(n), z(n), z(n)
        width = max([input_dim] + list(dims))
        self.tick, self.tock = z(batch, width), z(batch, width)
        acts_n = batch * sum(dims)
        self.pre, self.out = z(acts_n), z(acts_n)
        self.adam_state = torch.zeros(4, device=device, dtype=torch.int32)
        nbytes = lib().b200rl_mlp_backward_scratch_bytes(C.byref(self.shape), batch)
        self.scratch_bytes = nbytes
        self.scratch = torch.empty(max(nbytes, 4), device=device, dtype=torch.uint8)
        # forward workspace: the weights' tensor-core operand image of the layer in flight (0 bytes for small batches)
        self.workspace_bytes = lib().b200rl_mlp_forward_workspace_bytes(C.byref(self.shape), batch)
        self.workspace = torch.empty(max(self.workspace_bytes, 16), device=device, dtype=torch.uint8)
        self.hyper = AdamHyper()
        self.reset_optimizer_state()

    def extra(self, arena="params"):
        """View of the extra parameters (or their gradient / moments) behind the layers."""
        return getattr(self, arena)[self.n_mlp:]

    def save_code(self, name, batch=1):
        """The network as C++ source in the reference's export format (what its `save_code` writes for a forward-only MLP and its
        checkpoint step stores as checkpoint.h): see rl_tools_b200.export. Copies the parameters to the host."""
        from . import export
        names = {v: k for k, v in ACT.items()}
        dims = [self.shape.dims[l] for l in range(self.shape.n_layers)]
        acts = [names[self.shape.acts[l]] for l in range(self.shape.n_layers)]
        return export.save_code(self.params[:self.n_mlp].detach().cpu().numpy(), self.shape.input_dim, dims, acts, name, batch)

    def d_out_buffer(self):
        """A reusable [batch, O_last] buffer for the loss gradient."""
        import torch
        if not hasattr(self, "_d_out"):
            self._d_out = torch.empty((self.batch, self.shape.dims[self.shape.n_layers - 1]), device=self.device, dtype=torch.float32)
        return self._d_out

    def output(self):
        O = self.shape.dims[self.shape.n_layers - 1]
        return self.out[-self.batch * O:].view(self.batch, O)

    def evaluate(self, x, y=None):
        import torch
        O = self.shape.dims[self.shape.n_layers - 1]
        y = torch.empty((x.shape[0], O), device=x.device, dtype=torch.float32) if y is None else y
        ws_ok = x.shape[0] <= self.batch          # the workspace was sized for self.batch rows (the plan depends on the batch)
        check(lib().b200rl_mlp_evaluate_ws(C.byref(self.shape), _ptr(self.params), _ptr(x), x.stride(0), _ptr(y), y.stride(0), _ptr(self.tick), _ptr(self.tock),
                                           x.shape[0], _ptr(self.workspace) if ws_ok else None, self.workspace_bytes if ws_ok else 0, _stream()), "b200rl_mlp_evaluate")
        return y

    def forward(self, x):
        assert x.shape[0] == self.batch
        check(lib().b200rl_mlp_forward_ws(C.byref(self.shape), _ptr(self.params), _ptr(x), x.stride(0), _ptr(self.pre), _ptr(self.out), self.batch,
                                          _ptr(self.workspace), self.workspace_bytes, _stream()), "b200rl_mlp_forward")
        return self.output()

    def backward(self, x, d_out, d_input=None, accumulate_gradients=True):
        """accumulate_gradients=False is the reference's backward_input: only d_input is computed, the parameter gradients stay untouched."""
        check(lib().b200rl_mlp_backward(C.byref(self.shape), _ptr(self.params), _ptr(self.grads) if accumulate_gradients else None, _ptr(x), x.stride(0), _ptr(self.pre), _ptr(self.out),
                                        _ptr(d_out), _ptr(d_input), _ptr(self.tick), _ptr(self.tock), self.batch, _ptr(self.scratch), self.scratch_bytes,
                                        _stream()), "b200rl_mlp_backward")

    def zero_gradient(self):
        fill(self.grads, 0.0)

    def reset_optimizer_state(self):
        fill(self.m, 0.0)
        fill(self.v, 0.0)
        check(lib().b200rl_adam_reset(_ptr(self.adam_state), _stream()), "b200rl_adam_reset")

    def step(self):
        check(lib().b200rl_adam_step(_ptr(self.params), _ptr(self.grads), _ptr(self.m), _ptr(self.v), self.params.numel(), self.hyper,
                                     _ptr(self.adam_state), _stream()), "b200rl_adam_step")


def pendulum_rollout(shape, params, states, episode_step, truncated, episode_return, reset_states, n_steps, step_limit=200,
                     obs=None, act=None, rew=None, error_flag=None):
    """In-place on the runner state tensors; returns (obs, act, rew). All tensors live on the GPU."""
    import torch
    N = states.shape[0]
    dev = states.device
    obs = torch.empty((n_steps * N, 3), device=dev, dtype=torch.float32) if obs is None else obs
    act = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if act is None else act
    rew = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if rew is None else rew
    R = 0 if reset_states is None else reset_states.shape[0]
    check(lib().b200rl_pendulum_rollout(C.byref(shape), _ptr(params), _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return),
                                        _ptr(reset_states), R, N, n_steps, step_limit, _ptr(obs), _ptr(act), _ptr(rew), _ptr(error_flag), _stream()),
          "b200rl_pendulum_rollout")
    return obs, act, rew


def pendulum_rollout_host(shape, params, states, episode_step, truncated, episode_return, reset_states, n_steps, obs, act, rew, step_limit=200):
    """Host-buffer call (numpy arrays or pinned CPU torch tensors): copies in, rolls out, copies the trajectories back."""
    def hp(a):
        if a is None:
            return None
        return C.c_void_p(a.ctypes.data) if hasattr(a, "ctypes") else C.c_void_p(a.data_ptr())
    N = states.shape[0]
    R = 0 if reset_states is None else reset_states.shape[0]
    check(lib().b200rl_pendulum_rollout_host(C.byref(shape), hp(params), hp(states), hp(episode_step), hp(truncated), hp(episode_return), hp(reset_states),
                                             R, N, n_steps, step_limit, hp(obs), hp(act), hp(rew), _stream()), "b200rl_pendulum_rollout_host")


def reset_table_host(seed, n_envs, n_steps, episode_step, truncated, step_limit, n_rounds):
    """Reference-compatible reset states [n_rounds, n_envs, 2] drawn on the host in the runner's order (numpy in/out)."""
    import numpy as np
    state = np.zeros(625, np.uint32)
    check(lib().b200rl_rng_init_host(C.c_void_p(state.ctypes.data), seed), "b200rl_rng_init_host")
    table = np.zeros((n_rounds, n_envs, 2), np.float32)
    used = C.c_int(0)
    es = np.ascontiguousarray(episode_step, np.int32)
    tr = np.ascontiguousarray(truncated, np.uint8)
    check(lib().b200rl_reset_table_host(C.c_void_p(state.ctypes.data), n_envs, n_steps, C.c_void_p(es.ctypes.data), C.c_void_p(tr.ctypes.data), step_limit,
                                        C.c_void_p(table.ctypes.data), n_rounds, C.byref(used)), "b200rl_reset_table_host")
    return table, used.value


def rng_init_host(seed):
    """State of the reference-compatible host engine (numpy uint32[625]); advanced in place by the *_tables_host calls."""
    import numpy as np
    state = np.zeros(625, np.uint32)
    check(lib().b200rl_rng_init_host(C.c_void_p(state.ctypes.data), seed), "b200rl_rng_init_host")
    return state


def collect_tables_host(rng_state, n_envs, n_steps, episode_step, truncated, step_limit, n_rounds):
    """Draws of one on-policy collect call in the reference engine's order: (reset_states [n_rounds, n_envs, 2], noise [n_steps, n_envs])."""
    import numpy as np
    table = np.zeros((max(n_rounds, 1), n_envs, 2), np.float32)
    noise = np.empty((n_steps, n_envs), np.float32)
    used = C.c_int(0)
    es = np.ascontiguousarray(episode_step, np.int32)
    tr = np.ascontiguousarray(truncated, np.uint8)
    check(lib().b200rl_collect_tables_host(C.c_void_p(rng_state.ctypes.data), n_envs, n_steps, C.c_void_p(es.ctypes.data), C.c_void_p(tr.ctypes.data),
                                           step_limit, C.c_void_p(table.ctypes.data), n_rounds, C.byref(used), C.c_void_p(noise.ctypes.data)),
          "b200rl_collect_tables_host")
    return table[:n_rounds], noise, used.value


def pendulum_collect(shape, params, log_std, states, episode_step, truncated, episode_return, reset_states, noise, n_steps, step_limit,
                     dataset=None, error_flag=None, layers=None):
    """On-policy collect into the dataset matrix [(n_steps + 1) * N, 13] (GPU tensors; runner state updated in place).
    `layers` = six separately allocated parameter tensors (W1 b1 W2 b2 W3 b3) instead of the flat arena `params`."""
    import torch
    N = states.shape[0]
    dataset = torch.zeros(((n_steps + 1) * N, 13), device=states.device, dtype=torch.float32) if dataset is None else dataset
    R = 0 if reset_states is None else reset_states.shape[0]
    if layers is not None:
        table = (C.c_void_p * 6)(*[t.data_ptr() for t in layers])
        check(lib().b200rl_pendulum_collect_layers(C.byref(shape), table, _ptr(log_std), _ptr(states), _ptr(episode_step), _ptr(truncated),
                                                   _ptr(episode_return), _ptr(reset_states), R, _ptr(noise), N, n_steps, step_limit, _ptr(dataset),
                                                   dataset.stride(0), _ptr(error_flag), _stream()), "b200rl_pendulum_collect_layers")
    else:
        check(lib().b200rl_pendulum_collect(C.byref(shape), _ptr(params), _ptr(log_std), _ptr(states), _ptr(episode_step), _ptr(truncated),
                                            _ptr(episode_return), _ptr(reset_states), R, _ptr(noise), N, n_steps, step_limit, _ptr(dataset),
                                            dataset.stride(0), _ptr(error_flag), _stream()), "b200rl_pendulum_collect")
    return dataset


def pendulum_collect_device_rng(shape, params, log_std, states, episode_step, truncated, episode_return, seed, first_step, n_steps, step_limit,
                                dataset=None, error_flag=None):
    """On-policy collect with resets and action noise drawn on the device (Philox-4x32-10 keyed by `seed`, one block per environment and
    step, steps counted from `first_step`): no host draw tables. Same dataset layout as pendulum_collect."""
    import torch
    N = states.shape[0]
    dataset = torch.zeros(((n_steps + 1) * N, 13), device=states.device, dtype=torch.float32) if dataset is None else dataset
    check(lib().b200rl_pendulum_collect_device_rng(C.byref(shape), _ptr(params), _ptr(log_std), _ptr(states), _ptr(episode_step), _ptr(truncated),
                                                   _ptr(episode_return), seed, first_step, N, n_steps, step_limit, _ptr(dataset), dataset.stride(0),
                                                   _ptr(error_flag), _stream()), "b200rl_pendulum_collect_device_rng")
    return dataset


def pendulum_rollout_device_rng(shape, params, states, episode_step, truncated, episode_return, seed, first_step, n_steps, step_limit=200,
                                obs=None, act=None, rew=None, error_flag=None):
    """pendulum_rollout with the initial states of truncated environments drawn on the device (see pendulum_collect_device_rng)."""
    import torch
    N = states.shape[0]
    dev = states.device
    obs = torch.empty((n_steps * N, 3), device=dev, dtype=torch.float32) if obs is None else obs
    act = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if act is None else act
    rew = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if rew is None else rew
    check(lib().b200rl_pendulum_rollout_device_rng(C.byref(shape), _ptr(params), _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return),
                                                   seed, first_step, N, n_steps, step_limit, _ptr(obs), _ptr(act), _ptr(rew), _ptr(error_flag), _stream()),
          "b200rl_pendulum_rollout_device_rng")
    return obs, act, rew


def shuffle_permutation_host(rng_state, n_rows):
    """The row permutation of one PPO epoch shuffle, drawn on the reference-compatible host engine (advanced in place): numpy int32[n_rows]."""
    import numpy as np
    perm = np.empty(n_rows, np.int32)
    check(lib().b200rl_shuffle_permutation_host(C.c_void_p(rng_state.ctypes.data), n_rows, C.c_void_p(perm.ctypes.data)), "b200rl_shuffle_permutation_host")
    return perm


def permute_rows(data, n_rows, perm, columns):
    """data[i, c] = old data[perm[i], c] for the given columns (in place on a 2-D CUDA tensor; perm = int32 CUDA tensor)."""
    import torch
    mask = 0
    for c in columns:
        mask |= 1 << int(c)
    nbytes = lib().b200rl_permute_rows_scratch_bytes(n_rows, mask)
    scratch = torch.empty(max(nbytes, 4), device=data.device, dtype=torch.uint8)
    check(lib().b200rl_permute_rows(_ptr(data), data.stride(0), n_rows, _ptr(perm), mask, _ptr(scratch), nbytes, _stream()), "b200rl_permute_rows")


def pendulum_offpolicy_step(shape, params, states, episode_step, truncated, episode_return, reset_states, step_limit, observations, actions, next_observations,
                            replay, layout, error_flag=None, layers=None):
    """One off-policy runner step with per-environment replay buffers (`replay` = uint8 CUDA tensor laid out as `layout` describes)."""
    import torch
    N = states.shape[0]
    rew = torch.empty(N, device=states.device, dtype=torch.float32)
    was = torch.empty(N, device=states.device, dtype=torch.uint8)
    table = None if layers is None else (C.c_void_p * 6)(*[t.data_ptr() for t in layers])
    check(lib().b200rl_pendulum_offpolicy_step(C.byref(shape), _ptr(params) if layers is None else None, table, _ptr(states), _ptr(episode_step), _ptr(truncated),
                                               _ptr(episode_return), _ptr(reset_states), N, step_limit, _ptr(observations), _ptr(actions), _ptr(next_observations),
                                               _ptr(replay), C.byref(layout), _ptr(rew), _ptr(was), _ptr(error_flag), _stream()), "b200rl_pendulum_offpolicy_step")


def pendulum_offpolicy_prologue(states, episode_step, truncated, episode_return, observations, was_truncated, reset_states=None, seed=0, call_index=0, call_counter=None):
    """First half of the runner step around any policy: reset-if-truncated (from reset_states [N, 2], or drawn in the kernel keyed by
    (seed, environment, call_index + *call_counter)), counters of a fresh episode, observations [N, 3]."""
    check(lib().b200rl_pendulum_offpolicy_prologue(_ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return), _ptr(reset_states), seed, call_index,
                                                   _ptr(call_counter), states.shape[0], _ptr(observations), _ptr(was_truncated), _stream()), "b200rl_pendulum_offpolicy_prologue")


def pendulum_offpolicy_epilogue(states, episode_step, truncated, episode_return, step_limit, observations, actions, next_observations, replay, layout, was_truncated):
    """Second half: environment step with the given actions [N, 1], reward, counters, next observations, replay-buffer append."""
    check(lib().b200rl_pendulum_offpolicy_epilogue(_ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return), states.shape[0], step_limit, _ptr(observations),
                                                   _ptr(actions), _ptr(next_observations), _ptr(replay), C.byref(layout), _ptr(was_truncated), _stream()),
          "b200rl_pendulum_offpolicy_epilogue")


def replay_counters(replay, layout, n_envs):
    """(position int32[N], full uint8[N]) of every environment's replay buffer, as CUDA tensors."""
    import torch
    position = torch.empty(n_envs, device=replay.device, dtype=torch.int32)
    full = torch.empty(n_envs, device=replay.device, dtype=torch.uint8)
    check(lib().b200rl_replay_counters(_ptr(replay), C.byref(layout), n_envs, _ptr(position), _ptr(full), _stream()), "b200rl_replay_counters")
    return position, full


def gather_draws_host(rng_state, n_envs, batch, position, full, capacity):
    """The draws of one gather_batch on the reference-compatible host engine (advanced in place): (env_index, sample_offset) numpy int32[batch]."""
    import numpy as np
    position, full = np.ascontiguousarray(position, np.int32), np.ascontiguousarray(full, np.uint8)
    env_index, offset = np.empty(batch, np.int32), np.empty(batch, np.int32)
    check(lib().b200rl_gather_draws_host(C.c_void_p(rng_state.ctypes.data), n_envs, batch, C.c_void_p(position.ctypes.data), C.c_void_p(full.ctypes.data), capacity,
                                         C.c_void_p(env_index.ctypes.data), C.c_void_p(offset.ctypes.data)), "b200rl_gather_draws_host")
    return env_index, offset


def new_batch(batch, obs_dim=3, action_dim=1, device="cuda"):
    """Output tensors of gather_batch (sequence length 1, padded length 2)."""
    import torch
    u8 = dict(device=device, dtype=torch.uint8)
    return dict(oa_base=torch.zeros((2, batch, obs_dim + action_dim), device=device), rewards=torch.zeros(batch, device=device),
                terminated=torch.zeros(batch, **u8), reset=torch.zeros(batch, **u8), next_reset_base=torch.zeros((2, batch), **u8),
                final_step_mask=torch.zeros(batch, **u8), next_final_step_mask_base=torch.zeros((2, batch), **u8))


def gather_batch(replay, layout, n_envs, out, env_index=None, sample_offset=None, seed=None, call_index=0, max_episode_length=200, obs_dim=3, action_dim=1,
                 error_flag=None, call_counter=None):
    """Replay-buffer sampling into the batch tensors `out` (new_batch): indices either given (int32 CUDA tensors drawn by gather_draws_host) or
    drawn inside the kernel from (seed, call_index), or from (seed, *call_counter) with call_counter a one-element int64 CUDA tensor."""
    batch = out["rewards"].shape[0]
    tail = (batch, _ptr(out["oa_base"]), out["oa_base"].stride(1), _ptr(out["rewards"]), _ptr(out["terminated"]), _ptr(out["reset"]), _ptr(out["next_reset_base"]),
            _ptr(out["final_step_mask"]), _ptr(out["next_final_step_mask_base"]), _ptr(error_flag), _stream())
    if call_counter is not None:
        check(lib().b200rl_gather_batch_device_counter(_ptr(replay), C.byref(layout), n_envs, max_episode_length, obs_dim, action_dim, seed, _ptr(call_counter), *tail),
              "b200rl_gather_batch_device_counter")
    elif seed is None:
        check(lib().b200rl_gather_batch(_ptr(replay), C.byref(layout), n_envs, max_episode_length, obs_dim, action_dim, _ptr(env_index), _ptr(sample_offset), *tail),
              "b200rl_gather_batch")
    else:
        check(lib().b200rl_gather_batch_device_rng(_ptr(replay), C.byref(layout), n_envs, max_episode_length, obs_dim, action_dim, seed, call_index, *tail),
              "b200rl_gather_batch_device_rng")
    return out


class L2fParameters(C.Structure):
    """Mirror of b200rl_l2f_parameters: dynamics = the 85 floats of the reference's parameters.dynamics; defaults of the limits = the reference
    harness' STATE_LIMIT_* constants."""
    _fields_ = [("dynamics", C.c_float * 85), ("dt", C.c_float), ("state_limit_position", C.c_float), ("state_limit_velocity", C.c_float),
                ("state_limit_angular_velocity", C.c_float)]

    @staticmethod
    def make(dynamics, dt, limits=(100000.0, 100000.0, 100000.0)):
        p = L2fParameters()
        for i, v in enumerate(dynamics):
            p.dynamics[i] = float(v)
        p.dt = float(dt)
        p.state_limit_position, p.state_limit_velocity, p.state_limit_angular_velocity = (float(x) for x in limits)
        return p


def l2f_steps(parameters, states, actions, n_steps=1):
    """n_steps x the L2F quadrotor step per row of the CUDA tensor states [n, 23] (in place) with the row's normalised action [n, 4]."""
    assert states.is_contiguous() and actions.is_contiguous() and states.shape[1] == 23 and actions.shape == (states.shape[0], 4)
    check(lib().b200rl_l2f_steps(C.byref(parameters), _ptr(states), _ptr(actions), states.shape[0], n_steps, _stream()), "b200rl_l2f_steps")
    return states


def l2f_rollout(parameters, mdp, shape, params, states, episode_step, truncated, episode_return, reset_states, n_steps, step_limit=500, obs=None, act=None, rew=None,
                terminated=None, error_flag=None):
    """The fused runner loop on the L2F quadrotor (actor 18 -> H -> H -> 4): in place on the runner state tensors; mdp = 18 floats (numpy / list) of
    the reward function and the termination thresholds; reset_states [R, N, 23] or None. Returns (obs [T*N, 18], act [T*N, 4], rew [T*N], terminated [T*N])."""
    import torch
    N, dev = states.shape[0], states.device
    obs = torch.empty((n_steps * N, 18), device=dev) if obs is None else obs
    act = torch.empty((n_steps * N, 4), device=dev) if act is None else act
    rew = torch.empty(n_steps * N, device=dev) if rew is None else rew
    terminated = torch.empty(n_steps * N, device=dev, dtype=torch.uint8) if terminated is None else terminated
    mdp_c = (C.c_float * 18)(*[float(v) for v in mdp])
    R = 0 if reset_states is None else reset_states.shape[0]
    check(lib().b200rl_l2f_rollout(C.byref(parameters), mdp_c, C.byref(shape), _ptr(params), _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return),
                                   _ptr(reset_states), R, N, n_steps, step_limit, _ptr(obs), _ptr(act), _ptr(rew), _ptr(terminated), _ptr(error_flag), _stream()),
          "b200rl_l2f_rollout")
    return obs, act, rew, terminated


def l2f_rollout_device_rng(parameters, mdp, init, shape, params, states, episode_step, truncated, episode_return, seed, first_step, n_steps, step_limit=500,
                           obs=None, act=None, rew=None, terminated=None):
    """l2f_rollout with every reset's initial state drawn in the kernel from the 12 floats of `init` (the reference's mdp.init and disturbance
    distributions), keyed by (seed, environment, first_step + step): no reset table."""
    import torch
    N, dev = states.shape[0], states.device
    obs = torch.empty((n_steps * N, 18), device=dev) if obs is None else obs
    act = torch.empty((n_steps * N, 4), device=dev) if act is None else act
    rew = torch.empty(n_steps * N, device=dev) if rew is None else rew
    terminated = torch.empty(n_steps * N, device=dev, dtype=torch.uint8) if terminated is None else terminated
    mdp_c, init_c = (C.c_float * 18)(*[float(v) for v in mdp]), (C.c_float * 12)(*[float(v) for v in init])
    check(lib().b200rl_l2f_rollout_device_rng(C.byref(parameters), mdp_c, init_c, C.byref(shape), _ptr(params), _ptr(states), _ptr(episode_step), _ptr(truncated),
                                              _ptr(episode_return), seed, first_step, N, n_steps, step_limit, _ptr(obs), _ptr(act), _ptr(rew), _ptr(terminated), _stream()),
          "b200rl_l2f_rollout_device_rng")
    return obs, act, rew, terminated


def l2f_offpolicy_prologue(parameters, states, episode_step, truncated, episode_return, observations, was_truncated, reset_states=None, init=None, seed=0, call_index=0,
                           call_counter=None):
    """First half of the off-policy runner step on the L2F quadrotor: reset-if-truncated (reset_states [n, 23], or drawn in the kernel from the
    12 floats of `init`), observations [n, 18]."""
    init_c = None if init is None else (C.c_float * 12)(*[float(v) for v in init])
    check(lib().b200rl_l2f_offpolicy_prologue(C.byref(parameters), init_c, _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return), _ptr(reset_states), seed,
                                              call_index, _ptr(call_counter), states.shape[0], _ptr(observations), _ptr(was_truncated), _stream()), "b200rl_l2f_offpolicy_prologue")


def l2f_offpolicy_epilogue(parameters, mdp, states, episode_step, truncated, episode_return, step_limit, actions, next_observations, replay, layout, was_truncated):
    """Second half: step with actions [n, 4], reward, termination, counters, next_observations [n, 18], replay-buffer append (rows of 43 floats)."""
    mdp_c = (C.c_float * 18)(*[float(v) for v in mdp])
    check(lib().b200rl_l2f_offpolicy_epilogue(C.byref(parameters), mdp_c, _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return), states.shape[0], step_limit,
                                              _ptr(actions), _ptr(next_observations), _ptr(replay), C.byref(layout), _ptr(was_truncated), _stream()), "b200rl_l2f_offpolicy_epilogue")


def l2f_initial_states_from_draws(parameters, init, uniforms, normals):
    """The reference's sample_initial_state as a function of its draws: uniforms [n, 17] in [0, 1), normals [n, 6]; returns states [n, 23]."""
    import torch
    n = uniforms.shape[0]
    states = torch.empty((n, 23), device=uniforms.device)
    init_c = (C.c_float * 12)(*[float(v) for v in init])
    check(lib().b200rl_l2f_initial_states_from_draws(C.byref(parameters), init_c, _ptr(uniforms), _ptr(normals), _ptr(states), n, _stream()), "b200rl_l2f_initial_states_from_draws")
    return states


GATHER_FROM_INITIAL_STATE, GATHER_RANDOM_LENGTH, GATHER_FIRST_STEP_TARGET, GATHER_DETERMINISTIC = 1, 2, 4, 8


def new_sequence_batch(batch, sequence_length, obs_dim=3, action_dim=1, device="cuda"):
    """Zeroed output tensors of gather_batch_sequences (SequentialBatch with SEQUENCE_LENGTH = sequence_length, padded length + 1)."""
    import torch
    L, P = sequence_length, sequence_length + 1
    u8 = dict(device=device, dtype=torch.uint8)
    return dict(oa_base=torch.zeros((P, batch, obs_dim + action_dim), device=device), rewards=torch.zeros((L, batch), device=device),
                terminated=torch.zeros((L, batch), **u8), reset=torch.zeros((L, batch), **u8), next_reset_base=torch.zeros((P, batch), **u8),
                final_step_mask=torch.zeros((L, batch), **u8), next_final_step_mask_base=torch.zeros((P, batch), **u8))


def gather_batch_sequences(replay, layout, n_envs, out, flags=None, seed=0, call_index=0, call_counter=None, max_episode_length=200, nominal_probability=0.5,
                           obs_dim=3, action_dim=1, error_flag=None):
    """gather_batch for sequences into the tensors `out` (new_sequence_batch). flags: GATHER_* bits; None = the reference's defaults for the
    sequence length (all three sampling parameters on for sequences longer than 1, off for length 1)."""
    L = out["rewards"].shape[0]
    batch = out["rewards"].shape[1]
    if flags is None:
        flags = (GATHER_FROM_INITIAL_STATE | GATHER_RANDOM_LENGTH | GATHER_FIRST_STEP_TARGET) if L > 1 else 0
    check(lib().b200rl_gather_batch_sequences(_ptr(replay), C.byref(layout), n_envs, max_episode_length, obs_dim, action_dim, L, flags, nominal_probability, seed, call_index,
                                              _ptr(call_counter), batch, _ptr(out["oa_base"]), out["oa_base"].stride(1), _ptr(out["rewards"]), _ptr(out["terminated"]),
                                              _ptr(out["reset"]), _ptr(out["next_reset_base"]), _ptr(out["final_step_mask"]), _ptr(out["next_final_step_mask_base"]),
                                              _ptr(error_flag), _stream()), "b200rl_gather_batch_sequences")
    return out


def polyak_update(source, target, polyak, square=False):
    """target = polyak * target + (1 - polyak) * source [squared], in place on 2-D CUDA tensors (row pitches honoured)."""
    rows, cols = target.shape
    check(lib().b200rl_polyak_update(_ptr(source), source.stride(0), _ptr(target), target.stride(0), rows, cols, float(polyak), int(square), _stream()),
          "b200rl_polyak_update")
    return target


def sample_and_squash_forward(inp, noise, output=None, pre_squashing=None, log_probs=None):
    """SAC policy head on inp [B, 2A] (CUDA tensors): returns (output [B, A], pre_squashing [B, A], log_probs [B])."""
    import torch
    B, A = noise.shape
    output = torch.empty((B, A), device=inp.device) if output is None else output
    pre_squashing = torch.empty((B, A), device=inp.device) if pre_squashing is None else pre_squashing
    log_probs = torch.empty(B, device=inp.device) if log_probs is None else log_probs
    check(lib().b200rl_sample_and_squash_forward(_ptr(inp), inp.stride(0), _ptr(noise), noise.stride(0), B, A, _ptr(pre_squashing), _ptr(output), output.stride(0),
                                                 _ptr(log_probs), _stream()), "b200rl_sample_and_squash_forward")
    return output, pre_squashing, log_probs


def sample_and_squash_backward(inp, noise, pre_squashing, output, d_output, log_alpha, log_alpha_gradient=None, target_entropy=-1.0, d_input=None):
    """Backward of the SAC policy head: returns (d_input [B, 2A], d_log_alpha_per_sample [B]); log_alpha_gradient (1-element tensor) is incremented."""
    import torch
    B, A = noise.shape
    d_input = torch.empty((B, 2 * A), device=inp.device) if d_input is None else d_input
    per_sample = torch.empty(B, device=inp.device)
    check(lib().b200rl_sample_and_squash_backward(_ptr(inp), inp.stride(0), _ptr(noise), noise.stride(0), _ptr(pre_squashing), _ptr(output), output.stride(0),
                                                  _ptr(d_output), d_output.stride(0), _ptr(log_alpha), target_entropy, B, A, _ptr(d_input), d_input.stride(0),
                                                  _ptr(per_sample), _ptr(log_alpha_gradient), _stream()), "b200rl_sample_and_squash_backward")
    return d_input, per_sample


def sac_target_action_values(q1_next, q2_next, rewards, terminated, next_log_probs, log_alpha, gamma=0.99, ignore_termination=False, entropy_bonus=True,
                             entropy_bonus_next_step=True, target=None):
    import torch
    B = rewards.shape[0]
    target = torch.empty((B, 1), device=rewards.device) if target is None else target
    check(lib().b200rl_sac_target_action_values(_ptr(q1_next), q1_next.stride(0), _ptr(q2_next), q2_next.stride(0), _ptr(rewards), _ptr(terminated), _ptr(next_log_probs),
                                                _ptr(log_alpha), gamma, int(ignore_termination), int(entropy_bonus), int(entropy_bonus_next_step), _ptr(target),
                                                target.stride(0), B, _stream()), "b200rl_sac_target_action_values")
    return target


def sac_min_value_d_output(q1, q2, d_critic_1_input, d_critic_2_input, action_dim, d_actor_output=None):
    import torch
    B, D = d_critic_1_input.shape
    d_actor_output = torch.empty((B, action_dim), device=q1.device) if d_actor_output is None else d_actor_output
    assert d_critic_2_input.stride(0) == d_critic_1_input.stride(0)
    check(lib().b200rl_sac_min_value_d_output(_ptr(q1), q1.stride(0), _ptr(q2), q2.stride(0), _ptr(d_critic_1_input), _ptr(d_critic_2_input), d_critic_1_input.stride(0),
                                              D - action_dim, action_dim, _ptr(d_actor_output), d_actor_output.stride(0), B, _stream()), "b200rl_sac_min_value_d_output")
    return d_actor_output


def counter_advance(call_counter, increment=1):
    """call_counter (one-element int64 CUDA tensor) += increment, on the current stream."""
    check(lib().b200rl_counter_advance(_ptr(call_counter), increment, _stream()), "b200rl_counter_advance")


def randn_device_rng(dst, seed, stream_id=0, call_index=0, call_counter=None):
    """Fills the contiguous float32 CUDA tensor dst with standard normals from the counter-based generator."""
    assert dst.is_contiguous()
    check(lib().b200rl_randn_device_rng(_ptr(dst), dst.numel(), seed, stream_id, call_index, _ptr(call_counter), _stream()), "b200rl_randn_device_rng")
    return dst


class RunningNormalizer:
    """Mirror of rl::components::RunningNormalizer (running_normalizer.h:17-30): per-column running mean and standard deviation of the
    observation batches it has seen, plus the statistics of a standardize layer derived from them (mean, precision = 1 / std)."""

    def __init__(self, dim, device="cuda"):
        import torch
        self.dim, self.age = dim, 0
        self.mean, self.std = torch.zeros(dim, device=device), torch.ones(dim, device=device)            # init(), operations_generic.h:20-25
        self.layer_mean, self.layer_precision = torch.zeros(dim, device=device), torch.ones(dim, device=device)     # init_weights of the layer

    def update(self, data):
        """Folds the batch statistics of data [rows, dim] (a 2-D CUDA tensor or view) into the running values."""
        self.age += 1
        check(lib().b200rl_running_normalizer_update(_ptr(data), data.stride(0), data.shape[0], self.dim, _ptr(self.mean), _ptr(self.std), self.age, _stream()),
              "b200rl_running_normalizer_update")

    def set_statistics(self):
        """The standardize layer takes over the running values (set_statistics, nn/layers/standardize/operations_generic.h:52-66)."""
        check(lib().b200rl_standardize_set_statistics(_ptr(self.mean), _ptr(self.std), self.dim, _ptr(self.layer_mean), _ptr(self.layer_precision), _stream()),
              "b200rl_standardize_set_statistics")

    def standardize(self, x, y=None):
        """The standardize layer's forward pass: y = (x - mean) * precision."""
        import torch
        y = torch.empty((x.shape[0], self.dim), device=x.device) if y is None else y
        check(lib().b200rl_standardize_forward(_ptr(x), x.stride(0), _ptr(self.layer_mean), _ptr(self.layer_precision), _ptr(y), y.stride(0), x.shape[0], self.dim,
                                               _stream()), "b200rl_standardize_forward")
        return y


ENV_PENDULUM, ENV_ACROBOT_SWINGUP, ENV_ACROBOT = 0, 1, 2


def env_rollout(env, shape, params, states, episode_step, truncated, episode_return, reset_states, n_steps, step_limit, obs=None, act=None, rew=None, error_flag=None,
                terminated=None):
    """The fused rollout for an environment given by id (ENV_PENDULUM, ENV_ACROBOT_SWINGUP, ENV_ACROBOT): in place on the runner state tensors,
    returns (obs [T * N, OBS], act, rew). All tensors live on the GPU. terminated: an optional uint8 tensor [T * N] that receives the
    environment's terminated flag of every transition."""
    import torch
    N, dev = states.shape[0], states.device
    O = lib().b200rl_env_observation_dim(env)
    assert states.shape[1] == lib().b200rl_env_state_dim(env)
    obs = torch.empty((n_steps * N, O), device=dev, dtype=torch.float32) if obs is None else obs
    act = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if act is None else act
    rew = torch.empty((n_steps * N, 1), device=dev, dtype=torch.float32) if rew is None else rew
    R = 0 if reset_states is None else reset_states.shape[0]
    assert reset_states is None or reset_states.shape[1:] == (N, lib().b200rl_env_reset_dim(env))
    check(lib().b200rl_env_rollout_flags(env, C.byref(shape), _ptr(params), _ptr(states), _ptr(episode_step), _ptr(truncated), _ptr(episode_return), _ptr(reset_states), R,
                                         N, n_steps, step_limit, _ptr(obs), _ptr(act), _ptr(rew), _ptr(terminated), _ptr(error_flag), _stream()), "b200rl_env_rollout_flags")
    return obs, act, rew
