#!/usr/bin/env python
"""Benchmark of the fused Pendulum rollout (actor forward + environment step), the headline metric: env-steps/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

One "step" is one pass of the hot path over one batch: ONE rollout call of 65,536 environments x 200 steps with the
actor 3 -> 64 -> 64 -> 1 (ReLU, ReLU, tanh), synthetic seeded inputs, outputs obs/act/rew buffers (262 MB, larger
than L2) written to HBM. With N > 1 (launched by torch.distributed.run, one rank per GPU) every rank rolls out its
own 65,536 environments (weak scaling, no data-path collective); the time is the max over ranks.

Prints ONE JSON line: device-timed `value` (inputs resident in HBM, CUDA events on the launching stream), `e2e`
(the host-buffer C-ABI call, host<->device copies inside the timed region), `roofline` for the rollout kernel
against the measured peak, `cpu_baseline` (the reference's own CPU path timed on this box's cores, all cores and one
thread), `clocks`, and under `secondary` the other half of the metric: `mlp_train` = forward + backward + Adam samples/s of
the 64 -> 256 -> 256 -> 256 -> 16 MLP on 2^24 rows split over the ranks with ONE NCCL all-reduce of the gradient arena per
step (strong scaling, the all-reduce timed on its own), and `rollout_strong` = the same 65,536 environments split over the
ranks. `--impl reference` times only the reference CPU implementation, on the same metric and config.

`--workload {mlp_train, collect, ppo_update, critic_train, actor_eval, sac_update, acrobot_rollout, l2f_step, l2f_rollout, l2f_sac_loop}` print secondary lines in the same JSON form (sharded MLP training,
on-policy collect, the PPO update on the Ant shapes, batch-256 critic regression steps, batch-256 actor inference, the SAC training step, the generic rollout on AcrobotSwingup); the default workload is the headline rollout.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

N_ENVS, N_STEPS, STEP_LIMIT = 65536, 200, 200
FLOP_PER_ENV_STEP = 2 * (3 * 64 + 64 * 64 + 64 * 1)      # 8,704: actor GEMMs only, no padding, no 3x for any split
BYTES_PER_ENV_STEP = 20                                   # obs 12 + action 4 + reward 4 written per env-step
WORKLOAD = "pendulum_rollout_65536env_x200step_actor3-64-64-1"
TRAFFIC_BYTES_FULL_LAUNCH = 203.1e6                       # DRAM read + write bytes of one 65,536 x 200 launch (ncu, dram__bytes_read.sum + dram__bytes_write.sum)


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(tflops=float(p["bf16_tflops"]), hbm=float(p["hbm_gbs"]), source="measured")
    return dict(tflops=1590.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    FIELDS = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self, index):
        self.index, self.samples, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append([time.time()] + parts)

    def __exit__(self, *a):
        if self.proc:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self):
        inside = [s[1:] for s in self.samples if self.t_begin is not None and self.t_begin <= s[0] <= (self.t_end or 1e30)]
        window = "timed region"
        if not inside:          # region shorter than the sampling period: use the samples taken under load around it
            inside, window = [s[1:] for s in self.samples], "warm-up + timed region"
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        sm = [int(s[0]) for s in inside]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(s[2 + i].lower().startswith("active") for s in inside)]
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": int(inside[0][1]), "reasons": reasons, "samples": len(sm), "window": window}


def synthetic_inputs(seed, n_envs):
    """Seeded stand-in for the Pendulum-v1 rollout: actor weights U(+-1/sqrt(fan_in)) (the reference initialiser's
    bound), reset states theta ~ U[-pi, pi], theta_dot ~ U[-1, 1] from the reference-compatible engine."""
    import numpy as np
    from __graft_entry__ import load_package
    pkg = load_package()
    rng = np.random.default_rng(seed)
    parts, fan_in = [], 3
    for d in (64, 64, 1):
        parts.append((rng.uniform(-1, 1, d * fan_in + d) / np.sqrt(fan_in)).astype(np.float32))
        fan_in = d
    params = np.concatenate(parts)
    table, _ = pkg.reset_table_host(seed, n_envs, N_STEPS, np.zeros(n_envs, np.int32), np.ones(n_envs, np.uint8), STEP_LIMIT, 1)
    return params, table


def rollout_config(world, workload=None):
    """The `config` object of the headline line; both arms print the same keys."""
    return {"workload": workload or WORKLOAD, "envs_per_gpu": N_ENVS, "steps_per_env": N_STEPS, "l2": "flushed between timed iterations; outputs (262 MB) exceed L2",
            "parallelism": f"env-sharded x{world}, no collective"}


class CpuReference:
    """The reference's own CPU path (oracle/_ref: unmodified RLtools headers, CPU_OPENBLAS device, project flags, all
    host threads) on the same rollout; falls back to the plain-C oracle port (1 thread) where that build is absent."""

    def __init__(self):
        import numpy as np
        self.cores = os.cpu_count() or 1
        os.environ.setdefault("OPENBLAS_NUM_THREADS", str(self.cores))
        import oracle
        rng = np.random.default_rng(0)
        parts, fan_in = [], 3
        for d in (64, 64, 1):
            parts.append((rng.uniform(-1, 1, d * fan_in + d) / np.sqrt(fan_in)).astype(np.float32))
            fan_in = d
        params = np.concatenate(parts)
        orc = oracle.Oracle()
        N = N_ENVS
        table = orc.reset_table(0, N, 1, np.zeros(N, np.int32), np.ones(N, np.uint8), STEP_LIMIT, 1)
        st, es, tr, er = np.zeros((N, 2), np.float32), np.zeros(N, np.int32), np.ones(N, np.uint8), np.zeros(N, np.float32)
        self.build = "unmodified reference headers, CPU_OPENBLAS device, -O3 -ffast-math -march=x86-64-v3 (the project's -march=native pinned: built on one machine, timed on another)"
        if os.path.exists(oracle.REF_FAST_SO):
            ref = oracle.Reference("fast")
            self.ref = ref
            self.kind, self.threads = "reference", self.cores
            self.run = lambda T, threads=None: ref.pendulum_rollout(params, st, es, tr, er, table, T, STEP_LIMIT, chunk=65536, num_threads=threads or self.cores)
        else:
            self.ref = None
            self.kind, self.threads = "port", 1
            self.build = "plain-C restatement of the reference, -O2, one thread"
            shape = oracle.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
            self.run = lambda T, threads=None: orc.pendulum_rollout(shape, params, st, es, tr, er, table, T, STEP_LIMIT)
        t0 = time.perf_counter(); self.run(2); self.sec_per_env_step_batch = (time.perf_counter() - t0) / 2

    def set_blas_threads(self, n):
        """OpenBLAS reads OPENBLAS_NUM_THREADS once at load; later changes go through its own setter."""
        if self.ref is not None:
            try:
                self.ref.lib.openblas_set_num_threads(int(n))
            except AttributeError:
                pass

    def one_thread_rate(self, seconds=4.0):
        """The reference's recommended single-thread setting (one BLAS thread, environment loop on the calling thread)."""
        if self.ref is None:
            return None
        self.set_blas_threads(1)
        try:
            t0 = time.perf_counter(); self.run(2, 1); per = (time.perf_counter() - t0) / 2
            T = int(max(2, min(N_STEPS, seconds / max(per, 1e-6))))
            t0 = time.perf_counter(); self.run(T, 1)
            return N_ENVS * T / (time.perf_counter() - t0)
        finally:
            self.set_blas_threads(self.cores)

    def sample_steps(self, seconds):
        return int(max(2, min(N_STEPS, seconds / max(self.sec_per_env_step_batch, 1e-6))))

    def timed(self, T):
        t0 = time.perf_counter(); self.run(T)
        return N_ENVS * T / (time.perf_counter() - t0)

    def describe(self, T, reps, value, one_thread=None):
        return {"value": value, "unit": "env-steps/s", "cores": self.threads, "kind": self.kind, "cores_1_value": one_thread, "build": self.build,
                "sample": f"{N_ENVS} envs x {T} steps of the same rollout (observe -> evaluate -> step/reward), median of {reps}"}


def cpu_reference_rate(seconds_total=12.0, reps=3):
    cpu = CpuReference()
    T = cpu.sample_steps(seconds_total / reps)
    value = statistics.median(cpu.timed(T) for _ in range(reps))
    return cpu.describe(T, reps, value, cpu.one_thread_rate())


def run_reference(args):
    """--impl reference: each step is a bounded sample of the workload, sized so the whole run ends within ~2 minutes."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuReference()
    T = cpu.sample_steps(120.0 / max(1, args.warmup + args.steps))
    for _ in range(args.warmup):
        cpu.timed(T)
    rates = [cpu.timed(T) for _ in range(args.steps)]
    rate = statistics.median(rates)
    line = {"impl": "reference", "metric": "env-steps/s (fused actor fwd + env step)", "value": rate, "unit": "env-steps/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * N_ENVS * T / rate, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": rollout_config(args.gpus), "timed_on": "host CPU cores",
            "cpu_baseline": cpu.describe(T, args.steps, rate, cpu.one_thread_rate()), "e2e": {"value": rate, "unit": "env-steps/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    if not args.no_secondary:
        # the second half of the metric on the reference's CPU path, under the same key and config as the repository's arm
        mlp = mlp_cpu_reference()
        if mlp is not None:
            rows = args.train_rows
            line["secondary"] = {"mlp_train": {"metric": "MLP fwd+bwd+Adam samples/s", "value": mlp["value"], "unit": "samples/s", "n_gpus": args.gpus, "higher_is_better": True,
                                               "scaling": "strong", "dtype": "f32", "data": "synthetic", "timed_on": "host CPU cores", "cpu_baseline": mlp,
                                               "config": {"workload": f"mlp_train_64-256-256-256-16_rows{rows}", "rows_per_gpu": rows // max(1, args.gpus), "chunk_rows": TRAIN_CHUNK_ROWS,
                                                          "parallelism": f"dp{args.gpus}, one NCCL all-reduce of the 609 KB gradient arena per step",
                                                          "l2": "inputs (>= 0.6 GB per pass and GPU) exceed L2"}}}
    print(json.dumps(line))


def distributed_context():
    """(torch, device, dist or None, world, rank): one process per GPU, NCCL when launched by torch.distributed.run."""
    import torch
    world, rank, local_rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        if not dist.is_initialized():
            dist.init_process_group("nccl", device_id=dev)
    return torch, dev, dist, world, rank


def mlp_cpu_reference(params=None):
    """The reference's own forward + MSE gradient + backward + Adam of the 64 -> 256 -> 256 -> 256 -> 16 network on its CPU_OPENBLAS device, batch
    1024 (its largest instantiated batch of this network in the registry), all host threads: samples/s, or None where the reference was not built."""
    import numpy as np
    import oracle
    if not os.path.exists(oracle.REF_FAST_SO):
        return None
    os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
    ref = oracle.Reference("fast")
    rs = np.random.RandomState(0)
    if params is None:
        params = (rs.uniform(-1, 1, 152336) * 0.06).astype(np.float32)
    xs, ys = rs.randn(1024, 64).astype(np.float32), rs.randn(1024, 16).astype(np.float32)
    res = ref.mlp_run("c5_b1024", params, xs, ys, 2, 100)
    return {"value": 100 * 1024 / res["seconds"], "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "reference",
            "sample": "100 train steps (forward, mse gradient, backward, Adam) at batch 1024 of the same network, CPU_OPENBLAS build"}


MLP_FLOP_PER_SAMPLE = 876544.0          # forward 303,104 + weight gradient 303,104 + input gradient 270,336 (2 M N K each, no padding)


# Rows per forward / backward pass of the training step (gradients accumulate over the chunks of a rank's rows). The workload fixes the rows
# (2^24 over all ranks), not the chunk: per-chunk fixed costs (partial-sum reductions, operand images, tile tails) made 65,536-row chunks 227 ms
# per step on one GPU against 198 / 187 / 181 / 178 / 177 ms at 2^17 .. 2^21; 2^20 leaves two chunks per rank at eight GPUs (6.6 GB of activations).
TRAIN_CHUNK_ROWS = 1 << 20


def measure_mlp_train(args, pkg, torch, dev, dist, world, rank, cpu_baseline=True):
    """Data-parallel training of the MLP 64 -> 256 -> 256 -> 256 -> 16 (ReLU, fp32) on `--train-rows` synthetic N(0,1) rows split over the
    ranks (strong scaling); one step = forward + MSE gradient + backward over the rank's rows in chunks of TRAIN_CHUNK_ROWS, ONE all-reduce of
    the flat gradient arena (NCCL), ONE fused Adam launch. Returns the result dictionary on rank 0 (None elsewhere)."""
    from rl_tools_b200 import parallel
    chunk = TRAIN_CHUNK_ROWS
    b, e = parallel.shard_range(args.train_rows, rank, world)
    rows = (e - b) // chunk * chunk
    g = torch.Generator(device=dev); g.manual_seed(1234 + rank)
    x = torch.randn((rows, 64), device=dev, generator=g)
    y = torch.randn((rows, 16), device=dev, generator=g)
    net = pkg.Mlp(64, [256, 256, 256, 16], ["relu", "relu", "relu", "identity"], chunk, device=dev)
    gp = torch.Generator(device=dev); gp.manual_seed(7)            # identical replicas
    off, fan_in = 0, 64
    for d in (256, 256, 256, 16):
        n = d * fan_in + d
        net.params[off:off + n] = (torch.rand(n, device=dev, generator=gp) * 2 - 1) / fan_in ** 0.5
        off += n; fan_in = d
    steps, warmup = max(1, min(args.steps, 5)), 3
    ex = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    sync = lambda: (dist.barrier() if dist is not None else None, torch.cuda.synchronize())
    for _ in range(warmup):
        parallel.sharded_train_step(pkg, net, x, y, rows * world, dist)
    sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        parallel.sharded_train_step(pkg, net, x, y, rows * world, dist, exchange_events=ex[i])
    e1.record(); sync()
    tm = torch.tensor([e0.elapsed_time(e1), sum(a.elapsed_time(b) for a, b in ex)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms, exchange_ms = float(tm[0].item()) / steps, float(tm[1].item()) / steps
    replicas_equal = None
    if dist is not None:                 # identical replicas after identical updates of the all-reduced gradient
        lo, hi = net.params.clone(), net.params.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN); dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        replicas_equal = bool(torch.equal(lo, hi))
    del x, y
    if rank != 0:
        return None
    flop = MLP_FLOP_PER_SAMPLE * rows              # per GPU: the roofline compares one GPU's kernels with one GPU's peak
    peaks = measured_peaks()
    launches = steps * ((rows // chunk) * (4 + 1 + 4 * 3 + 3) + 2)
    cpu = mlp_cpu_reference(net.params.cpu().numpy()) if cpu_baseline else None
    # the reference's OWN CUDA device (cuBLAS SGEMM per layer + its kernels) on the same step, same rows resident in HBM, on this GPU: the second
    # baseline next to its CPU path. Present where oracle/_ref/libref_cuda.so was built from the reference's headers.
    cuda_reference = None
    if cpu_baseline and world == 1:
        import oracle
        if os.path.exists(oracle.REF_CUDA_SO):
            g2 = torch.Generator(device=dev); g2.manual_seed(1234)
            xr, yr = torch.randn((rows, 64), device=dev, generator=g2), torch.randn((rows, 16), device=dev, generator=g2)
            torch.cuda.synchronize()
            ref_ms, _, _ = oracle.ReferenceCuda().mlp_train("c5_b65536", net.params.cpu().numpy(), xr.data_ptr(), yr.data_ptr(), rows, steps=2, warmup=1)
            cuda_reference = {"value": rows / (ref_ms * 1e-3), "unit": "samples/s", "ms_per_step": ref_ms, "kind": "reference",
                              "build": "unmodified reference headers, devices::CUDA (cublasSgemm, fp32), nvcc -O3 sm_100a", "sample": "2 steps after 1 warm-up, same rows, in chunks of its compiled batch of 65,536"}
            del xr, yr
    tf = flop / (ms * 1e-3) / 1e12
    return {"metric": "MLP fwd+bwd+Adam samples/s", "value": rows * world / (ms * 1e-3), "unit": "samples/s", "n_gpus": world, "steps": steps,
            "warmup": warmup, "ms_per_step": ms, "allreduce_ms": exchange_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"mlp_train_64-256-256-256-16_rows{rows * world}", "rows_per_gpu": rows, "chunk_rows": chunk,
                       "parallelism": f"dp{world}, one NCCL all-reduce of the 609 KB gradient arena per step", "l2": "inputs (>= 0.6 GB per pass and GPU) exceed L2"},
            "replicas_bit_identical": replicas_equal,
            "roofline": {"bound": "tensor", "achieved": tf, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tf / peaks["tflops"], "traffic": None,
                         "peak_source": peaks["source"] + " bf16 dense (burst)", "frac_of_3xtf32_ceiling": tf / (peaks["tflops"] / 6.0)},
            "cpu_baseline": cpu, "cuda_reference": cuda_reference, "gpu_launches": launches}


def run_mlp_train(args):
    """--workload mlp_train: the data-parallel training line on its own."""
    from __graft_entry__ import load_package
    pkg = load_package()
    torch, dev, dist, world, rank = distributed_context()
    line = measure_mlp_train(args, pkg, torch, dev, dist, world, rank, cpu_baseline=not args.no_cpu_baseline)
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_collect(args):
    """Secondary line: the on-policy collect (PPO rollout) of `--envs` Pendulum environments per GPU x `--collect-steps` steps with the
    PPO default actor (3 -> 64 -> 64 -> 1, ReLU, identity output, Gaussian head) and STEP_LIMIT 100; draw tables resident in HBM.
    One step = one collect call = one kernel launch writing the [(T + 1) * N, 13] dataset matrix."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    world, rank, local_rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    N, T, limit = args.envs, args.collect_steps, 100
    shape = pkg.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "identity"])
    rs = np.random.RandomState(100 + rank)
    params = torch.from_numpy(np.concatenate([(rs.uniform(-1, 1, 4481) * 0.3).astype(np.float32), np.float32([-0.5])])).to(dev)
    # synthetic draw tables with the distributions of the real ones (initial states U(-pi, pi) x U(-1, 1), noise N(0, 1)); the
    # counters are reset before every call so that each call consumes the same table (one reset round at step 0)
    table = torch.from_numpy(np.stack([rs.uniform(-np.pi, np.pi, (1, N)), rs.uniform(-1, 1, (1, N))], -1).astype(np.float32)).to(dev)
    noise = torch.from_numpy(rs.standard_normal((T, N)).astype(np.float32)).to(dev)
    states, es, tr, er = torch.zeros((N, 2), device=dev), torch.zeros(N, dtype=torch.int32, device=dev), torch.ones(N, dtype=torch.uint8, device=dev), torch.zeros(N, device=dev)
    ds = torch.zeros(((T + 1) * N, 13), device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)

    device_rng = args.collect_rng == "device"
    calls = [0]

    def collect():
        if device_rng:      # resets and noise drawn inside the kernel; consecutive calls continue the counter stream
            pkg.pendulum_collect_device_rng(shape, params, params[4481:], states, es, tr, er, 1234 + rank, calls[0] * T, T, limit, dataset=ds, error_flag=flag)
            calls[0] += 1
        else:
            pkg.pendulum_collect(shape, params, params[4481:], states, es, tr, er, table, noise, T, limit, dataset=ds, error_flag=flag)

    def step():
        es.zero_(); tr.fill_(1)
        collect()

    sync = lambda: (dist.barrier() if dist is not None else None, torch.cuda.synchronize())
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    sync()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    for i in range(args.steps):
        flush.zero_(); es.zero_(); tr.fill_(1)
        starts[i].record()
        collect()
        stops[i].record()
    sync()
    assert int(flag.item()) == 0
    tm = torch.tensor([sum(a.elapsed_time(b) for a, b in zip(starts, stops))], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    ms = float(tm.item()) / args.steps
    host_tables_ms = None
    if rank == 0 and not device_rng:
        # what the table-driven entry point costs on the host per call when the tables are real: the reference-compatible engine
        # drawing T x N normals and the initial states, then the copy to the device (one call, wall clock)
        rng = pkg.rng_init_host(7)
        t0 = time.perf_counter()
        tab, nz, _ = pkg.collect_tables_host(rng, N, T, np.zeros(N, np.int32), np.ones(N, np.uint8), limit, 1)
        torch.from_numpy(tab).to(dev); torch.from_numpy(nz).to(dev); torch.cuda.synchronize()
        host_tables_ms = (time.perf_counter() - t0) * 1e3
    if rank == 0:
        peaks = measured_peaks()
        bytes_step = 40.0 if device_rng else 44.0      # 10 dataset floats written (+ 1 noise float read) per env-step
        tflops = FLOP_PER_ENV_STEP * N * T / (ms * 1e-3) / 1e12
        print(json.dumps({"metric": "env-steps/s (on-policy collect: actor fwd + Gaussian head + env step + dataset row)", "value": world * N * T / (ms * 1e-3),
                          "unit": "env-steps/s", "n_gpus": world, "steps": args.steps, "warmup": warmup, "ms_per_step": ms, "higher_is_better": True,
                          "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                          "config": {"workload": f"pendulum_collect_{N}env_x{T}step_actor3-64-64-1_limit{limit}", "l2": "flushed between timed iterations",
                                     "parallelism": f"env-sharded x{world}, no collective", "rng": "philox4x32-10 in the kernel" if device_rng else "host draw tables resident in HBM",
                                     "host_tables_ms_per_call": host_tables_ms},
                          "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                       "peak_source": peaks["source"] + " bf16 dense (burst)", "hbm_gbs": bytes_step * N * T / (ms * 1e-3) / 1e9, "hbm_peak_gbs": peaks["hbm"]},
                          "gpu_launches": args.steps}))
    if dist is not None:
        dist.destroy_process_group()


def run_ppo_update(args):
    """Secondary line: the PPO update on the Ant shapes of the PPO configuration -- observation 27, actor 27 -> 64 -> 64 -> 8 tanh +
    log_std, critic 27 -> 64 -> 64 -> 1, 64 envs x 1024 steps, GAE (gamma 0.99, lambda 0.95), minibatch 2048, 10 epochs with the
    reference's epoch shuffle (permutation drawn on the host engine inside the timed region). One step = GAE + train() over the whole
    dataset = 320 minibatch updates; value = minibatch samples per second. Single GPU (replicas only)."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from rl_tools_b200 import ppo
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    OBS, ACT, N, T, B, E = 27, 8, 64, 1024, 2048, 10
    layout = ppo.DatasetLayout(OBS, ACT)
    g = torch.Generator(device=dev); g.manual_seed(5)
    rows = (T + 1) * N
    acts = ["tanh", "tanh", "identity"]
    actor, critic = pkg.Mlp(OBS, [64, 64, ACT], acts, B, extra_params=ACT), pkg.Mlp(OBS, [64, 64, 1], acts, B)
    init = {}
    for net, dims in ((actor, (64, 64, ACT)), (critic, (64, 64, 1))):
        off, fan_in = 0, OBS
        for d in dims:
            n = d * fan_in + d
            net.params[off:off + n] = (torch.rand(n, device=dev, generator=g) * 2 - 1) / fan_in ** 0.5
            off += n; fan_in = d
        init[net] = net.params.clone()
    actor.extra("params").fill_(float(np.log(0.5)))
    init[actor] = actor.params.clone()
    base = torch.zeros((rows, layout.data_dim), device=dev)
    base[:, layout.observations] = torch.randn((rows, OBS), device=dev, generator=g)
    base[:, layout.actions_mean] = 0.3 * torch.randn((rows, ACT), device=dev, generator=g)
    base[:, layout.actions] = base[:, layout.actions_mean] + 0.5 * torch.randn((rows, ACT), device=dev, generator=g)
    base[:, layout.action_log_probs] = -5.5 + 0.8 * torch.randn(rows, device=dev, generator=g)
    base[:, layout.rewards] = torch.randn(rows, device=dev, generator=g)
    base[:, layout.truncated] = (torch.rand(rows, device=dev, generator=g) < 1e-3).float()
    dataset = base.clone()
    rng_state = pkg.rng_init_host(1)
    graphs = ppo.MinibatchGraphs(actor, critic, dataset, layout, N * T, B)       # one captured graph per minibatch position

    def step():
        dataset.copy_(base)
        for net in (actor, critic):
            net.params.copy_(init[net]); net.reset_optimizer_state()
        e0.record()
        ppo.evaluate_values(critic, dataset, layout)
        ppo.estimate_generalized_advantages(dataset, layout, N, T)
        ppo.train(actor, critic, dataset, layout, N * T, B, n_epochs=E, shuffle_rng_state=rng_state, graphs=graphs)
        e1.record()

    steps, warmup = min(args.steps, 5), 3
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    ms = []
    for _ in range(steps):
        step(); torch.cuda.synchronize(); ms.append(e0.elapsed_time(e1))
    ms = sum(ms) / len(ms)
    samples = N * T * E
    flop_per_sample = 3 * 2 * ((OBS * 64 + 64 * 64 + 64 * ACT) + (OBS * 64 + 64 * 64 + 64))       # forward + both backward contractions, actor + critic
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
            ref = oracle.Reference("fast")
            na, nc = OBS * 64 + 64 + 64 * 64 + 64 + 64 * ACT + ACT + ACT, OBS * 64 + 64 + 64 * 64 + 64 + 64 + 1
            sec = ref.ppo_train(N, T, B, 1, init[actor].cpu().numpy()[:na], init[critic].cpu().numpy()[:nc], base.cpu().numpy(), shuffle_seed=1, env="ant", want_seconds=True)[7]
            cpu = {"value": N * T / sec, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "reference",
                   "sample": "one epoch (32 minibatches of 2048) of the reference's train() with the epoch shuffle, CPU_OPENBLAS build"}
    peaks = measured_peaks()
    tflops = flop_per_sample * samples / (ms * 1e-3) / 1e12
    launches = steps * (E * (N * T // B) * 24 + E * 2 + 70)
    print(json.dumps({"metric": "PPO update minibatch-samples/s", "value": samples / (ms * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "ppo_update_ant_shapes_obs27_act8_64envx1024step_mb2048_10epochs_shuffled", "updates_per_step": E * (N * T // B),
                                 "l2": "the dataset (13 MB) fits L2: this workload is launch- and latency-bound", "launching": "one CUDA graph replay per minibatch update",
                                 "parallelism": "single GPU"},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                   "peak_source": peaks["source"] + " bf16 dense (burst)"},
                      "cpu_baseline": cpu, "gpu_launches": launches}))


def run_critic_train(args):
    """Secondary line: the SAC critic regression step of the off-policy configuration -- Q-net 4 -> 256 -> 256 -> 1 ReLU, batch 256,
    N(0,1) inputs and targets, zero_gradient + forward + MSE gradient + backward + Adam, 1000 steps per timed call, eager launches and
    replayed as a CUDA graph of the same C-ABI calls. value = training samples per second (graph replay). Single GPU."""
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, STEPS = 256, 1000
    g = torch.Generator(device=dev); g.manual_seed(3)
    net = pkg.Mlp(4, [256, 256, 1], ["relu", "relu", "identity"], B)
    off, fan_in = 0, 4
    for d in (256, 256, 1):
        n = d * fan_in + d
        net.params[off:off + n] = (torch.rand(n, device=dev, generator=g) * 2 - 1) / fan_in ** 0.5
        off += n; fan_in = d
    x, y = torch.randn((B, 4), device=dev, generator=g), torch.randn((B, 1), device=dev, generator=g)
    d_out = net.d_out_buffer()

    def train_step():
        net.zero_gradient()
        out = net.forward(x)
        pkg.mse_gradient(out, y, 1.0, d_a=d_out)
        net.backward(x, d_out)
        net.step()

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(20):
            train_step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(10):
            train_step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 10)
    def timed(fn):
        fn(); torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    ms_eager = timed(lambda: [train_step() for _ in range(STEPS)])
    ms_graph = timed(lambda: [graph.replay() for _ in range(STEPS // 10)])
    flop = 3 * 2 * B * (4 * 256 + 256 * 256 + 256)
    cpu = None
    if not args.no_cpu_baseline:
        import numpy as np
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
            ref = oracle.Reference("fast")
            res = ref.mlp_run("c3_critic", net.params.cpu().numpy(), x.cpu().numpy(), y.cpu().numpy(), 2, 200)
            cpu = {"value": 200 * B / res["seconds"], "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "reference",
                   "sample": "200 train steps (zero_gradient, forward, mse gradient, backward, Adam) of the reference, CPU_OPENBLAS build"}
    peaks = measured_peaks()
    tflops = flop * STEPS / (ms_graph * 1e-3) / 1e12
    print(json.dumps({"metric": "SAC-critic train samples/s (batch 256)", "value": STEPS * B / (ms_graph * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": reps,
                      "warmup": 1, "ms_per_step": ms_graph, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "critic_train_4-256-256-1_batch256_x1000steps", "us_per_train_step_graph": ms_graph, "us_per_train_step_eager": ms_eager,
                                 "l2": "working set (1 MB) is L2-resident by design: latency-bound", "parallelism": "single GPU"},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                   "peak_source": peaks["source"] + " bf16 dense (burst)"},
                      "cpu_baseline": cpu, "gpu_launches": reps * STEPS * 15}))


def run_sac_update(args):
    """Secondary line: one SAC training step of the off-policy loop on the Pendulum shapes with the critic of the off-policy configuration --
    gather_batch (indices drawn in the kernel) from 64 replay buffers of 4096 transitions, train_critic x 2, update_critic_targets, train_actor
    incl. the log_alpha step; actor 3 -> 256 -> 256 -> 2 + sample-and-squash head, critics 4 -> 256 -> 256 -> 1, batch 256. Eager launches and
    replayed as a CUDA graph of the same C-ABI calls. value = sampled transitions per second (graph replay). Single GPU."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    from rl_tools_b200 import sac
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, H, N, CAP, UPDATES = 256, 256, 64, 4096, 100
    rs = np.random.RandomState(5)
    agent = sac.ActorCritic(3, 1, H, B)
    for net in [agent.actor] + agent.critics:
        off, fan_in = 0, net.shape.input_dim
        for l in range(3):
            d = net.shape.dims[l]
            n = d * fan_in + d
            net.params[off:off + n] = torch.from_numpy(((rs.rand(n) * 2 - 1) / fan_in ** 0.5).astype(np.float32)).to(dev)
            off += n; fan_in = d
    agent.copy_critics_to_targets()
    L = pkg.ReplayLayout.packed(CAP)
    raw = np.zeros((N, L.env_stride), np.uint8)
    theta, theta_dot = rs.uniform(-np.pi, np.pi, (N, CAP)), rs.uniform(-8, 8, (N, CAP))
    rows = np.stack([np.cos(theta), np.sin(theta), theta_dot, rs.uniform(-1, 1, (N, CAP)), rs.uniform(-16, 0, (N, CAP)), np.cos(theta + 0.1), np.sin(theta + 0.1), theta_dot,
                     np.zeros((N, CAP)), (rs.rand(N, CAP) < 0.005)], -1).astype(np.float32)
    raw[:, :40 * CAP] = rows.reshape(N, -1).view(np.uint8)
    raw[:, 44 * CAP + 8] = 1                                     # full buffers, position 0
    replay = torch.from_numpy(raw.reshape(-1)).to(dev)
    batch = pkg.new_batch(B)
    noise = torch.empty((3, B, 1), device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    counter = torch.zeros(1, dtype=torch.int64, device=dev)       # device-resident call index: a replayed graph samples fresh batches and noise

    def update():
        pkg.gather_batch(replay, L, N, batch, seed=11, call_counter=counter, error_flag=flag)
        pkg.randn_device_rng(noise, 11, stream_id=1, call_counter=counter)          # the reference's randn() into its noise buffers
        agent.update(batch, noise[0], noise[1], noise[2])
        pkg.counter_advance(counter, 1)

    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(20):
            update()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(10):
            update()
    torch.cuda.synchronize()
    assert int(flag.item()) == 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 10)
    seen = int(counter.item())

    def timed(fn):
        fn(); torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    ms_eager = timed(lambda: [update() for _ in range(UPDATES)])
    ms_graph = timed(lambda: [graph.replay() for _ in range(UPDATES // 10)])
    assert int(counter.item()) == seen + 2 * (reps + 1) * UPDATES and int(flag.item()) == 0      # every update of both timed loops ran and advanced the counter
    # contractions per update: critic updates 2 x (actor fwd + 2 target fwd + critic fwd + dW + dX), actor update (actor fwd, 2 critic fwd + dX, actor dW + dX)
    fa, fc = 2 * B * (3 * H + H * H + H * 2), 2 * B * (4 * H + H * H + H)
    flop = 2 * (fa + 2 * fc + 3 * fc) + (fa + 2 * 2 * fc + 2 * fa)
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
            ref = oracle.Reference("fast")
            U = 50
            na, nc = agent.actor.params.numel(), agent.critics[0].params.numel()
            oa = rs.uniform(-1, 1, (U, 2, B, 4)).astype(np.float32)
            a = [agent.actor.params.cpu().numpy(), np.float32(-0.7), np.stack([c.params.cpu().numpy() for c in agent.critics]),
                 np.stack([c.params.cpu().numpy() for c in agent.critics_target]), oa, rs.uniform(-16, 0, (U, B)).astype(np.float32), np.zeros((U, B), np.uint8),
                 rs.standard_normal((U, 2, B, 1)).astype(np.float32), rs.standard_normal((U, B, 1)).astype(np.float32)]
            ref.sac_updates(B, H, *a)                             # warm-up
            t0 = time.perf_counter()
            ref.sac_updates(B, H, *a)
            sec = time.perf_counter() - t0
            cpu = {"value": U * B / sec, "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "reference",
                   "sample": f"{U} updates (train_critic x 2, update_critic_targets, train_actor) of the reference on hand-filled batches, CPU_OPENBLAS build; batch "
                             "sampling and network setup / teardown of the call included"}
    peaks = measured_peaks()
    tflops = flop * UPDATES / (ms_graph * 1e-3) / 1e12
    print(json.dumps({"metric": "SAC update samples/s (batch 256: gather_batch, 2 x train_critic, target update, train_actor)", "value": UPDATES * B / (ms_graph * 1e-3),
                      "unit": "samples/s", "n_gpus": 1, "steps": reps, "warmup": 1, "ms_per_step": ms_graph, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
                      "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"sac_update_actor3-{H}-{H}-2_critics4-{H}-{H}-1_batch{B}_x{UPDATES}updates", "us_per_update_graph": ms_graph * 1e3 / UPDATES,
                                 "us_per_update_eager": ms_eager * 1e3 / UPDATES, "replay": f"{N} buffers x {CAP} transitions, full", "noise": "3 x [256, 1] normals drawn on the device per update",
                                 "graph": "10 updates per captured graph; a device-resident call counter gives every replay fresh indices and noise",
                                 "l2": "working set (a few MB) is L2-resident by design: latency-bound", "parallelism": "single GPU"},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                   "peak_source": peaks["source"] + " bf16 dense (burst)"},
                      "cpu_baseline": cpu, "gpu_launches": reps * UPDATES * 113}))


def run_acrobot_rollout(args):
    """Secondary line: the environment-generic fused rollout on AcrobotSwingup -- `--envs` environments x 100 steps per launch (RK4 dynamics
    with the reference's double-precision cos / sin, actor 6 -> 64 -> 64 -> 1, episode limit 500), the tensor-core rollout kernel with the Acrobot as
    its environment policy. Single GPU."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    N, T, limit = args.envs, 100, 500
    rs = np.random.RandomState(9)
    shape = pkg.MlpShape.make(6, [64, 64, 1], ["relu", "relu", "tanh"])
    params_h = (rs.uniform(-1, 1, 6 * 64 + 64 + 64 * 64 + 64 + 64 + 1) * 0.3).astype(np.float32)
    params = torch.from_numpy(params_h).to(dev)
    table = torch.from_numpy(rs.uniform(-np.pi, np.pi, (1, N, 2)).astype(np.float32)).to(dev)
    states, es, tr, er = torch.zeros((N, 4), device=dev), torch.zeros(N, dtype=torch.int32, device=dev), torch.ones(N, dtype=torch.uint8, device=dev), torch.zeros(N, device=dev)
    obs, act, rew = torch.empty((T * N, 6), device=dev), torch.empty((T * N, 1), device=dev), torch.empty((T * N, 1), device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)

    def step():
        es.zero_(); tr.fill_(1)
        pkg.env_rollout(pkg.ENV_ACROBOT_SWINGUP, shape, params, states, es, tr, er, table, T, limit, obs=obs, act=act, rew=rew, error_flag=flag)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    steps = min(args.steps, 20)
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(steps):
        flush.zero_(); es.zero_(); tr.fill_(1)
        e0.record()
        pkg.env_rollout(pkg.ENV_ACROBOT_SWINGUP, shape, params, states, es, tr, er, table, T, limit, obs=obs, act=act, rew=rew, error_flag=flag)
        e1.record(); torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    assert int(flag.item()) == 0
    ms = total / steps
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            ref = oracle.Reference("fast")
            n, t = 512, 50
            a = [params_h, np.zeros((n, 4), np.float32), np.zeros(n, np.int32), np.ones(n, np.uint8), np.zeros(n, np.float32), rs.uniform(-np.pi, np.pi, (1, n, 2)).astype(np.float32), t, limit]
            ref.acrobot_rollout(*a)
            t0 = time.perf_counter()
            ref.acrobot_rollout(*a)
            cpu = {"value": n * t / (time.perf_counter() - t0), "unit": "env-steps/s", "cores": 1, "kind": "reference",
                   "sample": f"{n} environments x {t} steps through the reference's observe / evaluate / step / reward, one environment at a time, one thread"}
    peaks = measured_peaks()
    flop = 2 * (6 * 64 + 64 * 64 + 64)
    tflops = flop * N * T / (ms * 1e-3) / 1e12
    print(json.dumps({"metric": "env-steps/s (fused actor fwd + AcrobotSwingup RK4 step)", "value": N * T / (ms * 1e-3), "unit": "env-steps/s", "n_gpus": 1, "steps": steps,
                      "warmup": warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32 (dynamics partly f64, as the reference)",
                      "data": "synthetic", "config": {"workload": f"acrobot_swingup_rollout_{N}env_x{T}step_actor6-64-64-1", "l2": "flushed between timed iterations",
                                                      "kernel": "tensor-core second layer (split fp16), environment as a compile-time policy", "parallelism": "single GPU"},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                   "peak_source": peaks["source"] + " bf16 dense (burst)", "hbm_write_gbs": 32.0 * N * T / (ms * 1e-3) / 1e9, "hbm_peak_gbs": peaks["hbm"]},
                      "cpu_baseline": cpu, "gpu_launches": steps}))


def run_l2f_step(args):
    """Secondary line: the L2F quadrotor step in the configuration of the reference's own GPU throughput harness -- 4096 x 512 quadrotors
    (its grid), 100 steps per launch with a constant action each, states in place. value = quadrotor steps per second. Single GPU.
    Parameter values and the sample states come from the committed fixture (written from the reference)."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    here = os.path.dirname(os.path.abspath(__file__))
    fix = np.load(os.path.join(here, "tests", "golden", "l2f.npz"))
    sys.path.insert(0, os.path.join(here, "tests", "golden"))
    import make_golden as mg
    N, T = 4096 * 512, 100
    params = pkg.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    base_states, base_actions = mg.l2f_inputs(4096, seed=21)
    states0 = torch.from_numpy(base_states).to(dev).repeat(512, 1).contiguous()
    actions = torch.from_numpy(np.clip(base_actions, -1, 1) * np.float32(0.2)).to(dev).repeat(512, 1).contiguous()
    states = states0.clone()
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    warmup, steps = max(args.warmup, 3), min(args.steps, 20)
    for _ in range(warmup):
        states.copy_(states0); pkg.l2f_steps(params, states, actions, T)
    torch.cuda.synchronize()
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(steps):
        states.copy_(states0); flush.zero_()
        e0.record()
        pkg.l2f_steps(params, states, actions, T)
        e1.record(); torch.cuda.synchronize()
        total += e0.elapsed_time(e1)
    ms = total / steps
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            ref = oracle.Reference("fast")
            n, t = 4096, 100
            ref.l2f_steps(base_states, base_actions, 2)
            t0 = time.perf_counter()
            ref.l2f_steps(base_states, base_actions, t)
            cpu = {"value": n * t / (time.perf_counter() - t0), "unit": "quadrotor-steps/s", "cores": 1, "kind": "reference",
                   "sample": f"{n} quadrotors x {t} steps through the reference's step() (project flags), one thread"}
    peaks = measured_peaks()
    flop = 4 * 157 + 5 * 21 * 2 + 60           # four dynamics evaluations (the reference's own count), the state algebra of RK4, post-integration
    print(json.dumps({"metric": "quadrotor-steps/s (L2F step, RK4)", "value": N * T / (ms * 1e-3), "unit": "quadrotor-steps/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"l2f_step_{N}quadrotors_x{T}step", "l2": "flushed between timed iterations", "parallelism": "single GPU",
                                 "kernel": "one thread per quadrotor, state in registers, no multiply-add contraction (bit-for-bit with the reference's CPU step)"},
                      "roofline": {"bound": "hbm", "achieved": 2 * 92.0 * N / (ms * 1e-3) / 1e9, "peak": peaks["hbm"], "unit": "GB/s", "frac": 2 * 92.0 * N / (ms * 1e-3) / 1e9 / peaks["hbm"],
                                   "traffic": None, "peak_source": peaks["source"], "note": "CUDA-core fp32 arithmetic in registers: neither HBM nor the tensor pipe bounds it",
                                   "fp32_tflops": flop * N * T / (ms * 1e-3) / 1e12},
                      "cpu_baseline": cpu, "gpu_launches": steps}))


def run_l2f_rollout(args):
    """Secondary line: the fused runner loop on the L2F quadrotor -- `--envs` quadrotors x 100 steps per launch (observe, actor 18 -> 64 -> 64 -> 4,
    RK4 step, reward, termination; episode limit 500, initial states of the reference's sampler from the committed fixture). Single GPU."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    here = os.path.dirname(os.path.abspath(__file__))
    fix = np.load(os.path.join(here, "tests", "golden", "l2f.npz"))
    N, T, limit, H = args.envs, 100, 500, 64
    rs = np.random.RandomState(4)
    shape = pkg.MlpShape.make(18, [H, H, 4], ["relu", "relu", "tanh"])
    params_h = (rs.uniform(-1, 1, 18 * H + H + H * H + H + 4 * H + 4) * 0.05).astype(np.float32)
    params = torch.from_numpy(params_h).to(dev)
    p = pkg.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    init = fix["initial_states"].reshape(-1, 23)
    table = torch.from_numpy(init[rs.randint(0, init.shape[0], (8, N))]).to(dev).contiguous()            # eight reset rounds per environment
    states, es, er = torch.zeros((N, 23), device=dev), torch.zeros(N, dtype=torch.int32, device=dev), torch.zeros(N, device=dev)
    tr = torch.ones(N, dtype=torch.uint8, device=dev)
    obs, act, rew = torch.empty((T * N, 18), device=dev), torch.empty((T * N, 4), device=dev), torch.empty(T * N, device=dev)
    term = torch.empty(T * N, dtype=torch.uint8, device=dev)
    flag = torch.zeros(1, dtype=torch.int32, device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)
    warmup, steps = max(args.warmup, 3), min(args.steps, 20)
    total = 0.0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for it in range(warmup + steps):
        flush.zero_(); es.zero_(); tr.fill_(1)
        e0.record()
        pkg.l2f_rollout(p, fix["mdp"], shape, params, states, es, tr, er, table, T, limit, obs=obs, act=act, rew=rew, terminated=term, error_flag=flag)
        e1.record(); torch.cuda.synchronize()
        if it >= warmup:
            total += e0.elapsed_time(e1)
    ms = total / steps
    peaks = measured_peaks()
    out_bytes = (18 + 4 + 1) * 4 + 1
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        orc = oracle.Oracle()
        n, oshape = 2048, oracle.MlpShape.make(18, [H, H, 4], ["relu", "relu", "tanh"])
        sample = np.ascontiguousarray(table[:, :n].cpu().numpy())
        t0 = time.perf_counter()
        orc.l2f_rollout(oshape, params_h, fix["dynamics"], float(fix["dt"]), fix["mdp"], np.zeros((n, 23), np.float32), np.zeros(n, np.int32), np.ones(n, np.uint8),
                        np.zeros(n, np.float32), sample, T, limit)
        cpu = {"value": n * T / (time.perf_counter() - t0), "unit": "env-steps/s", "cores": 1, "kind": "port",
               "sample": f"the oracle's loop (observe, MLP, step, reward) over the first {n} quadrotors x {T} steps, one thread"}
    print(json.dumps({"metric": "env-steps/s (fused actor fwd + L2F quadrotor step)", "value": N * T / (ms * 1e-3), "unit": "env-steps/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
                      "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": f"l2f_rollout_{N}env_x{T}step_actor18-64-64-4", "l2": "flushed between timed iterations", "parallelism": "single GPU",
                                 "kernel": "l2f_rollout_kernel: a lane per quadrotor for the environment, per-warp register tiles for the hidden layers, dynamics without multiply-add contraction", "resets_exhausted": int(flag.item())},
                      "roofline": {"bound": "hbm", "achieved": out_bytes * N * T / (ms * 1e-3) / 1e9, "peak": peaks["hbm"], "unit": "GB/s", "frac": out_bytes * N * T / (ms * 1e-3) / 1e9 / peaks["hbm"],
                                   "traffic": None, "peak_source": peaks["source"], "note": "CUDA-core fp32 arithmetic: neither HBM nor the tensor pipe bounds it"},
                      "cpu_baseline": cpu, "gpu_launches": steps}))


def run_l2f_sac_loop(args):
    """Secondary line: the off-policy training loop on the L2F quadrotor (16 environments; per loop step: runner step with resets drawn in the kernel,
    gather_batch, train_critic x 2, update_critic_targets, train_actor at batch 256), every step one CUDA-graph replay. Single GPU."""
    import numpy as np
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    from importlib import import_module
    loops = import_module(pkg.__name__ + ".loops")
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    here = os.path.dirname(os.path.abspath(__file__))
    fix = np.load(os.path.join(here, "tests", "golden", "l2f.npz"))
    p = pkg.L2fParameters.make(fix["dynamics"], float(fix["dt"]))
    N_ENVS, BATCH, WARM, STEPS = 16, 256, 200, 5000
    torch.manual_seed(0)
    loop = loops.L2fSacLoop(p, fix["mdp"], fix["init"], n_envs=N_ENVS, batch_size=BATCH, step_limit=WARM + 100 + STEPS, n_warmup_steps=WARM, replay_capacity=8192, seed=1)
    _, len0 = loop.evaluate()
    for _ in range(WARM + 100):                      # warm-up with random actions, the capture, and the first replays
        loop.step()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record()
    for _ in range(STEPS):
        loop.step()
    e1.record(); torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    _, len1 = loop.evaluate()
    print(json.dumps({"metric": "SAC loop steps/s on the L2F quadrotor (runner step of 16 environments + one update at batch 256)", "value": STEPS / (ms * 1e-3), "unit": "loop-steps/s",
                      "n_gpus": 1, "steps": STEPS, "warmup": WARM + 100, "ms_per_step": ms / STEPS, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                      "data": "synthetic", "config": {"workload": "l2f_sac_loop_16env_batch256_hidden64", "l2": "working set (a few MB) is L2-resident by design: latency-bound",
                                                       "parallelism": "single GPU", "evaluation_episode_length_before_after": [len0, len1]},
                      "roofline": None, "cpu_baseline": None, "gpu_launches": None}))


def run_actor_eval(args):
    """Secondary line: the batched actor inference of the CPU-runnable configuration -- fp32 input [256, 3], MLP 3 -> 64 -> 64 -> 2 (ReLU,
    ReLU, identity), evaluate() = three fused dense launches, 1000 calls per timed step, eager and replayed as a CUDA graph.
    value = inferred samples per second (graph replay). Single GPU."""
    import torch
    from __graft_entry__ import load_package
    pkg = load_package()
    if int(os.environ.get("RANK", "0")) != 0:
        return
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    B, CALLS = 256, 1000
    g = torch.Generator(device=dev); g.manual_seed(4)
    net = pkg.Mlp(3, [64, 64, 2], ["relu", "relu", "identity"], B)
    off, fan_in = 0, 3
    for d in (64, 64, 2):                                   # Glorot-uniform weights, zero biases
        bound = (6.0 / (fan_in + d)) ** 0.5
        net.params[off:off + d * fan_in] = (torch.rand(d * fan_in, device=dev, generator=g) * 2 - 1) * bound
        off += d * fan_in + d; fan_in = d
    x = torch.rand((B, 3), device=dev, generator=g) * 2 - 1
    y = torch.empty((B, 2), device=dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        for _ in range(5):
            net.evaluate(x, y=y)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        for _ in range(10):
            net.evaluate(x, y=y)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    reps = min(args.steps, 10)
    def timed(fn):
        fn(); torch.cuda.synchronize()
        e0.record()
        for _ in range(reps):
            fn()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / reps
    ms_eager = timed(lambda: [net.evaluate(x, y=y) for _ in range(CALLS)])
    ms_graph = timed(lambda: [graph.replay() for _ in range(CALLS // 10)])
    cpu = None
    if not args.no_cpu_baseline:
        import oracle
        if os.path.exists(oracle.REF_FAST_SO):
            os.environ.setdefault("OPENBLAS_NUM_THREADS", str(os.cpu_count() or 1))
            ref = oracle.Reference("fast")
            res = ref.mlp_run("c1_actor_eval", net.params.cpu().numpy(), x.cpu().numpy(), None, 0, 20000)
            cpu = {"value": 20000 * B / res["seconds"], "unit": "samples/s", "cores": os.cpu_count() or 1, "kind": "reference",
                   "sample": "20,000 evaluate() calls of the reference at batch 256, CPU_OPENBLAS build"}
    peaks = measured_peaks()
    tflops = 2 * B * (3 * 64 + 64 * 64 + 64 * 2) * CALLS / (ms_graph * 1e-3) / 1e12
    print(json.dumps({"metric": "actor inference samples/s (batch 256)", "value": CALLS * B / (ms_graph * 1e-3), "unit": "samples/s", "n_gpus": 1, "steps": reps, "warmup": 1,
                      "ms_per_step": ms_graph, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
                      "config": {"workload": "actor_eval_3-64-64-2_batch256_x1000calls", "us_per_call_graph": ms_graph, "us_per_call_eager": ms_eager,
                                 "l2": "working set (20 KB) is L2-resident by design: latency-bound", "parallelism": "single GPU"},
                      "roofline": {"bound": "tensor", "achieved": tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": tflops / peaks["tflops"], "traffic": None,
                                   "peak_source": peaks["source"] + " bf16 dense (burst)"},
                      "cpu_baseline": cpu, "gpu_launches": reps * CALLS * 3}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-secondary", action="store_true", help="headline rollout only: skip the mlp_train and strong-scaling measurements")
    ap.add_argument("--envs", type=int, default=N_ENVS, help="environments per GPU (default: the benchmark workload)")
    ap.add_argument("--rollout-steps", type=int, default=N_STEPS, help="steps per environment per call (default: the benchmark workload)")
    ap.add_argument("--allow-short-warmup", action="store_true", help="profiling runs only: do not force 3 warm-up steps")
    ap.add_argument("--workload", default="rollout", choices=["rollout", "mlp_train", "collect", "ppo_update", "critic_train", "actor_eval", "sac_update", "acrobot_rollout", "l2f_step", "l2f_rollout", "l2f_sac_loop"],
                    help="rollout = the headline benchmark; mlp_train = secondary line: sharded forward+backward+Adam of the 64-256-256-256-16 MLP; "
                         "collect = secondary line: on-policy (PPO) collect into the dataset matrix; ppo_update = secondary line: GAE + PPO train() "
                         "on the Ant shapes; critic_train = secondary line: batch-256 SAC critic regression steps (eager and CUDA graph)")
    ap.add_argument("--collect-steps", type=int, default=64, help="collect: steps per environment per call")
    ap.add_argument("--collect-rng", default="tables", choices=["tables", "device"],
                    help="collect: random numbers from host draw tables (bit-compatible with the reference's host engine) or drawn inside the kernel")
    ap.add_argument("--train-rows", type=int, default=1 << 24, help="mlp_train: total input rows over all GPUs")
    args = ap.parse_args()
    import faulthandler
    faulthandler.enable()                          # a crash in native code prints the Python stack it happened under
    if args.workload == "mlp_train":
        return run_mlp_train(args)
    if args.workload == "collect":
        return run_collect(args)
    if args.workload == "sac_update":
        return run_sac_update(args)
    if args.workload == "acrobot_rollout":
        return run_acrobot_rollout(args)
    if args.workload == "l2f_step":
        return run_l2f_step(args)
    if args.workload == "l2f_rollout":
        return run_l2f_rollout(args)
    if args.workload == "l2f_sac_loop":
        return run_l2f_sac_loop(args)
    if args.workload == "ppo_update":
        return run_ppo_update(args)
    if args.workload == "critic_train":
        return run_critic_train(args)
    if args.workload == "actor_eval":
        return run_actor_eval(args)
    if args.impl == "reference":
        return run_reference(args)
    if not args.allow_short_warmup:
        args.warmup = max(args.warmup, 3)
    globals().update(N_ENVS=args.envs, N_STEPS=args.rollout_steps)
    workload = WORKLOAD if (args.envs, args.rollout_steps) == (65536, 200) else f"pendulum_rollout_{args.envs}env_x{args.rollout_steps}step_actor3-64-64-1 (reduced: profiling only)"

    import numpy as np
    from __graft_entry__ import load_package
    pkg = load_package()
    pkg.lib()                                     # fails loudly if the CUDA library is missing
    torch, dev, dist, world, rank = distributed_context()
    local_rank = dev.index

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    shape = pkg.MlpShape.make(3, [64, 64, 1], ["relu", "relu", "tanh"])
    params_h, table_h = synthetic_inputs(seed=rank, n_envs=N_ENVS)
    t = lambda a: torch.from_numpy(a).to(dev)
    params, table = t(params_h), t(table_h)
    states, es, tr, er = (torch.zeros((N_ENVS, 2), device=dev), torch.zeros(N_ENVS, dtype=torch.int32, device=dev),
                          torch.ones(N_ENVS, dtype=torch.uint8, device=dev), torch.zeros(N_ENVS, device=dev))
    rows = N_ENVS * N_STEPS
    obs, act, rew = torch.empty((rows, 3), device=dev), torch.empty((rows, 1), device=dev), torch.empty((rows, 1), device=dev)
    flush = torch.empty(256 * 1024 * 1024 // 4, device=dev)   # 256 MB > 126 MB L2
    flag = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        # every episode is exactly 200 steps, so each call starts with all environments truncated -> reset from the table
        pkg.pendulum_rollout(shape, params, states, es, tr, er, table, N_STEPS, STEP_LIMIT, obs=obs, act=act, rew=rew, error_flag=flag)

    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    with ClockSampler(local_rank) as clocks:
        for _ in range(args.warmup):
            flush.zero_(); step()
        barrier()
        clocks.mark_begin()
        wall0 = time.perf_counter()
        for i in range(args.steps):
            flush.zero_()                          # L2 flush between timed iterations (not inside the event pair)
            starts[i].record(); step(); stops[i].record()
        barrier()
        wall = time.perf_counter() - wall0
        clocks.mark_end()
    assert int(flag.item()) == 0
    dev_ms = sum(a.elapsed_time(b) for a, b in zip(starts, stops))
    tm = torch.tensor([dev_ms], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
    total_ms = float(tm.item())
    ms_per_step = total_ms / args.steps
    value = world * N_ENVS * N_STEPS * args.steps / (total_ms * 1e-3)

    # ---- end to end: host buffers through the C ABI, copies inside the timed region ----
    pin = lambda *s, dtype=torch.float32: torch.empty(*s, dtype=dtype).pin_memory()
    h_obs, h_act, h_rew = pin(rows, 3), pin(rows, 1), pin(rows, 1)
    h_states, h_es, h_tr, h_er = pin(N_ENVS, 2), pin(N_ENVS, dtype=torch.int32), pin(N_ENVS, dtype=torch.uint8), pin(N_ENVS)
    h_table, h_params = pin(*table_h.shape), pin(params_h.size)
    h_table.copy_(torch.from_numpy(table_h)); h_params.copy_(torch.from_numpy(params_h))
    h_states.zero_(); h_es.zero_(); h_tr.fill_(1); h_er.zero_()

    def e2e_step():
        pkg.pendulum_rollout_host(shape, h_params, h_states, h_es, h_tr, h_er, h_table, N_STEPS, h_obs, h_act, h_rew, STEP_LIMIT)

    e2e_value = None
    if not args.no_e2e:
        for _ in range(2):
            e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        e2e_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(e2e_s, op=dist.ReduceOp.MAX)
        e2e_value = world * N_ENVS * N_STEPS * args.e2e_steps / float(e2e_s.item())
    # what the host link alone allows at this rank count: the same device-to-host bytes (the three trajectory arrays, already on the device)
    # copied to the same pinned buffers by all ranks at once, nothing else -- the ceiling of any host-buffer call on this machine
    copy_only_value = None
    if not args.no_e2e:
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            h_obs.copy_(obs, non_blocking=True); h_act.copy_(act, non_blocking=True); h_rew.copy_(rew, non_blocking=True)
        barrier()
        c_s = torch.tensor([time.perf_counter() - t0], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(c_s, op=dist.ReduceOp.MAX)
        copy_only_value = world * N_ENVS * N_STEPS * args.e2e_steps / float(c_s.item())
    h2d = params_h.nbytes + table_h.nbytes + N_ENVS * (8 + 4 + 1 + 4)
    d2h = rows * BYTES_PER_ENV_STEP + N_ENVS * (8 + 4 + 1 + 4) + 4
    pkg.lib().b200rl_release_host_staging()
    del h_obs, h_act, h_rew

    # ---- strong scaling of the same workload: the 65,536 environments split over the ranks (each rank rolls out N_ENVS / world) ----
    strong = None
    if not args.no_secondary:
        n_local = N_ENVS // world // 4 * 4
        s_states, s_es, s_tr, s_er = states[:n_local].clone(), es[:n_local].clone(), tr[:n_local].clone(), er[:n_local].clone()
        s_table = table[:, :n_local].contiguous()
        s_rows = n_local * N_STEPS
        s_steps = max(3, min(args.steps, 20))
        s0 = [torch.cuda.Event(enable_timing=True) for _ in range(s_steps)]
        s1 = [torch.cuda.Event(enable_timing=True) for _ in range(s_steps)]
        sstep = lambda: pkg.pendulum_rollout(shape, params, s_states, s_es, s_tr, s_er, s_table, N_STEPS, STEP_LIMIT, obs=obs[:s_rows], act=act[:s_rows], rew=rew[:s_rows], error_flag=flag)
        for _ in range(3):
            flush.zero_(); sstep()
        barrier()
        for i in range(s_steps):
            flush.zero_(); s0[i].record(); sstep(); s1[i].record()
        barrier()
        stm = torch.tensor([sum(a.elapsed_time(b) for a, b in zip(s0, s1))], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(stm, op=dist.ReduceOp.MAX)
        s_ms = float(stm.item()) / s_steps
        strong = {"metric": "env-steps/s (fused actor fwd + env step)", "value": world * n_local * N_STEPS / (s_ms * 1e-3), "unit": "env-steps/s", "scaling": "strong",
                  "n_gpus": world, "ms_per_step": s_ms, "steps": s_steps, "config": {"workload": workload, "envs_total": world * n_local, "envs_per_gpu": n_local, "steps_per_env": N_STEPS}}
        assert int(flag.item()) == 0
    del obs, act, rew
    torch.cuda.empty_cache()
    mlp = None
    if not args.no_secondary:
        mlp = measure_mlp_train(args, pkg, torch, dev, dist, world, rank, cpu_baseline=not args.no_cpu_baseline)

    if rank == 0:
        peaks = measured_peaks()
        achieved_tflops = FLOP_PER_ENV_STEP * N_ENVS * N_STEPS / (ms_per_step * 1e-3) / 1e12
        # traffic: dram__bytes_read + dram__bytes_write of one full-size launch, a constant taken from an ncu capture of this workload
        # (it cannot be measured inside an unprofiled run); other sizes were not captured
        traffic = TRAFFIC_BYTES_FULL_LAUNCH if (N_ENVS, N_STEPS) == (65536, 200) else None
        roofline = {"bound": "tensor", "achieved": achieved_tflops, "peak": peaks["tflops"], "unit": "TFLOP/s", "frac": achieved_tflops / peaks["tflops"],
                    "traffic": traffic, "traffic_source": "ncu capture of this workload, constant", "peak_source": peaks["source"] + " bf16 dense (burst)",
                    # the contraction runs as three passes of fp16 parts (fp32 accuracy), each at the dense 16-bit rate: the attainable ceiling is a third of the peak
                    "frac_of_split_ceiling": achieved_tflops / (peaks["tflops"] / 3.0),
                    # the same number against the ceiling of the 3xTF32 form this kernel had before (tf32 at half the 16-bit rate, three passes)
                    "frac_of_3xtf32_ceiling": achieved_tflops / (peaks["tflops"] / 6.0),
                    "hbm_write_gbs": BYTES_PER_ENV_STEP * N_ENVS * N_STEPS / (ms_per_step * 1e-3) / 1e9, "hbm_peak_gbs": peaks["hbm"]}
        cpu = None if args.no_cpu_baseline else cpu_reference_rate()
        # the reference's OWN CUDA runner (prologue kernel, per-layer bias / cublasSgemm / activation, epilogue kernel: ~12 launches per step) on
        # this GPU, same environment count, step limit and actor: the second baseline next to its CPU path
        cuda_reference = None
        if not args.no_cpu_baseline and (N_ENVS, N_STEPS) == (65536, 200):
            import oracle
            if os.path.exists(oracle.REF_CUDA_SO):
                ref_ms, mean_return = oracle.ReferenceCuda().rollout("65536env", params_h[:4481], steps=2, warmup=1)
                cuda_reference = {"value": N_ENVS * N_STEPS / (ref_ms * 1e-3), "unit": "env-steps/s", "ms_per_step": ref_ms, "kind": "reference",
                                  "build": "unmodified reference headers, devices::CUDA off-policy runner step<0> (cublasSgemm, fp32, cuRAND resets), nvcc -O3 sm_100a",
                                  "sample": "2 rollouts of 200 runner steps after 1 warm-up rollout, incl. the replay-buffer append the runner does",
                                  "mean_episode_return": mean_return}
        line = {"metric": "env-steps/s (fused actor fwd + env step)", "value": value, "unit": "env-steps/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": rollout_config(world, workload),
                "roofline": roofline, "cpu_baseline": cpu, "cuda_reference": cuda_reference, "clocks": clocks.summary(),
                "e2e": {"value": e2e_value, "unit": "env-steps/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": args.e2e_steps,
                        "copy_only_value": copy_only_value, "copy_only_note": "the same device-to-host bytes copied by all ranks at once and nothing else: the host link's ceiling for this call"},
                "gpu_launches": 2 * args.steps,          # per timed step: pack_w1_pairs_kernel and rollout_tc_kernel (the constant-bank fills are copies)
                "wall_s_timed_region": wall,
                "secondary": {"mlp_train": mlp, "rollout_strong": strong}}
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
