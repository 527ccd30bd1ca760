/*
 * b200rl.h -- C ABI of libb200rl.so: the sm_100a kernels for the RLtools hot path
 * (dense layer evaluate/forward/backward, MSE gradient, Adam, and the batched Pendulum environment step that the
 * runners interleave with actor inference).
 *
 * Conventions
 *   - every entry point returns an int status (B200RL_OK == 0); nothing aborts, nothing throws;
 *   - all pointers are DEVICE pointers unless the parameter name ends in _host;
 *   - matrices are row-major fp32 with an explicit row pitch in ELEMENTS (ld*), so views into wider tables work
 *     (the reference's Matrix views carry a row pitch, containers/matrix/matrix.h:84-85); column pitch is 1;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued asynchronously on it, no entry point
 *     synchronises or allocates unless its comment says so;
 *   - "reference" citations are paths inside the RLtools tree (include/rl_tools/...).
 */
#ifndef B200RL_H
#define B200RL_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define B200RL_OK 0
#define B200RL_ERR_INVALID_ARGUMENT 1   /* null pointer, negative size, pitch smaller than the row */
#define B200RL_ERR_UNSUPPORTED 2        /* a shape / activation this build has no kernel for */
#define B200RL_ERR_CUDA 3               /* a CUDA runtime call failed; see b200rl_last_cuda_error() */
#define B200RL_ERR_DEVICE_FLAG 4        /* a kernel reported a problem through its error flag */
#define B200RL_ERR_SCRATCH_LIMIT 5      /* the problem needs more scratch than the built-in static buffer holds */

/* activation ids: nn/activation_functions.h:10-20 */
#define B200RL_ACT_IDENTITY 0
#define B200RL_ACT_RELU 1
#define B200RL_ACT_TANH 2
#define B200RL_ACT_FAST_TANH 3
#define B200RL_ACT_SIGMOID 4

#define B200RL_MAX_LAYERS 8

typedef void* b200rl_stream_t; /* cudaStream_t */

int b200rl_version(void);
const char* b200rl_status_string(int status);
/* text of the last CUDA error seen by this library on the calling thread ("" if none) */
const char* b200rl_last_cuda_error(void);

/* Wide networks at small batches (at most four layers, widths and batch at most 512, too large for the whole-network kernels of small
 * networks) run b200rl_mlp_backward as ONE cooperative launch with grid-wide barriers between the layers (B200RL_COOPERATIVE_PASS=0 in the
 * environment keeps them on the per-layer kernels, =2 also takes forward / evaluate there). Every barrier wait has a limit; *status = 1
 * when a wait on the current device ever ran into it (the pass's results are then undefined), else 0. Synchronous (a device-to-host copy). */
int b200rl_cooperative_pass_status(int* status);

/* Reads (and synchronises for) the library's device-side error word into *state_host: non-zero after a bounded wait
 * inside a tensor-core dense kernel expired (the kernel then left its loops and released its tensor memory instead of
 * spinning). The reference has no counterpart (its asserts are no-ops in kernels, utils/assert/operations_cuda.h:17-21). */
int b200rl_device_error_state(int* state_host);
/* Sets that word back to zero on the current device (synchronises), so that a later b200rl_device_error_state reports only what happened since. */
int b200rl_device_error_clear(void);

/* ---------------------------------------------------------------------------------------------------------
 * Dense layer. W is [O, I] row-major (weights.parameters), bias is [O].
 * ------------------------------------------------------------------------------------------------------- */

/* y = act(x W^T + b); if pre != NULL the pre-activations are stored as well.
 * Replaces evaluate (nn/layers/dense/operations_cuda.h:236-274: set_biases_kernel + cublasSgemm +
 * activation_kernel) when pre == NULL and forward (:276-316, which adds a device-to-device copy of the
 * pre-activations) when pre != NULL -- one launch instead of three or four. x must not alias y. */
int b200rl_dense_forward(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                         int batch, int input_dim, int output_dim, int activation, b200rl_stream_t stream);

/* The same with a caller-owned workspace of b200rl_dense_forward_workspace_bytes(...) bytes (16-byte aligned device memory; 0 for
 * shapes that do not take the tensor-core kernel): the weights are split into their tensor-core operand parts once per call into the
 * workspace instead of once per 128-row tile of the batch -- the fast form for large batches. Contents of the workspace need not be
 * kept between calls; calls that share one workspace must be ordered on one stream. workspace == NULL behaves like b200rl_dense_forward.
 * (No counterpart in the reference: cuBLAS manages its own workspace.) */
size_t b200rl_dense_forward_workspace_bytes(int batch, int input_dim, int output_dim);
int b200rl_dense_forward_ws(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                            int batch, int input_dim, int output_dim, int activation, void* workspace, size_t workspace_bytes, b200rl_stream_t stream);

/* d_pre = act'(pre) * d_out (written back into d_out, as the reference does);
 * d_bias[o] += sum_b d_pre[b][o];  d_W[o][i] += sum_b d_pre[b][o] * x[b][i];  d_in[b][i] = sum_o d_pre[b][o] W[o][i].
 * Gradients ACCUMULATE (zero them with b200rl_fill). d_in == NULL skips the input gradient (first layer),
 * d_W == d_bias == NULL gives backward_input.
 * Replaces backward / backward_full / backward_input (nn/layers/dense/operations_cuda.h:358-413:
 * d_activation_accumulate_bias_gradient_kernel + two cublasSgemm).
 * `scratch` is device memory of at least b200rl_dense_backward_scratch_bytes(...) bytes (may be NULL when that
 * returns 0); it holds split-batch partial sums of d_W and d_bias that are reduced in a fixed order, so the
 * result does not depend on scheduling. */
size_t b200rl_dense_backward_scratch_bytes(int batch, int input_dim, int output_dim);
int b200rl_dense_backward(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                          float* d_W, float* d_bias, float* d_in, int ldi, int batch, int input_dim, int output_dim, int activation,
                          void* scratch, size_t scratch_bytes, b200rl_stream_t stream);

/* The same backward pass for callers that have no scratch buffer to give and must not allocate one.
 * (No counterpart in the reference: its backward takes no scratch argument because cuBLAS manages its own workspace.)
 * Who needs it: code that sits behind the reference's own signature backward(device, layer, input, d_output, buffer)
 * -- there is no parameter through which scratch could arrive, and calling cudaMalloc inside a training step is not an
 * option there, since it synchronises the whole device and the memory is usually already handed out to another
 * allocator. The split-batch partial sums live instead in a static device array inside the library,
 * B200RL_STATIC_SCRATCH_BYTES (8 MiB) large, which every GPU that loads the library holds until the process exits.
 *   - any batch size is accepted: the batch is split into as many partial sums as the array holds (fewer than the caller-scratch
 *     entry point would use for a large batch -- slower there, same accuracy, still a fixed summation order);
 *   - a layer with more than B200RL_STATIC_SCRATCH_MAX_WEIGHTS weights (input_dim * output_dim > 2^20, e.g. wider than 1024 x 1024),
 *     for which the array cannot hold even two partial sums, is refused with B200RL_ERR_SCRATCH_LIMIT when gradients are asked for;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress); make that first call
 *     before any stream capture begins on that device;
 *   - the call makes no cudaMalloc / cudaFree and uses no allocating library routine;
 *   - all calls share the one array: two calls whose kernels can overlap on the GPU (different streams) race on it.
 *     Nothing in it has to start at zero -- every partial sum that is read was written earlier in the same call. */
#define B200RL_STATIC_SCRATCH_BYTES (8u * 1024u * 1024u)
#define B200RL_STATIC_SCRATCH_MAX_WEIGHTS (B200RL_STATIC_SCRATCH_BYTES / 8u)   /* input_dim * output_dim of the largest accepted layer: 2^20 */
int b200rl_dense_backward_static_scratch(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                                         float* d_W, float* d_bias, float* d_in, int ldi, int batch, int input_dim, int output_dim,
                                         int activation, b200rl_stream_t stream);

/* d_a = 2 w (a - b) / (rows cols). Replaces nn::loss_functions::mse::gradient (nn/loss_functions/mse/operations_cuda.h:41-58). */
int b200rl_mse_gradient(const float* a, int lda, const float* b, int ldb, float* d_a, int ldd, int rows, int cols, float loss_weight,
                        b200rl_stream_t stream);

/* The loss value itself: loss_weight * sum (a - b)^2 / (rows * cols), returned through *loss_host (host memory; the call synchronises the
 * stream, as a function that returns the value must). Replaces nn::loss_functions::mse::evaluate
 * (nn/loss_functions/mse/operations_generic.h:9-22, a host loop over get() in the reference). The squares are summed in double in a
 * fixed order and rounded once. */
int b200rl_mse_evaluate(const float* a, int lda, const float* b, int ldb, int rows, int cols, float loss_weight, float* loss_host,
                        b200rl_stream_t stream);

/* dst[0..n) = value. Replaces the cudaMemsetAsync pairs of zero_gradient / _reset_optimizer_state
 * (nn/layers/dense/operations_cuda.h:415-432) -- with the flat arena below it is one call per network. */
int b200rl_fill(float* dst, size_t n, float value, b200rl_stream_t stream);
/* Target-network (Polyak) update: target = polyak * target + (1 - polyak) * source, or with source * source when square != 0
 * (update / update_squared, utils/polyak/operations_generic.h:10-40; CUDA form utils/polyak/operations_cuda.h:12-52; called per layer by
 * update_critic_targets, rl/algorithms/sac/operations_generic.h:486-496). Row-major [rows, cols] matrices with row pitches ld_*. */
int b200rl_polyak_update(const float* source, int ld_source, float* target, int ld_target, int rows, int cols, float polyak, int square,
                         b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * MLP on a flat parameter arena. For each layer l: W_l [O_l, I_l] row-major, then b_l [O_l]; gradients and both
 * Adam moments use the same layout in their own arenas, so zero_gradient, the optimizer step and a gradient
 * all-reduce are each ONE pass over contiguous memory (the reference allocates 8 tensors per layer,
 * nn/layers/dense/layer.h:82-127, nn/optimizers/adam/adam.h:88-95).
 * ------------------------------------------------------------------------------------------------------- */
typedef struct {
    int n_layers;                    /* 1..B200RL_MAX_LAYERS */
    int input_dim;
    int dims[B200RL_MAX_LAYERS];     /* output dim per layer */
    int acts[B200RL_MAX_LAYERS];     /* activation per layer */
} b200rl_mlp_shape;

size_t b200rl_mlp_num_params(const b200rl_mlp_shape* shape);

/* y [batch, O_last] = mlp(x); no state is kept. tick/tock are two [batch, max hidden dim] ping-pong buffers
 * (nn_models::mlp buffers, nn_models/mlp/network.h). Replaces nn_models::mlp evaluate
 * (nn_models/mlp/operations_generic.h:77-102 recursing into the dense CUDA ops). */
int b200rl_mlp_evaluate(const b200rl_mlp_shape* shape, const float* params, const float* x, int ldx, float* y, int ldy,
                        float* tick, float* tock, int batch, b200rl_stream_t stream);

/* forward that keeps per-layer pre-activations and outputs, concatenated layer after layer, each [batch, O_l]
 * dense. Replaces nn_models::mlp forward (nn_models/mlp/operations_generic.h:103-120). */
int b200rl_mlp_forward(const b200rl_mlp_shape* shape, const float* params, const float* x, int ldx, float* pre, float* out,
                       int batch, b200rl_stream_t stream);

/* evaluate / forward with a caller-owned workspace (b200rl_mlp_forward_workspace_bytes = the largest layer's
 * b200rl_dense_forward_workspace_bytes), see b200rl_dense_forward_ws. */
size_t b200rl_mlp_forward_workspace_bytes(const b200rl_mlp_shape* shape, int batch);
int b200rl_mlp_evaluate_ws(const b200rl_mlp_shape* shape, const float* params, const float* x, int ldx, float* y, int ldy,
                           float* tick, float* tock, int batch, void* workspace, size_t workspace_bytes, b200rl_stream_t stream);
int b200rl_mlp_forward_ws(const b200rl_mlp_shape* shape, const float* params, const float* x, int ldx, float* pre, float* out,
                          int batch, void* workspace, size_t workspace_bytes, b200rl_stream_t stream);

/* backward through all layers; d_out [batch, O_last] is clobbered; grads accumulate (grads == NULL: only the input gradient is
 * propagated, backward_input of nn_models/mlp/operations_generic.h:130-150, d_input required); d_input may be NULL
 * (input layer then gets the weights-only backward, nn_models/mlp/operations_generic.h:180-204; non-NULL gives
 * backward_full :152-179). tick/tock: two [batch, max(dim)] buffers. scratch as for b200rl_dense_backward with the
 * largest layer. */
size_t b200rl_mlp_backward_scratch_bytes(const b200rl_mlp_shape* shape, int batch);
int b200rl_mlp_backward(const b200rl_mlp_shape* shape, const float* params, float* grads, const float* x, int ldx, const float* pre,
                        const float* out, float* d_out, float* d_input, float* tick, float* tock, int batch,
                        void* scratch, size_t scratch_bytes, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Adam. Hyper-parameters as nn::optimizers::adam::Parameters (nn/optimizers/adam/adam.h:13-25).
 * ------------------------------------------------------------------------------------------------------- */
typedef struct {
    float alpha, beta_1, beta_2, epsilon, epsilon_sqrt;
} b200rl_adam_hyper;

/* Device-resident optimizer state, 4 x 32-bit words: {uint32 age, uint32 ticket, float c1, float c2}.
 * b200rl_adam_reset sets age = 1 (reset_optimizer_state, nn/optimizers/adam/operations_generic.h:43-46). */
int b200rl_adam_reset(uint32_t* state, b200rl_stream_t stream);

/* One optimizer step over a flat arena of n parameters, ONE launch:
 *   c1 = 1/(1-beta_1^age), c2 = 1/(1-beta_2^age), age += 1          (_step, adam/operations_generic.h:49-59)
 *   m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g g;  p -= alpha c1 m / (sqrt(max(v c2, eps_sqrt)) + eps)
 * Replaces the <<<1,1>>> _step kernel plus one update_kernel per layer (nn/optimizers/adam/operations_cuda.h:56-69,
 * nn/layers/dense/operations_cuda.h:193-233,434-446). The age lives on the device so the call can sit inside a
 * captured CUDA graph; the last block to finish bumps it. */
int b200rl_adam_step(float* params, const float* grads, float* m, float* v, size_t n, b200rl_adam_hyper hyper, uint32_t* state,
                     b200rl_stream_t stream);

/* Per-tensor form of the same optimizer for hosts that keep the reference's one-tensor-per-parameter storage and its
 * device-resident optimizer struct (nn::optimizers::Adam: parameters, bias-correction scalars, age):
 *   hyper9 -> nn::optimizers::adam::Parameters<float> on the device (alpha, beta_1, beta_2, epsilon, epsilon_sqrt, ...);
 *   b200rl_adam_advance_dev = _step (nn/optimizers/adam/operations_cuda.h:56-58): c1, c2 from the age, age += 1;
 *   b200rl_adam_update_dev  = update of one parameter tensor (nn/optimizers/adam/instance/operations_cuda.h:60-70). */
int b200rl_adam_advance_dev(const float* hyper9, uint32_t* age, float* c1, float* c2, b200rl_stream_t stream);
int b200rl_adam_update_dev(float* params, const float* grads, float* m, float* v, size_t n, const float* hyper9, const float* c1,
                           const float* c2, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * PPO update pieces (host scalar loops in the reference, which therefore cannot run on its CUDA device).
 * All column arguments carry an element pitch (ld_*): pass the dataset matrix's row pitch to work on column views of the
 * on-policy dataset (rl/components/on_policy_runner/on_policy_runner.h:38-72, row = step * n_envs + env), or 1 for plain
 * arrays. Flags are stored as floats (non-zero = true), as the dataset stores them.
 * ------------------------------------------------------------------------------------------------------- */

/* Generalized advantage estimation, one backward scan per environment. all_values has (steps + 1) * n_envs rows.
 * Replaces estimate_generalized_advantages (rl/algorithms/ppo/operations_generic.h:59-95). */
int b200rl_gae(const float* rewards, int ld_rewards, const float* all_values, int ld_values, const float* terminated, int ld_terminated,
               const float* truncated, int ld_truncated, float* advantages, int ld_advantages, float* target_values, int ld_targets,
               int n_envs, int steps, float gamma, float lambda, int ignore_termination, b200rl_stream_t stream);

/* Gradient of the clipped-surrogate PPO loss of one minibatch with respect to the actor output (d_actions [batch, A]) and
 * the state-independent log_std (d_log_std [A], ACCUMULATED): advantage mean/std over the minibatch, Gaussian log-prob of
 * the rollout actions under the current policy, ratio clipping, entropy bonus.
 * Replaces the per-sample loop of train (rl/algorithms/ppo/operations_generic.h:173-184, 214-296; Gaussian head
 * random/operations_generic.h:87-121). current_actions = actor forward output on the minibatch observations.
 * scratch: b200rl_ppo_scratch_bytes(batch, action_dim) bytes of device memory; action_dim <= 64. */
size_t b200rl_ppo_scratch_bytes(int batch, int action_dim);
int b200rl_ppo_policy_gradient(const float* current_actions, int ld_current, const float* rollout_actions, int ld_rollout, const float* log_std,
                               const float* rollout_log_probs, int ld_log_probs, const float* advantages, int ld_advantages, float* d_actions, int ld_d,
                               float* d_log_std, int batch, int action_dim, float epsilon_clip, float entropy_coefficient, float advantage_epsilon,
                               int normalize_advantage, int learn_action_std, void* scratch, size_t scratch_bytes, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Device memory and copies for hosts compiled without the CUDA toolkit (the header-only adapter needs nothing but
 * this header). Replace cudaMalloc / cudaFree / cudaMemcpyAsync + synchronise in containers/matrix/operations_cuda.h
 * :16-40,105-195 and containers/tensor/operations_cuda.h:16-40,74-166. kind: 0 = host to device, 1 = device to host,
 * 2 = device to device. b200rl_memcpy_2d copies `rows` rows of `width_bytes` with independent pitches (views).
 * Copies that touch host memory synchronise the stream before returning, as the reference's do.
 * ------------------------------------------------------------------------------------------------------- */
int b200rl_device_malloc(void** ptr, size_t bytes);
int b200rl_device_free(void* ptr);
int b200rl_memcpy(void* dst, const void* src, size_t bytes, int kind, b200rl_stream_t stream);
int b200rl_memcpy_2d(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes, size_t width_bytes, size_t rows, int kind,
                     b200rl_stream_t stream);
int b200rl_stream_synchronize(b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Pendulum rollout: T x { reset-if-truncated, observe, actor forward, step, reward, counters } for N environments in
 * ONE persistent launch. Semantics per step are the off-policy runner's prologue / interlude / epilogue with
 * deterministic actions (rl/components/off_policy_runner/operations_generic_per_env.h:8-108,
 * operations_cuda.h:60-115,184-204) on rl::environments::Pendulum with default parameters
 * (rl/environments/pendulum/pendulum.h:11-25, operations_generic.h:57-160); T == 1 is one runner step.
 *   states [N,2] (theta, theta_dot), episode_step [N], truncated [N] (0/1), episode_return [N]: in/out runner state
 *   (truncated starts as 1 so the first step resets, off_policy_runner/operations_generic.h init);
 *   reset_states [R,N,2] (any 4-byte aligned address: it is read with scalar loads, so a view into a larger table works): the k-th
 *   reset of env e inside this call takes reset_states[k][e]; the values are drawn on
 *   the host in the reference engine's order (b200rl_reset_table_host), mirroring how the reference's own CPU<->GPU
 *   tests feed CPU-drawn noise to the device; may be NULL if no env can reset during the call;
 *   obs [T*N,3], act [T*N,1], rew [T*N,1]: row t*N + env.
 *   error_flag (device int, may be NULL) is set to 1 if an env needed more than R resets.
 * The actor must be 3 -> H -> H -> 1 with H in {16, 32, 64, 128}; activations are free. H = 64 runs on the tensor-core kernel, the other
 * widths on the one-thread-per-environment kernel of b200rl_env_rollout (the device_rng, collect and runner-step entries take H = 64 only). */
int b200rl_pendulum_rollout(const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step,
                            uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds,
                            int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, int* error_flag,
                            b200rl_stream_t stream);

/* HOST-buffer variant of the above: every pointer except `stream` is host memory (pinned host memory makes the
 * copies asynchronous). Copies the runner state and reset table in, runs the rollout in slabs of steps and streams the
 * obs/act/rew slabs back while the next slab computes; synchronises before returning. Allocates its device staging
 * on first use and keeps it (freed by b200rl_release_host_staging). This is the call a host-side user of the
 * runner makes when the rollout data is consumed on the CPU. */
int b200rl_pendulum_rollout_host(const b200rl_mlp_shape* actor, const float* actor_params_host, float* states_host,
                                 int32_t* episode_step_host, uint8_t* truncated_host, float* episode_return_host,
                                 const float* reset_states_host, int n_reset_rounds, int n_envs, int n_steps, int step_limit,
                                 float* obs_host, float* act_host, float* rew_host, b200rl_stream_t stream);
int b200rl_release_host_staging(void);

/* Reference-compatible random streams on the HOST (std::mt19937 seeded with seed+1 and libstdc++'s
 * uniform_real_distribution<float>, exactly what random/operations_cpu.h:21-35 drives), so that resets are
 * bit-identical to a reference CPU run. rng_state_host is 625 x uint32 owned by the caller. */
int b200rl_rng_init_host(uint32_t* rng_state_host, uint32_t seed);
/* init_weights of one dense layer on that host engine, uploaded to W [O, I] and bias [O] (synchronises): per output row the bias draw
 * U(-bias_bound, bias_bound) (skipped, bias = 0, when draw_biases == 0) followed by the row's I weight draws U(-weight_bound, weight_bound)
 * -- the draw order of nn/layers/dense/operations_generic.h:59-87. The reference's default (legacy Kaiming-uniform, layer.h:28-39) is
 * weight_bound = bias_bound = 1 / sqrt(I) evaluated in float as sqrt(3) * (sqrt(2 / (1 + sqrt(5)^2)) / sqrt(I)) and 1 / sqrt(I).
 * Replaces the CUDA form nn/layers/dense/operations_cuda.h:17-67 (which draws on its device engines). */
int b200rl_dense_init_weights(uint32_t* rng_state_host, float weight_bound, float bias_bound, int draw_biases, float* W, float* bias,
                              int input_dim, int output_dim, b200rl_stream_t stream);
/* randn(device, matrix, rng) with the host engine: rows * cols standard normals in row-major order (one fresh
 * std::normal_distribution per element, random/operations_cpu.h:40-48) into a device matrix with row pitch ld; synchronises.
 * Replaces containers/matrix/operations_cuda.h:197-223 for callers that need the host stream's exact values. */
int b200rl_randn_host_rng(uint32_t* rng_state_host, float* dst, int ld, int rows, int cols, b200rl_stream_t stream);
/* Fills reset_states_host [R,N,2] in the runner's draw order (each step, envs ascending, theta then theta_dot for
 * every truncated env; off_policy_runner/operations_cpu.h:46-50) for a call of n_steps steps starting from the
 * given counters. Returns the number of reset rounds used in *rounds_used_host. */
int b200rl_reset_table_host(uint32_t* rng_state_host, int n_envs, int n_steps, const int32_t* episode_step_host,
                            const uint8_t* truncated_host, int step_limit, float* reset_states_host, int n_reset_rounds,
                            int* rounds_used_host);

/* ---------------------------------------------------------------------------------------------------------
 * On-policy collect for PPO: T x { reset-if-truncated, observe, actor forward -> action mean, Gaussian action noise, log-prob,
 * step, reward, flags } for N Pendulum environments in ONE launch, written as rows of the runner's dataset matrix.
 * Replaces collect (rl/components/on_policy_runner/operations_generic.h:105-146; prologue / epilogue per environment
 * operations_generic_per_env.h:9-79; Gaussian head random/operations_cpu.h:40-48, random/operations_generic.h:87-97).
 *   dataset [(T + 1) * N, ld_dataset], row = step * N + env, columns as on_policy_runner.h:38-72 for observation 3 / action 1:
 *     0-2 observation, 3 action mean, 4 action, 5 log-prob, 6 reward, 7 terminated, 8 truncated, 9 reset, 10 value, 11 advantage,
 *     12 target value (10-12 are not touched). reset[env] of step 0 = the incoming truncated flag, reset[pos + N] = truncated[pos];
 *     rows T * N + env receive the final observation. ld_dataset >= 13.
 *   noise [T, N]: the standard-normal variate of every action draw, reset_states [R, N, 2]: both in the order the reference's single
 *     engine produces them (b200rl_collect_tables_host); action = noise * exp(log_std) + mean.
 *   log_std: device scalar (the state-independent log standard deviation of nn_models/mlp_unconditional_stddev).
 *   step_limit == 0 disables truncation. Runner state arguments as in b200rl_pendulum_rollout.
 * The actor must be 3 -> 64 -> 64 -> 1. The _layers variant takes the six parameter tensors W1 b1 W2 b2 W3 b3 as separate device
 * pointers (how the reference's containers allocate them) and packs them into a file-scope device arena first; that arena is shared by
 * all calls on a device, which are therefore ordered with an event -- a stream that is being captured is refused (B200RL_ERR_UNSUPPORTED):
 * capture the flat-arena entry point instead. */
#define B200RL_COLLECT_DATA_DIM 13
int b200rl_pendulum_collect(const b200rl_mlp_shape* actor, const float* actor_params, const float* log_std, float* states,
                            int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states,
                            int n_reset_rounds, const float* noise, int n_envs, int n_steps, int step_limit, float* dataset,
                            int ld_dataset, int* error_flag, b200rl_stream_t stream);
int b200rl_pendulum_collect_layers(const b200rl_mlp_shape* actor, const float* const* layer_params, const float* log_std,
                                   float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                                   const float* reset_states, int n_reset_rounds, const float* noise, int n_envs, int n_steps,
                                   int step_limit, float* dataset, int ld_dataset, int* error_flag, b200rl_stream_t stream);
/* Device-side random numbers: the same two kernels without host draw tables. Every (environment e, step s) owns one block of the
 * counter-based Philox-4x32-10 generator, counter = (e, s low, s high, 0), key = seed: words 0-1 give the standard-normal action noise
 * (Box-Muller), words 2-3 the initial state (theta uniform in (-pi, pi), theta_dot in (-1, 1), the distribution of
 * rl/environments/pendulum/operations_generic.h:57-61). s counts from first_step: pass the number of steps already collected so that
 * consecutive calls continue the stream. The draws do not depend on how environments are sharded over launches or GPUs. This is the
 * counterpart of the reference's device engines (random/operations_cuda.h uses cuRAND state per thread): statistically equivalent
 * to, not bit-identical with, the host engine of the table-driven entry points. */
int b200rl_pendulum_collect_device_rng(const b200rl_mlp_shape* actor, const float* actor_params, const float* log_std, float* states,
                                       int32_t* episode_step, uint8_t* truncated, float* episode_return, unsigned long long seed,
                                       unsigned long long first_step, int n_envs, int n_steps, int step_limit, float* dataset,
                                       int ld_dataset, int* error_flag, b200rl_stream_t stream);
int b200rl_pendulum_rollout_device_rng(const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step,
                                       uint8_t* truncated, float* episode_return, unsigned long long seed, unsigned long long first_step,
                                       int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, int* error_flag,
                                       b200rl_stream_t stream);
/* Host tables for one collect call in the reference engine's draw order (per step: environments ascending, initial state of every
 * truncated environment; then environments ascending, one normal draw per action). rng_state_host as in b200rl_rng_init_host,
 * advanced in place, so consecutive calls continue the reference's stream. */
int b200rl_collect_tables_host(uint32_t* rng_state_host, int n_envs, int n_steps, const int32_t* episode_step_host,
                               const uint8_t* truncated_host, int step_limit, float* reset_states_host, int n_reset_rounds,
                               int* rounds_used_host, float* noise_host);

/* ---------------------------------------------------------------------------------------------------------
 * Off-policy runner step with per-environment replay buffers: step<POLICY>(device, runner, policy, buffers, rng)
 * (rl/components/off_policy_runner/operations_generic.h:219-238, CUDA form operations_cuda.h:184-204): reset-if-truncated from
 * reset_states [N, 2] (one round, drawn on the host in environment order for the environments whose truncated flag is set), observe
 * into observations [N, 3], actor forward into actions [N, 1], step + reward, counters, next_observations [N, 3], then the transition
 * is appended to the environment's replay buffer (rl/components/replay_buffer/operations_generic.h:54-79: row = observation 3,
 * action 1, reward 1, next observation 3, terminated, truncated; episode_start[position] = current_episode_start; position wraps at
 * capacity; full is set when it returns to 0; a reset marks the previous transition truncated, operations_generic_per_env.h:41-52).
 * The replay buffers are described by byte offsets into one struct per environment, so that the reference's statically allocated
 * ReplayBuffer structs in device memory can be written in place. Either actor_params (flat arena) or layer_params (six tensors).
 * reward_scratch [N] floats and was_truncated_scratch [N] bytes are work areas. Like the reference (whose add() overload for
 * ReplayBufferWithStates is not selected), the per-transition state copies are not written. */
typedef struct b200rl_replay_layout {
    size_t env_stride;                    /* bytes from one environment's replay buffer to the next */
    size_t off_data;                      /* data matrix [capacity, ld_data] floats */
    size_t off_episode_start;             /* episode_start [capacity] indices */
    size_t off_position, off_full, off_current_episode_start;   /* index, 1-byte flag, index */
    int capacity, ld_data, index_bytes;   /* index_bytes: 4 or 8 */
} b200rl_replay_layout;
int b200rl_pendulum_offpolicy_step(const b200rl_mlp_shape* actor, const float* actor_params, const float* const* layer_params, float* states,
                                   int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int n_envs,
                                   int step_limit, float* observations, float* actions, float* next_observations, void* replay_buffers,
                                   const b200rl_replay_layout* layout, float* reward_scratch, uint8_t* was_truncated_scratch, int* error_flag,
                                   b200rl_stream_t stream);

/* The same runner step in two halves around ANY policy -- how the reference's CUDA runner is built (operations_cuda.h:184-204: prologue
 * kernel, evaluate(policy), epilogue kernel): an exploration policy with a stochastic head (SAC's sample-and-squash actor) is evaluated by
 * the caller between the two calls.
 * prologue: reset-if-truncated (reset_states [N, 2] in environment order, or, if NULL, drawn in the kernel from the counter-based generator
 *   keyed by (seed, environment, call + *call_counter); call_counter is an optional device-resident 64-bit integer, so that a captured
 *   graph draws fresh states on every replay), episode counters of a fresh episode, observations [N, 3]; was_truncated_scratch [N] keeps
 *   the truncated flags for the epilogue.
 * epilogue: environment step with actions [N, 1], reward, counters, truncation at step_limit, next_observations [N, 3], append to the
 *   replay buffers (layout and bookkeeping as in b200rl_pendulum_offpolicy_step). */
int b200rl_pendulum_offpolicy_prologue(float* states, int32_t* episode_step, const uint8_t* truncated, float* episode_return, const float* reset_states,
                                       unsigned long long seed, unsigned long long call, const unsigned long long* call_counter, int n_envs,
                                       float* observations, uint8_t* was_truncated_scratch, b200rl_stream_t stream);
int b200rl_pendulum_offpolicy_epilogue(float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return, int n_envs, int step_limit,
                                       const float* observations, const float* actions, float* next_observations, void* replay_buffers,
                                       const b200rl_replay_layout* layout, const uint8_t* was_truncated_scratch, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * L2F quadrotor, the configuration of the reference's own GPU throughput harness (src/rl/environments/l2f/cuda/benchmark.cu:31-60: state =
 * StateRotors<StateRandomForce<StateBase>>): n_steps x step(device, env, parameters, state, action, next_state, rng)
 * (rl/environments/l2f/operations_generic.h:93-131) per quadrotor, in place. A state row is position 3, orientation quaternion 4 (w first),
 * linear velocity 3, angular velocity 3, disturbance force 3, disturbance torque 3 (constant over the steps), rotor speeds 4 = 23 floats;
 * actions [n, 4] are the normalised rotor set-points a policy emits (clamped to [-1, 1], constant over the steps of a call). parameters
 * (host): dynamics = the 85 floats of the reference's parameters.dynamics in declaration order (multirotor.h:22-41: rotor positions, thrust
 * and torque directions [4][3], thrust coefficients [4][3], torque constants, rising / falling time constants [4], mass, gravity [3], J,
 * J_inv [3][3], hovering throttle, action limits min / max), the integration step and the three STATE_LIMIT_* constants. The action noise of
 * the default parameter set is 0 and is not applied; observation, reward, termination and the randomised initial state / parameters of the
 * environment are not part of this entry point. Results equal the reference's CPU step bit for bit (the kernel keeps its association and
 * is compiled without multiply-add contraction).
 * ------------------------------------------------------------------------------------------------------- */
typedef struct b200rl_l2f_parameters {
    float dynamics[85];
    float dt;
    float state_limit_position, state_limit_velocity, state_limit_angular_velocity;
} b200rl_l2f_parameters;
int b200rl_l2f_steps(const b200rl_l2f_parameters* parameters, float* states, const float* actions, int n, int n_steps, b200rl_stream_t stream);
/* The runner loop on this environment, fused like b200rl_env_rollout: per step reset-if-truncated from reset_states [R, N, 23] (the k-th reset
 * of environment e inside the call takes reset_states[k][e]; initial states are the caller's, e.g. the reference's sample_initial_state drawn on
 * the host), observe (rl/environments/l2f/operations_generic/40_observe.h:42-147: position 3, rotation matrix 9, linear velocity 3, angular
 * velocity 3 = 18 values; the default observation noise is 0), actor forward 18 -> H -> H -> 4 (H in {16, 32, 64}; fp32 FMA chains in the
 * reference's order), step, reward (parameters/reward_functions/squared/operations_generic.h:12-103, desired state at the origin), terminated
 * on the next state (operations_generic.h:143-158); an episode ends (truncated) at termination or at step_limit
 * (rl/components/off_policy_runner/operations_generic_per_env.h:62-108). mdp (host, 18 floats): the reward function's non_negative flag, scale,
 * constant, termination penalty and its weights position, position clip, orientation, linear velocity, angular velocity, linear acceleration,
 * angular acceleration, action, d_action, position error integral; then termination enabled, position / linear velocity / angular velocity
 * thresholds. obs [T * N, 18], act [T * N, 4], rew [T * N], terminated [T * N] (may be NULL), row = step * N + env; error_flag as for the
 * other rollouts. Next states equal the reference's bit for bit given the action; observations bit for bit; the reward within the GPU's acosf. */
int b200rl_l2f_rollout(const b200rl_l2f_parameters* parameters, const float* mdp, const b200rl_mlp_shape* actor, const float* actor_params, float* states,
                       int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps,
                       int step_limit, float* obs, float* act, float* rew, uint8_t* terminated, int* error_flag, b200rl_stream_t stream);
/* sample_initial_state(device, env, parameters, state, rng) of the same configuration (rl/environments/l2f/operations_generic/
 * 30_sample_initial_state.h:19-207) as a function of its draws: uniforms [n, 17] in [0, 1) (guidance; position 3; orientation u, v, angle;
 * linear velocity 3; angular velocity 3; rotor speeds 4), normals [n, 6] standard normals (force 3, torque 3). init (host, 12 floats):
 * mdp.init guidance, max_position, max_angle, max_linear_velocity, max_angular_velocity, relative_rpm, min_rpm, max_rpm, then the
 * disturbances' force mean / std and torque mean / std. states [n, 23]; equal to the reference's bit for bit except the orientation
 * (the GPU's sinf / cosf). */
int b200rl_l2f_initial_states_from_draws(const b200rl_l2f_parameters* parameters, const float* init, const float* uniforms, const float* normals, float* states, int n,
                                         b200rl_stream_t stream);
/* b200rl_l2f_rollout with the initial state of every reset drawn in the kernel from `init` (a counter-based generator keyed by seed,
 * environment and first_step + step, as b200rl_pendulum_rollout_device_rng: no reset table, any number of resets). */
int b200rl_l2f_rollout_device_rng(const b200rl_l2f_parameters* parameters, const float* mdp, const float* init, const b200rl_mlp_shape* actor, const float* actor_params,
                                  float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return, unsigned long long seed,
                                  unsigned long long first_step, int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, uint8_t* terminated,
                                  b200rl_stream_t stream);
/* The off-policy runner step on this environment in two halves around ANY policy, like b200rl_pendulum_offpolicy_prologue / _epilogue
 * (rl/components/off_policy_runner/operations_cuda.h:184-204 around operations_generic_per_env.h:8-61 and :62-108). Prologue: environments
 * whose truncated flag is set are reset -- from reset_states [n, 23] when given, else drawn in the kernel from `init` (12 floats, see
 * b200rl_l2f_initial_states_from_draws) with the generator keyed by (seed, environment, call + *call_counter) -- and start a fresh episode;
 * observations [n, 18]; was_truncated_scratch [n] remembers the flags for the epilogue. Epilogue: step with actions [n, 4], reward,
 * terminated on the next state, counters (an episode ends at termination or at step_limit), next_observations [n, 18], and the transition
 * appended to the environment's replay buffer (row = observation 18 | action 4 | reward | next observation 18 | terminated | truncated:
 * layout->ld_data >= 43; rl/components/replay_buffer/operations_generic.h:54-79). */
int b200rl_l2f_offpolicy_prologue(const b200rl_l2f_parameters* parameters, const float* init, float* states, int32_t* episode_step, const uint8_t* truncated,
                                  float* episode_return, const float* reset_states, unsigned long long seed, unsigned long long call,
                                  const unsigned long long* call_counter, int n_envs, float* observations, uint8_t* was_truncated_scratch, b200rl_stream_t stream);
int b200rl_l2f_offpolicy_epilogue(const b200rl_l2f_parameters* parameters, const float* mdp, float* states, int32_t* episode_step, uint8_t* truncated,
                                  float* episode_return, int n_envs, int step_limit, const float* actions, float* next_observations, void* replay_buffers,
                                  const b200rl_replay_layout* layout, const uint8_t* was_truncated_scratch, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Replay-buffer sampling: gather_batch(device, runner, batch, rng) for SequentialBatch with SEQUENCE_LENGTH 1 and its default sampling
 * parameters (rl/components/off_policy_runner/operations_generic.h:239-423, off_policy_runner.h:80-156; CUDA form
 * operations_cuda.h:136-182). Per batch element the reference draws the environment index, then a sample offset in [0, eligible - 1]
 * (eligible = full ? capacity : position of that environment's replay buffer); the transition index is the offset, or
 * (position + max_episode_length + offset) mod capacity once the buffer is full. Outputs (device):
 *   oa_base [2, batch, ld_oa]: step 0 = observation | action of the transition, step 1 = its next observation | zeros
 *     (observations_actions_base of the batch: observations_current / actions_current view step 0, observations_next step 1);
 *   rewards [batch] floats; terminated, reset (= 1), final_step_mask (= 1) [batch] bytes;
 *   next_reset_base (= 1, 1), next_final_step_mask_base (= 0, 1) [2, batch] bytes.
 * Rows of the replay data matrix are observation | action | reward | next observation | terminated | truncated
 * (rl/components/replay_buffer/replay_buffer.h:32-62). max_episode_length is the ENVIRONMENT's EPISODE_STEP_LIMIT
 * (off_policy_runner.h:41). An index outside its range sets *error_flag = 2 and skips the element.
 * b200rl_replay_counters copies (position, full) of every environment's buffer into dense device arrays (for the host draws);
 * b200rl_gather_draws_host makes the draws on the reference-compatible host engine in the reference's order, advanced in place. */
int b200rl_replay_counters(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int32_t* position, uint8_t* full,
                           b200rl_stream_t stream);
int b200rl_gather_draws_host(uint32_t* rng_state_host, int n_envs, int batch, const int32_t* position_host, const uint8_t* full_host,
                             int capacity, int32_t* env_index_host, int32_t* sample_offset_host);
int b200rl_gather_batch(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim,
                        int action_dim, const int32_t* env_index, const int32_t* sample_offset, int batch, float* oa_base, int ld_oa,
                        float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                        uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream);

/* gather_batch for ANY sequence length (the same reference function; SequentialBatch with SEQUENCE_LENGTH = sequence_length, padded length
 * P = sequence_length + 1): per batch element the padded sequence is filled by walking the environment's replay buffer as gather_batch_step
 * does (operations_generic.h:239-411). flags are the batch's sampling parameters (off_policy_runner.h:80-87; the reference's defaults for
 * sequence_length > 1 are the first three together) and the DETERMINISTIC template flag of gather_batch:
 *   B200RL_GATHER_FROM_INITIAL_STATE  ALWAYS_SAMPLE_FROM_INITIAL_STATE: a sequence starts at the first step of the sampled transition's episode
 *   B200RL_GATHER_RANDOM_LENGTH       RANDOM_SEQ_LENGTH: sequences are cut at the nominal length with probability nominal_probability
 *                                     (NOMINAL_SEQUENCE_LENGTH_PROBABILITY, 0.5), else at a length drawn from 1 .. sequence_length - 1
 *   B200RL_GATHER_FIRST_STEP_TARGET   INCLUDE_FIRST_STEP_IN_TARGETS: next_reset views next_reset_base from step 0 instead of step 1
 *   B200RL_GATHER_DETERMINISTIC       environment 0 and sample offset = the batch element's index instead of draws
 * Draws come from the counter-based generator keyed by (seed, batch element, call_index + *call_counter); call_counter (device, 64-bit) may be
 * NULL. Outputs (device): oa_base [P, batch, ld_oa] (observation | action per step; the step after a sequence's last transition holds that
 * transition's next observation and a zero action), rewards [L, batch] floats, terminated / reset / final_step_mask [L, batch] bytes,
 * next_reset_base / next_final_step_mask_base [P, batch] bytes. Entries the reference leaves unwritten (rewards of padding steps, rows behind the
 * last sequence's end) are left as they are. An empty sampling range sets *error_flag = 2 and skips the element. */
#define B200RL_GATHER_FROM_INITIAL_STATE 1
#define B200RL_GATHER_RANDOM_LENGTH 2
#define B200RL_GATHER_FIRST_STEP_TARGET 4
#define B200RL_GATHER_DETERMINISTIC 8
int b200rl_gather_batch_sequences(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim, int action_dim,
                                  int sequence_length, int flags, float nominal_probability, unsigned long long seed, unsigned long long call_index,
                                  const unsigned long long* call_counter, int batch, float* oa_base, int ld_oa, float* rewards, uint8_t* terminated, uint8_t* reset,
                                  uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream);

/* The same gather with both indices drawn inside the kernel (the counterpart of the reference's device-side sampling,
 * operations_cuda.h:166-182): Philox-4x32-10 block (batch element, call_index low, call_index high, 1) keyed by seed, word 0 -> environment,
 * word 1 -> sample offset, each bounded by the high half of word * range. No host round trip: usable inside a captured graph when
 * call_index is advanced by the caller between launches. An empty replay buffer sets *error_flag = 2. */
int b200rl_gather_batch_device_rng(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length,
                                   int obs_dim, int action_dim, unsigned long long seed, unsigned long long call_index, int batch,
                                   float* oa_base, int ld_oa, float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base,
                                   uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * SAC update pieces (rl/algorithms/sac/operations_generic.h, CUDA forms rl/algorithms/sac/operations_cuda.h and
 * nn/layers/sample_and_squash/operations_cuda.h). All matrices row-major with row pitches ld_*.
 *
 * Sample-and-squash policy head with external noise (nn/layers/sample_and_squash/operations_generic.h:149-195, 212-260):
 *   input [B, 2A] = mean | log_std; log_std clamped to [-20, 2]; sample = mean + noise * exp(log_std); output = tanh(sample);
 *   log_probs[b] = sum_a normal_log_prob(mean, log_std, sample) - log(1 - output^2 + 1e-6). pre_squashing [B, A] dense (needed by the
 *   backward pass) and log_probs may be NULL.
 * Backward (backward_full, :290-398): d_input [B, 2A] from d_output [B, A] plus the entropy term alpha / B * d log_prob, zero log_std
 *   gradient outside the clamp; d_log_alpha_per_sample[b] = alpha * (entropy_b - target_entropy); their in-order sum / B is ADDED to
 *   *log_alpha_gradient (NULL skips it). log_alpha: device scalar. */
int b200rl_sample_and_squash_forward(const float* input, int ld_in, const float* noise, int ld_noise, int batch, int action_dim, float* pre_squashing,
                                     float* output, int ld_out, float* log_probs, b200rl_stream_t stream);
int b200rl_sample_and_squash_backward(const float* input, int ld_in, const float* noise, int ld_noise, const float* pre_squashing, const float* output,
                                      int ld_out, const float* d_output, int ld_dout, const float* log_alpha, float target_entropy, int batch,
                                      int action_dim, float* d_input, int ld_din, float* d_log_alpha_per_sample, float* log_alpha_gradient,
                                      b200rl_stream_t stream);
/* Critic target (target_action_values, rl/algorithms/sac/operations_generic.h:133-178): min of the two target critics' values at the next
 * state, entropy bonus -alpha * next_log_prob (inside or outside the discounted term), gamma, termination mask, reward. */
int b200rl_sac_target_action_values(const float* q1_next, int ld_q1, const float* q2_next, int ld_q2, const float* rewards, const uint8_t* terminated,
                                    const float* next_log_probs, const float* log_alpha, float gamma, int ignore_termination, int entropy_bonus,
                                    int entropy_bonus_next_step, float* target, int ld_target, int batch, b200rl_stream_t stream);
/* Actor loss gradient w.r.t. the action (min_value_d_output, :341-376): columns [action_offset, action_offset + A) of the input gradient of
 * whichever critic has the smaller value for that sample (critic 1 if q1 < q2). */
int b200rl_sac_min_value_d_output(const float* q1, int ld_q1, const float* q2, int ld_q2, const float* d_critic_1_input, const float* d_critic_2_input,
                                  int ld_d_input, int action_offset, int action_dim, float* d_actor_output, int ld_out, int batch,
                                  b200rl_stream_t stream);

/* The small tensor operations between the network passes of train_critic / train_actor, with every operand in device memory, so that the
 * reference's generic verbs (rl/algorithms/sac/operations_generic.h:243-336, 378-456) run on the device without a host read-back.
 *  b200rl_mse_gradient_dev_weight  mse::gradient with the loss weight in a one-element device tensor (nn/loss_functions/mse/operations_generic.h:66-79)
 *  b200rl_mask_count               result[0] = number of set entries of a bool mask (cast_reduce_sum<T>, containers/tensor/operations_generic.h:838-845;
 *                                  CUDA form containers/tensor/operations_cuda.h:308-315), n < 2^24
 *  b200rl_scale                    t[i] = t[i] * scale, or (1 / t[i]) * scale with reciprocal != 0 (scale, containers/tensor/operations_generic.h:712-719, 433-445)
 *  b200rl_fill_from_device         dst[0..n) = value[0] (set_all(tensor, one-element tensor), :741-748)
 *  b200rl_mask_rows                rows r of target [rows, cols] with (mask[r] != 0) != (invert != 0) receive row r of source, or zeros when source == NULL
 *                                  (mask_actions and mask_gradient, rl/algorithms/sac/operations_generic.h:180-232; CUDA forms sac/operations_cuda.h:76-127) */
int b200rl_mse_gradient_dev_weight(const float* a, int lda, const float* b, int ldb, float* d_a, int ldd, int rows, int cols, const float* loss_weight,
                                   b200rl_stream_t stream);
int b200rl_mask_count(const uint8_t* mask, size_t n, float* result, b200rl_stream_t stream);
int b200rl_scale(float* t, size_t n, float scale, int reciprocal, b200rl_stream_t stream);
int b200rl_fill_from_device(float* dst, size_t n, const float* value, b200rl_stream_t stream);
int b200rl_mask_rows(const float* source, int ld_source, float* target, int ld_target, const uint8_t* mask, int rows, int cols, int invert,
                     b200rl_stream_t stream);

/* Randomness kept entirely on the device, for update loops captured in a CUDA graph: *call_counter (a device-resident 64-bit integer)
 * takes the place of call_index in the sampling kernel and in the normal generator, and b200rl_counter_advance adds to it on the stream,
 * so that every replay of one captured graph draws fresh indices and noise. b200rl_randn_device_rng fills dst[0..n) with standard normals:
 * Philox block (element / 4, call low, call high, 2 + stream_id) keyed by seed, Box-Muller on the word pairs; call = call_index +
 * *call_counter (call_counter may be NULL); different stream_id values give independent streams for the same call (the counterpart of
 * the reference's randn(device, matrix, rng) on its device engines, containers/matrix/operations_cuda.h:197-223). */
int b200rl_counter_advance(unsigned long long* call_counter, unsigned long long increment, b200rl_stream_t stream);
int b200rl_randn_device_rng(float* dst, size_t n, unsigned long long seed, unsigned int stream_id, unsigned long long call_index,
                            const unsigned long long* call_counter, b200rl_stream_t stream);
int b200rl_gather_batch_device_counter(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length,
                                       int obs_dim, int action_dim, unsigned long long seed, const unsigned long long* call_counter, int batch,
                                       float* oa_base, int ld_oa, float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base,
                                       uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * Observation normalisation of the PPO loop (rl/algorithms/ppo/loop/core/operations_generic.h:99-131): per loop step the running
 * normaliser is updated with the collected observations and its statistics are handed to the standardize layer in front of actor and critic.
 * b200rl_running_normalizer_update: update(device, normalizer, data) (rl/components/running_normalizer/operations_generic.h:27-47):
 *   per column the batch mean and the batch standard deviation about that mean (0 when the sum of squared deviations is below 1e-6, else
 *   sqrt(sum / (rows - 1))), then running += (batch - running) / age. age = the normaliser's age AFTER its increment (a host integer in
 *   the reference). The column sums are taken in double and rounded once (the reference sums in fp32 in row order).
 * b200rl_standardize_set_statistics: set_statistics (nn/layers/standardize/operations_generic.h:52-66): precision = std == 0 ? 0 : 1 / std.
 * b200rl_standardize_forward: evaluate / forward of the layer (:69-92; CUDA form nn/layers/standardize/operations_cuda.h): (x - mean) * precision,
 *   the product skipped where precision is 0. The layer has no trainable parameters; as the first layer of its network it needs no backward. */
int b200rl_running_normalizer_update(const float* data, int ld, int rows, int dim, float* mean, float* std, unsigned long long age,
                                     b200rl_stream_t stream);
int b200rl_standardize_set_statistics(const float* mean, const float* std, int dim, float* layer_mean, float* layer_precision, b200rl_stream_t stream);
int b200rl_standardize_forward(const float* x, int ldx, const float* mean, const float* precision, float* y, int ldy, int rows, int dim,
                               b200rl_stream_t stream);

/* ---------------------------------------------------------------------------------------------------------
 * The fused rollout of b200rl_pendulum_rollout for environments given as device functions (CUDA-core kernel): the same runner
 * semantics (rl/components/off_policy_runner/operations_generic_per_env.h:8-108 with deterministic actions), T steps per launch.
 *   B200RL_ENV_PENDULUM:        state [N, 2], observation 3 (rl/environments/pendulum/operations_generic.h)
 *   B200RL_ENV_ACROBOT_SWINGUP: state [N, 4] = theta_1, theta_2, theta_1_dot, theta_2_dot, observation 6 = cos / sin of both angles and
 *                               the velocities; RK4 step of dt 0.2, swing-up reward on the next state, never terminates
 *                               (rl/environments/acrobot/operations_generic.h:46-199, default parameters acrobot.h:11-27)
 *   B200RL_ENV_ACROBOT:         the variant that TERMINATES (rl::environments::Acrobot): same dynamics and observation, reward -1 per step
 *                               (:154-156), terminated when the tip is above the bar, evaluated on the next state (:193-195); an episode ends
 *                               (truncated) at termination or at the step limit (operations_generic_per_env.h:93-97)
 * reset_states [R, N, D] with D = b200rl_env_reset_dim(env): the draws of an initial state in the reference engine's order (Pendulum:
 * theta, theta_dot; AcrobotSwingup: theta_1, theta_2, velocities 0; Acrobot: all four components, U(-0.1, 0.1)).
 * The actor is OBS -> H -> H -> 1 with H in {16, 32, 64, 128}. obs [T * N, OBS], act / rew [T * N, 1], row = step * N + env.
 * b200rl_env_rollout_flags additionally writes the environment's terminated flag of every transition (terminated [T * N], may be NULL):
 * the column the replay buffer and the critic target need for environments that terminate. */
#define B200RL_ENV_PENDULUM 0
#define B200RL_ENV_ACROBOT_SWINGUP 1
#define B200RL_ENV_ACROBOT 2
int b200rl_env_observation_dim(int env);
int b200rl_env_state_dim(int env);
int b200rl_env_reset_dim(int env);
int b200rl_env_rollout(int env, const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step, uint8_t* truncated,
                       float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps, int step_limit, float* obs,
                       float* act, float* rew, int* error_flag, b200rl_stream_t stream);
int b200rl_env_rollout_flags(int env, const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step, uint8_t* truncated,
                       float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps, int step_limit, float* obs,
                       float* act, float* rew, uint8_t* terminated, int* error_flag, b200rl_stream_t stream);

/* Epoch shuffle of the PPO update (SHUFFLE_EPOCH, rl/algorithms/ppo/operations_generic.h:127-158): the reference swaps row i with a
 * row drawn by std::uniform_int_distribution from [i, n-1], for i = 0..n-1, on the observation, action, advantage, log-prob and
 * target-value columns. b200rl_shuffle_permutation_host replays those draws on the host engine (advanced in place, as the reference
 * would) and returns perm_host[i] = the original row that ends at position i; b200rl_permute_rows applies it on the device to the
 * columns whose bit is set in column_mask (columns < 64): data[i][c] = old data[perm[i]][c]. scratch: b200rl_permute_rows_scratch_bytes. */
int b200rl_shuffle_permutation_host(uint32_t* rng_state_host, int n_rows, int32_t* perm_host);
size_t b200rl_permute_rows_scratch_bytes(int n_rows, unsigned long long column_mask);
int b200rl_permute_rows(float* data, int ld, int n_rows, const int32_t* perm, unsigned long long column_mask, void* scratch, size_t scratch_bytes,
                        b200rl_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif
