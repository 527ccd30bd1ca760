// Entry points of the fused Pendulum rollout (reset-if-truncated, observe, actor forward 3 -> 64 -> 64 -> 1, environment step, reward and
// episode counters for T steps in ONE launch of the tensor-core kernel in rollout_tc.cu), of the on-policy collect, of the off-policy runner
// step with replay buffers, and of replay-buffer sampling.
#include "common.cuh"
#include "pendulum.cuh"
#include "rollout.cuh"
#include <mutex>

namespace b200rl {

int validate_actor(const b200rl_mlp_shape* actor){
    if(!actor) return B200RL_ERR_INVALID_ARGUMENT;
    if(actor->n_layers != 3 || actor->input_dim != 3 || actor->dims[2] != 1 || actor->dims[0] != actor->dims[1]) return B200RL_ERR_UNSUPPORTED;
    if(actor->dims[0] != 64) return B200RL_ERR_UNSUPPORTED;
    for(int l = 0; l < 3; l++) if(!valid_activation(actor->acts[l])) return B200RL_ERR_INVALID_ARGUMENT;
    return B200RL_OK;
}

// one kernel: the tensor-core rollout of the 64-wide actor (validate_actor admits nothing else)
int rollout_dispatch(const b200rl_mlp_shape* actor, const RolloutArgs& a, cudaStream_t s){
    if(actor->dims[0] != 64) return B200RL_ERR_UNSUPPORTED;
    return launch_rollout_tc(a, s);
}

}  // namespace b200rl
using namespace b200rl;

// device_rng: resets (and, for collect, the action noise) from the counter-based generator instead of host tables
struct DeviceRng { int enabled; unsigned long long seed, step0; };

static int rollout_launch(const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step,
                          uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds,
                          int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, int* error_flag,
                          DeviceRng rng, cudaStream_t stream){
    // hidden widths other than the tensor-core kernel's 64 run on the one-thread-per-environment kernel (table-driven resets only)
    if(actor && !rng.enabled && actor->n_layers == 3 && actor->input_dim == 3 && actor->dims[0] == actor->dims[1] && actor->dims[0] != 64)
        return b200rl_env_rollout(B200RL_ENV_PENDULUM, actor, actor_params, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds,
                                  n_envs, n_steps, step_limit, obs, act, rew, error_flag, (b200rl_stream_t)stream);
    int rc = validate_actor(actor);
    if(rc) return rc;
    if(!actor_params || !states || !episode_step || !truncated || !episode_return || !obs || !act || !rew || n_envs < 0 || n_steps < 0 || n_reset_rounds < 0 || step_limit < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(reset_states == nullptr && n_reset_rounds != 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0 || n_steps == 0) return B200RL_OK;
    RolloutArgs a{};
    a.params = actor_params; a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return;
    a.reset_states = reset_states; a.n_reset_rounds = n_reset_rounds; a.n_envs = n_envs; a.env_begin = 0; a.env_count = n_envs;
    a.n_steps = n_steps; a.step_limit = step_limit; a.obs = obs; a.act = act; a.rew = rew; a.error_flag = error_flag;
    a.device_rng = rng.enabled; a.rng_seed = rng.seed; a.rng_step0 = rng.step0;
    for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
    return rollout_dispatch(actor, a, stream);
}

extern "C" int b200rl_pendulum_rollout(const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step,
                                       uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds,
                                       int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, int* error_flag,
                                       b200rl_stream_t stream){
    return rollout_launch(actor, actor_params, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds, n_envs, n_steps,
                          step_limit, obs, act, rew, error_flag, DeviceRng{0, 0, 0}, (cudaStream_t)stream);
}

extern "C" int b200rl_pendulum_rollout_device_rng(const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step,
                                                  uint8_t* truncated, float* episode_return, unsigned long long seed, unsigned long long first_step,
                                                  int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, int* error_flag,
                                                  b200rl_stream_t stream){
    return rollout_launch(actor, actor_params, states, episode_step, truncated, episode_return, nullptr, 0, n_envs, n_steps,
                          step_limit, obs, act, rew, error_flag, DeviceRng{1, seed, first_step}, (cudaStream_t)stream);
}

// ---------------------------------------------------------------------------------------------------------------
// On-policy collect (rl/components/on_policy_runner/operations_generic.h:105-146): the same kernels with the Gaussian
// policy head and the dataset-row writer switched on.
// ---------------------------------------------------------------------------------------------------------------
static int collect_launch(const b200rl_mlp_shape* actor, const float* actor_params, const float* log_std, float* states, int32_t* episode_step,
                          uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds, const float* noise,
                          int n_envs, int n_steps, int step_limit, float* dataset, int ld_dataset, int* error_flag, cudaStream_t stream,
                          DeviceRng rng = DeviceRng{0, 0, 0}){
    int rc = validate_actor(actor);
    if(rc) return rc;
    if(!actor_params || !log_std || !states || !episode_step || !truncated || !episode_return || !dataset || n_envs < 0 || n_steps < 0 ||
       n_reset_rounds < 0 || step_limit < 0 || ld_dataset < COLLECT_DATA_DIM || (noise == nullptr && n_steps > 0 && !rng.enabled))
        return B200RL_ERR_INVALID_ARGUMENT;
    if(reset_states == nullptr && n_reset_rounds != 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    RolloutArgs a{};
    a.params = actor_params; a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return;
    a.reset_states = reset_states; a.n_reset_rounds = n_reset_rounds; a.n_envs = n_envs; a.env_begin = 0; a.env_count = n_envs;
    a.n_steps = n_steps; a.step_limit = step_limit; a.error_flag = error_flag;
    a.dataset = dataset; a.ld_dataset = ld_dataset; a.noise = noise; a.log_std = log_std;
    a.neg_half_log_2pi = (float)(-0.5 * logf(2 * 3.14159265358979323846f));      // random/operations_generic.h:89
    a.device_rng = rng.enabled; a.rng_seed = rng.seed; a.rng_step0 = rng.step0;
    for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
    return rollout_dispatch(actor, a, stream);
}

extern "C" int b200rl_pendulum_collect(const b200rl_mlp_shape* actor, const float* actor_params, const float* log_std, float* states,
                                       int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states,
                                       int n_reset_rounds, const float* noise, int n_envs, int n_steps, int step_limit, float* dataset,
                                       int ld_dataset, int* error_flag, b200rl_stream_t stream){
    return collect_launch(actor, actor_params, log_std, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds, noise,
                          n_envs, n_steps, step_limit, dataset, ld_dataset, error_flag, (cudaStream_t)stream);
}

extern "C" int b200rl_pendulum_collect_device_rng(const b200rl_mlp_shape* actor, const float* actor_params, const float* log_std, float* states,
                                                  int32_t* episode_step, uint8_t* truncated, float* episode_return, unsigned long long seed,
                                                  unsigned long long first_step, int n_envs, int n_steps, int step_limit, float* dataset,
                                                  int ld_dataset, int* error_flag, b200rl_stream_t stream){
    return collect_launch(actor, actor_params, log_std, states, episode_step, truncated, episode_return, nullptr, 0, nullptr,
                          n_envs, n_steps, step_limit, dataset, ld_dataset, error_flag, (cudaStream_t)stream, DeviceRng{1, seed, first_step});
}

// Actor given as separately allocated layer tensors (how the reference's containers hold them): packed into a file-scope
// device arena by device-to-device copies on the launch stream. Calls are ordered against each other by an event, since they
// share that arena.
static __device__ __align__(16) float g_collect_actor_arena[64 * 3 + 64 + 64 * 64 + 64 + 64 + 1 + 3];

// packs six separately allocated layer tensors (W1 b1 W2 b2 W3 b3) into the file-scope arena of the current device; *order_event is
// recorded by the caller after its kernel launch. The arena is shared by every call on the device, so calls are ordered with an event --
// which a stream capture cannot wait on (the event was recorded outside the capture): a capturing stream is refused.
static int pack_actor_layers(const float* const* layer_params, cudaStream_t s, float** arena_out, cudaEvent_t* order_event){
    if(!layer_params) return B200RL_ERR_INVALID_ARGUMENT;
    for(int i = 0; i < 6; i++) if(!layer_params[i]) return B200RL_ERR_INVALID_ARGUMENT;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200RL_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
    if(cap != cudaStreamCaptureStatusNone) return B200RL_ERR_UNSUPPORTED;
    static struct { cudaEvent_t order; float* arena; } per_device[MAX_DEVICES] = {};
    static std::mutex mutex;
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    std::lock_guard<std::mutex> lock(mutex);
    auto& st = per_device[dev];
    if(!st.order) B200RL_CUDA_TRY(cudaEventCreateWithFlags(&st.order, cudaEventDisableTiming));
    if(!st.arena) B200RL_CUDA_TRY(cudaGetSymbolAddress((void**)&st.arena, g_collect_actor_arena));
    B200RL_CUDA_TRY(cudaStreamWaitEvent(s, st.order, 0));
    const size_t counts[6] = {64 * 3, 64, 64 * 64, 64, 64, 1};
    size_t off = 0;
    for(int i = 0; i < 6; i++){
        B200RL_CUDA_TRY(cudaMemcpyAsync(st.arena + off, layer_params[i], sizeof(float) * counts[i], cudaMemcpyDeviceToDevice, s));
        off += counts[i];
    }
    *arena_out = st.arena; *order_event = st.order;
    return B200RL_OK;
}

extern "C" int b200rl_pendulum_collect_layers(const b200rl_mlp_shape* actor, const float* const* layer_params, const float* log_std,
                                              float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                                              const float* reset_states, int n_reset_rounds, const float* noise, int n_envs, int n_steps,
                                              int step_limit, float* dataset, int ld_dataset, int* error_flag, b200rl_stream_t stream){
    int rc = validate_actor(actor);
    if(rc) return rc;
    cudaStream_t s = (cudaStream_t)stream;
    float* arena = nullptr; cudaEvent_t ev = nullptr;
    rc = pack_actor_layers(layer_params, s, &arena, &ev);
    if(rc) return rc;
    rc = collect_launch(actor, arena, log_std, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds, noise,
                        n_envs, n_steps, step_limit, dataset, ld_dataset, error_flag, s);
    B200RL_CUDA_TRY(cudaEventRecord(ev, s));
    return rc;
}

// ---------------------------------------------------------------------------------------------------------------
// Off-policy runner step with per-environment replay buffers (rl/components/off_policy_runner/operations_generic.h:219-238):
// one fused rollout step into the runner's step buffers, then one thread per environment appends the transition to that environment's
// replay buffer with the reference's bookkeeping (operations_generic_per_env.h:41-52, replay_buffer/operations_generic.h:54-79).
// ---------------------------------------------------------------------------------------------------------------
namespace b200rl {
// appends one transition of environment e to its replay buffer; (next_theta, next_theta_dot) is the state after the step
template <typename INDEX>
__device__ __forceinline__ void replay_append(int e, float next_theta, float next_theta_dot, bool trunc, bool was_truncated, const float* __restrict__ observations,
                                              float action, float reward, float* __restrict__ next_observations, unsigned char* replay, const b200rl_replay_layout& L){
    unsigned char* rb = replay + (size_t)e * L.env_stride;
    float* data = reinterpret_cast<float*>(rb + L.off_data);
    INDEX* episode_start = reinterpret_cast<INDEX*>(rb + L.off_episode_start);
    INDEX& position_ref = *reinterpret_cast<INDEX*>(rb + L.off_position);
    INDEX& ces_ref = *reinterpret_cast<INDEX*>(rb + L.off_current_episode_start);
    unsigned char& full_ref = *(rb + L.off_full);
    INDEX position = position_ref, ces = ces_ref;
    bool full = full_ref != 0;
    if(was_truncated && (full || position > 0)){               // prologue: the environment was reset at the start of this step
        const INDEX prev = position == 0 ? (INDEX)(L.capacity - 1) : position - 1;
        data[(size_t)prev * L.ld_data + 9] = 1.0f;
        ces = position;
    }
    float sn, cs;
    sincosf(next_theta, &sn, &cs);
    next_observations[3 * e] = cs; next_observations[3 * e + 1] = sn; next_observations[3 * e + 2] = next_theta_dot;
    float* row = data + (size_t)position * L.ld_data;
    row[0] = observations[3 * e]; row[1] = observations[3 * e + 1]; row[2] = observations[3 * e + 2];
    row[3] = action; row[4] = reward;
    row[5] = cs; row[6] = sn; row[7] = next_theta_dot;
    row[8] = 0.0f; row[9] = trunc ? 1.0f : 0.0f;              // Pendulum never terminates
    episode_start[position] = ces;
    position = (position + 1) % (INDEX)L.capacity;
    if(trunc) ces = position;
    if(position == 0 && !full) full = true;
    position_ref = position; ces_ref = ces; full_ref = full ? 1 : 0;
}

template <typename INDEX>
__global__ void replay_add_kernel(int n_envs, const float* __restrict__ states, const uint8_t* __restrict__ truncated, const uint8_t* __restrict__ was_truncated,
                                  const float* __restrict__ observations, const float* __restrict__ actions, const float* __restrict__ rewards,
                                  float* __restrict__ next_observations, unsigned char* replay, b200rl_replay_layout L){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n_envs) return;
    replay_append<INDEX>(e, states[2 * e], states[2 * e + 1], truncated[e] != 0, was_truncated[e] != 0, observations, actions[e], rewards[e], next_observations, replay, L);
}

// The runner step in two halves around ANY policy (how the reference's CUDA runner is built: prologue kernel, evaluate(policy), epilogue
// kernel; rl/components/off_policy_runner/operations_cuda.h:184-204 around operations_generic_per_env.h:8-61 and :62-108).
// Prologue: reset-if-truncated (from the table, or drawn in the kernel), counters of a fresh episode, observation.
__global__ void offpolicy_prologue_kernel(int n_envs, float* __restrict__ states, int32_t* __restrict__ episode_step, const uint8_t* __restrict__ truncated,
                                          float* __restrict__ episode_return, const float* __restrict__ reset_states, unsigned long long seed, unsigned long long call,
                                          const unsigned long long* __restrict__ call_counter, float* __restrict__ observations, uint8_t* __restrict__ was_truncated){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n_envs) return;
    float theta = states[2 * e], theta_dot = states[2 * e + 1];
    const bool trunc = truncated[e] != 0;
    was_truncated[e] = trunc ? 1 : 0;
    if(trunc){
        if(reset_states){ theta = __ldg(reset_states + 2 * e); theta_dot = __ldg(reset_states + 2 * e + 1); }
        else{           // theta ~ U(-pi, pi), theta_dot ~ U(-1, 1) (rl/environments/pendulum/operations_generic.h:57-61), one Philox block per (environment, call)
            const StepDraws d = step_draws(seed, call + (call_counter ? *call_counter : 0ull), (uint32_t)e);
            theta = fmaf(d.u_theta, 2.0f * pendulum::PI_F, -pendulum::PI_F); theta_dot = fmaf(d.u_theta_dot, 2.0f, -1.0f);
        }
        states[2 * e] = theta; states[2 * e + 1] = theta_dot;
        episode_step[e] = 0; episode_return[e] = 0.0f;
    }
    float sn, cs;
    sincosf(theta, &sn, &cs);
    observations[3 * e] = cs; observations[3 * e + 1] = sn; observations[3 * e + 2] = theta_dot;
}
// Epilogue: environment step with the given actions, reward, counters, truncation, next observation, replay-buffer append.
template <typename INDEX>
__global__ void offpolicy_epilogue_kernel(int n_envs, int step_limit, float* __restrict__ states, int32_t* __restrict__ episode_step, uint8_t* __restrict__ truncated,
                                          float* __restrict__ episode_return, const float* __restrict__ observations, const float* __restrict__ actions,
                                          float* __restrict__ next_observations, const uint8_t* __restrict__ was_truncated, unsigned char* replay, b200rl_replay_layout L){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n_envs) return;
    const float theta = states[2 * e], theta_dot = states[2 * e + 1], action = actions[e];
    float nt, ntd;
    pendulum::step(theta, theta_dot, observations[3 * e + 1], action, nt, ntd);          // the observation's second component is sin(theta)
    const float rwd = pendulum::reward(theta, theta_dot, action);
    const int es = episode_step[e] + 1;
    const bool trunc = es == step_limit;
    states[2 * e] = nt; states[2 * e + 1] = ntd;
    episode_step[e] = es; episode_return[e] = __fadd_rn(episode_return[e], rwd); truncated[e] = trunc ? 1 : 0;
    replay_append<INDEX>(e, nt, ntd, trunc, was_truncated[e] != 0, observations, action, rwd, next_observations, replay, L);
}
}  // namespace b200rl

extern "C" int b200rl_pendulum_offpolicy_step(const b200rl_mlp_shape* actor, const float* actor_params, const float* const* layer_params, float* states,
                                              int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int n_envs,
                                              int step_limit, float* observations, float* actions, float* next_observations, void* replay_buffers,
                                              const b200rl_replay_layout* layout, float* reward_scratch, uint8_t* was_truncated_scratch, int* error_flag,
                                              b200rl_stream_t stream){
    int rc = validate_actor(actor);
    if(rc) return rc;
    if((!actor_params && !layer_params) || !states || !episode_step || !truncated || !episode_return || !observations || !actions || !next_observations ||
       !replay_buffers || !layout || !reward_scratch || !was_truncated_scratch || n_envs < 0 || step_limit < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(layout->capacity < 1 || layout->ld_data < 10 || (layout->index_bytes != 4 && layout->index_bytes != 8)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    cudaEvent_t ev = nullptr;
    if(!actor_params){
        float* arena = nullptr;
        rc = pack_actor_layers(layer_params, s, &arena, &ev);
        if(rc) return rc;
        actor_params = arena;
    }
    B200RL_CUDA_TRY(cudaMemcpyAsync(was_truncated_scratch, truncated, (size_t)n_envs, cudaMemcpyDeviceToDevice, s));
    RolloutArgs a{};
    a.params = actor_params; a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return;
    a.reset_states = reset_states; a.n_reset_rounds = reset_states ? 1 : 0; a.n_envs = n_envs; a.env_begin = 0; a.env_count = n_envs;
    a.n_steps = 1; a.step_limit = step_limit; a.obs = observations; a.act = actions; a.rew = reward_scratch; a.error_flag = error_flag;
    for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
    rc = rollout_dispatch(actor, a, s);
    if(ev) B200RL_CUDA_TRY(cudaEventRecord(ev, s));
    if(rc) return rc;
    const int threads = 128, blocks = (n_envs + threads - 1) / threads;
    if(layout->index_bytes == 4)
        replay_add_kernel<uint32_t><<<blocks, threads, 0, s>>>(n_envs, states, truncated, was_truncated_scratch, observations, actions, reward_scratch,
                                                              next_observations, static_cast<unsigned char*>(replay_buffers), *layout);
    else
        replay_add_kernel<unsigned long long><<<blocks, threads, 0, s>>>(n_envs, states, truncated, was_truncated_scratch, observations, actions, reward_scratch,
                                                                        next_observations, static_cast<unsigned char*>(replay_buffers), *layout);
    B200RL_LAUNCH_CHECK("replay_add");
    return B200RL_OK;
}

extern "C" int b200rl_pendulum_offpolicy_prologue(float* states, int32_t* episode_step, const uint8_t* truncated, float* episode_return, const float* reset_states,
                                                  unsigned long long seed, unsigned long long call, const unsigned long long* call_counter, int n_envs,
                                                  float* observations, uint8_t* was_truncated_scratch, b200rl_stream_t stream){
    if(!states || !episode_step || !truncated || !episode_return || !observations || !was_truncated_scratch || n_envs < 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    const int threads = 128, blocks = (n_envs + threads - 1) / threads;
    offpolicy_prologue_kernel<<<blocks, threads, 0, (cudaStream_t)stream>>>(n_envs, states, episode_step, truncated, episode_return, reset_states, seed, call, call_counter,
                                                                           observations, was_truncated_scratch);
    B200RL_LAUNCH_CHECK("offpolicy_prologue");
    return B200RL_OK;
}

extern "C" int b200rl_pendulum_offpolicy_epilogue(float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return, int n_envs, int step_limit,
                                                  const float* observations, const float* actions, float* next_observations, void* replay_buffers,
                                                  const b200rl_replay_layout* layout, const uint8_t* was_truncated_scratch, b200rl_stream_t stream){
    if(!states || !episode_step || !truncated || !episode_return || !observations || !actions || !next_observations || !replay_buffers || !layout ||
       !was_truncated_scratch || n_envs < 0 || step_limit < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(layout->capacity < 1 || layout->ld_data < 10 || (layout->index_bytes != 4 && layout->index_bytes != 8)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    const int threads = 128, blocks = (n_envs + threads - 1) / threads;
    cudaStream_t s = (cudaStream_t)stream;
    if(layout->index_bytes == 4)
        offpolicy_epilogue_kernel<uint32_t><<<blocks, threads, 0, s>>>(n_envs, step_limit, states, episode_step, truncated, episode_return, observations, actions,
                                                                      next_observations, was_truncated_scratch, static_cast<unsigned char*>(replay_buffers), *layout);
    else
        offpolicy_epilogue_kernel<unsigned long long><<<blocks, threads, 0, s>>>(n_envs, step_limit, states, episode_step, truncated, episode_return, observations, actions,
                                                                                next_observations, was_truncated_scratch, static_cast<unsigned char*>(replay_buffers), *layout);
    B200RL_LAUNCH_CHECK("offpolicy_epilogue");
    return B200RL_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// Replay-buffer sampling: gather_batch with sequence length 1 (rl/components/off_policy_runner/operations_generic.h:239-423). The two
// random indices of every batch element are drawn on the host (b200rl_gather_draws_host) in the reference's order; the kernel applies
// the reference's index arithmetic and writes the batch tensors.
// ---------------------------------------------------------------------------------------------------------------
namespace b200rl {
template <typename INDEX>
__global__ void replay_counters_kernel(int n_envs, const unsigned char* __restrict__ replay, b200rl_replay_layout L, int32_t* __restrict__ position,
                                       uint8_t* __restrict__ full){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n_envs) return;
    const unsigned char* rb = replay + (size_t)e * L.env_stride;
    position[e] = (int32_t)*reinterpret_cast<const INDEX*>(rb + L.off_position);
    full[e] = *(rb + L.off_full) != 0;
}

struct GatherArgs {
    const unsigned char* replay; b200rl_replay_layout L;
    int n_envs, max_episode_length, batch, obs_dim, action_dim;
    const int32_t *env_index, *sample_offset;
    float* oa_base; int ld_oa;
    float* rewards; uint8_t *terminated, *reset, *next_reset_base, *final_step_mask, *next_final_step_mask_base;
    int* error_flag;
    int device_rng; unsigned long long seed, call;      // device draws: Philox block (batch element, call low, call high, 1) keyed by seed
    const unsigned long long* call_counter;             // optional device-resident call index added to `call` (advanced by a later launch)
};
// one warp per batch element: lanes stride over the columns of the transition row
template <typename INDEX>
__global__ void gather_batch_kernel(GatherArgs a){
    const int b = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if(b >= a.batch) return;
    int e, offset = 0;
    uint32_t word1 = 0;
    if(a.device_rng){         // bounded draws by the high half of word * range (bias below range / 2^32)
        const unsigned long long call = a.call + (a.call_counter ? *a.call_counter : 0ull);
        uint32_t c[4] = {(uint32_t)b, (uint32_t)call, (uint32_t)(call >> 32), 1u};
        Philox::block(c, (uint32_t)a.seed, (uint32_t)(a.seed >> 32));
        e = (int)__umulhi(c[0], (uint32_t)a.n_envs);
        word1 = c[1];
    }
    else{ e = a.env_index[b]; offset = a.sample_offset[b]; }
    bool ok = e >= 0 && e < a.n_envs && offset >= 0;
    long long index = 0;
    const unsigned char* rb = a.replay + (size_t)(ok ? e : 0) * a.L.env_stride;
    if(ok){
        const long long position = (long long)*reinterpret_cast<const INDEX*>(rb + a.L.off_position);
        const bool full = *(rb + a.L.off_full) != 0;
        if(a.device_rng) offset = (int)__umulhi(word1, (uint32_t)(full ? (long long)a.L.capacity : position));
        ok = offset < (full ? (long long)a.L.capacity : position);                                       // :257
        index = full ? (position + a.max_episode_length + offset) % a.L.capacity : (long long)offset;     // :303-311
    }
    if(!ok){
        if(lane == 0 && a.error_flag) *a.error_flag = 2;
        return;
    }
    const float* row = reinterpret_cast<const float*>(rb + a.L.off_data) + (size_t)index * a.L.ld_data;
    const int O = a.obs_dim, A = a.action_dim;
    float* step0 = a.oa_base + (size_t)b * a.ld_oa;
    float* step1 = a.oa_base + ((size_t)a.batch + b) * a.ld_oa;
    for(int c = lane; c < O + A; c += 32) step0[c] = row[c];                                  // observation, action (:318-341)
    for(int c = lane; c < O; c += 32) step1[c] = row[O + A + 1 + c];                          // next observation (:385-390)
    for(int c = lane; c < A; c += 32) step1[O + c] = 0.0f;                                    // :400-402
    if(lane == 0){
        a.rewards[b] = row[O + A];
        a.terminated[b] = row[2 * O + A + 1] != 0.0f;
        a.reset[b] = 1; a.final_step_mask[b] = 1;                                             // :279-281, :296-299, :352, :381-383
        a.next_reset_base[b] = 1; a.next_reset_base[a.batch + b] = 1;                         // :285-286
        a.next_final_step_mask_base[b] = 0; a.next_final_step_mask_base[a.batch + b] = 1;     // :291
    }
}
}  // namespace b200rl

// ---------------------------------------------------------------------------------------------------------------
// Replay-buffer sampling for any sequence length (rl/components/off_policy_runner/operations_generic.h:239-423): one thread per batch
// element walks the padded sequence through its environment's replay buffer exactly as gather_batch_step does -- a new start index
// whenever the previous step was padding, the episode's first step if sequences start from the initial state, a cut at a truncated
// transition, at the newest transition, at the second to last padded step or at a random length -- and writes the batch tensors
// [step, batch, ...]. Draws (environment, sample offsets, sequence lengths) come from a counter-based stream per (batch element, call);
// with B200RL_GATHER_DETERMINISTIC the environment is 0 and the offset the element's index, as with the reference's DETERMINISTIC flag.
// ---------------------------------------------------------------------------------------------------------------
namespace b200rl {
struct GatherSeqArgs {
    const unsigned char* replay; b200rl_replay_layout L;
    int n_envs, max_episode_length, batch, obs_dim, action_dim, seq, flags;
    float nominal_probability;
    float* oa_base; int ld_oa;
    float* rewards; uint8_t *terminated, *reset, *next_reset_base, *final_step_mask, *next_final_step_mask_base;
    int* error_flag;
    unsigned long long seed, call; const unsigned long long* call_counter;
};
// successive 32-bit draws of one (batch element, call): Philox blocks (element, call low, call high, 2 + block index)
struct DrawStream {
    uint32_t c[4]; uint32_t element, call_lo, call_hi, k0, k1; int block, used;
    __device__ void init(unsigned long long seed, unsigned long long call, uint32_t e){ element = e; call_lo = (uint32_t)call; call_hi = (uint32_t)(call >> 32); k0 = (uint32_t)seed; k1 = (uint32_t)(seed >> 32); block = 0; used = 4; }
    __device__ uint32_t next(){
        if(used == 4){ c[0] = element; c[1] = call_lo; c[2] = call_hi; c[3] = 2u + (uint32_t)block; Philox::block(c, k0, k1); block++; used = 0; }
        return c[used++];
    }
    __device__ long long below(long long n){ return (long long)__umulhi(next(), (uint32_t)n); }            // U{0 .. n-1}, bias below n / 2^32
    __device__ float unit(){ return (float)(next() >> 8) * 5.9604644775390625e-8f; }                        // [0, 1) in steps of 2^-24
};
template <typename INDEX>
__global__ void __launch_bounds__(128) gather_sequences_kernel(GatherSeqArgs a){
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if(b >= a.batch) return;
    const bool from_initial = a.flags & B200RL_GATHER_FROM_INITIAL_STATE, random_length = a.flags & B200RL_GATHER_RANDOM_LENGTH, deterministic = a.flags & B200RL_GATHER_DETERMINISTIC;
    const int next_offset = (a.flags & B200RL_GATHER_FIRST_STEP_TARGET) ? 0 : 1;
    const int Lq = a.seq, P = Lq + 1, O = a.obs_dim, A = a.action_dim;
    const size_t B = (size_t)a.batch;
    DrawStream draws; draws.init(a.seed, a.call + (a.call_counter ? *a.call_counter : 0ull), (uint32_t)b);
    const int e = deterministic ? 0 : (int)draws.below(a.n_envs);
    const unsigned char* rb = a.replay + (size_t)e * a.L.env_stride;
    const float* data = reinterpret_cast<const float*>(rb + a.L.off_data);
    const INDEX* episode_start = reinterpret_cast<const INDEX*>(rb + a.L.off_episode_start);
    const long long position = (long long)*reinterpret_cast<const INDEX*>(rb + a.L.off_position), capacity = a.L.capacity;
    const bool full = *(rb + a.L.off_full) != 0;
    const long long eligible = full ? (from_initial ? capacity - a.max_episode_length : capacity) : position;      // :258
    if(eligible < 1 || (deterministic && b >= eligible)){ if(a.error_flag) *a.error_flag = 2; return; }             // the reference requires a non-empty range (:251-255)
    auto draw_length = [&]() -> long long {                                                                       // :263-272
        if(draws.unit() < a.nominal_probability) return Lq;
        return Lq > 1 ? 1 + draws.below(Lq - 1) : Lq;
    };
    long long index = 0, length = Lq, seq_step = 0;
    if(random_length) length = draw_length();
    bool previous_truncated = false, previous_padding = true;
    for(int q = 0; q < Lq; q++){ a.final_step_mask[q * B + b] = 0; a.reset[q * B + b] = 0; }
    for(int q = 0; q < P; q++){ a.next_final_step_mask_base[q * B + b] = 0; a.next_reset_base[q * B + b] = 0; }
    a.reset[b] = 1; a.next_reset_base[b] = 1; a.next_reset_base[next_offset * B + b] = 1;                           // :284-286
    for(int q = 0; q < P; q++){
        if(previous_truncated){                                                                                    // :288-297
            previous_truncated = false; previous_padding = true;
            a.next_final_step_mask_base[q * B + b] = 1;
            if(q < P - 1) a.reset[q * B + b] = 1;
            continue;
        }
        if(previous_padding){                                                                                      // :298-317
            if(q < P - 1) a.reset[q * B + b] = 1;
            a.next_reset_base[q * B + b] = 1;
            const long long offset = deterministic ? b : draws.below(eligible);
            index = full ? (position + a.max_episode_length + offset) % capacity : offset;
            if(from_initial) index = (long long)episode_start[index];
        }
        const float* row = data + (size_t)index * a.L.ld_data;
        float* step = a.oa_base + (q * B + b) * a.ld_oa;
        for(int c = 0; c < O + A; c++) step[c] = row[c];                                                            // observation, action
        if(q < P - 1){ a.rewards[q * B + b] = row[O + A]; a.terminated[q * B + b] = row[2 * O + A + 1] != 0.0f; }
        bool truncated = row[2 * O + A + 2] != 0.0f;
        long long next_index = index + 1;
        if(full) next_index %= capacity;
        if(next_index == position) truncated = true;                                                               // the newest transition
        if(q == P - 2) truncated = true;
        if(random_length){                                                                                         // :361-381
            if(seq_step == length - 1){
                truncated = true;
                length = Lq > 1 ? draw_length() : Lq;
            }
            seq_step = truncated ? 0 : seq_step + 1;
        }
        if(truncated && q < P - 1){                                                                                // :386-403
            a.final_step_mask[q * B + b] = 1;
            float* next = a.oa_base + ((q + 1) * B + b) * a.ld_oa;
            for(int c = 0; c < O; c++) next[c] = row[O + A + 1 + c];
            for(int c = 0; c < A; c++) next[O + c] = 0.0f;
        }
        index = next_index;
        previous_padding = false;
        previous_truncated = truncated;
    }
}
}  // namespace b200rl

extern "C" int b200rl_gather_batch_sequences(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim, int action_dim,
                                             int sequence_length, int flags, float nominal_probability, unsigned long long seed, unsigned long long call_index,
                                             const unsigned long long* call_counter, int batch, float* oa_base, int ld_oa, float* rewards, uint8_t* terminated, uint8_t* reset,
                                             uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream){
    if(!replay_buffers || !layout || !oa_base || !rewards || !terminated || !reset || !next_reset_base || !final_step_mask || !next_final_step_mask_base || n_envs < 1 ||
       batch < 0 || obs_dim < 1 || action_dim < 1 || sequence_length < 1 || max_episode_length < 0 || ld_oa < obs_dim + action_dim)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(layout->capacity < 1 || layout->ld_data < 2 * obs_dim + action_dim + 3 || (layout->index_bytes != 4 && layout->index_bytes != 8)) return B200RL_ERR_INVALID_ARGUMENT;
    if((flags & B200RL_GATHER_FROM_INITIAL_STATE) && layout->capacity < max_episode_length) return B200RL_ERR_INVALID_ARGUMENT;     // the reference's static_assert (:256)
    if(batch == 0) return B200RL_OK;
    GatherSeqArgs a{};
    a.replay = static_cast<const unsigned char*>(replay_buffers); a.L = *layout; a.n_envs = n_envs; a.max_episode_length = max_episode_length; a.batch = batch;
    a.obs_dim = obs_dim; a.action_dim = action_dim; a.seq = sequence_length; a.flags = flags; a.nominal_probability = nominal_probability;
    a.oa_base = oa_base; a.ld_oa = ld_oa; a.rewards = rewards; a.terminated = terminated; a.reset = reset; a.next_reset_base = next_reset_base;
    a.final_step_mask = final_step_mask; a.next_final_step_mask_base = next_final_step_mask_base; a.error_flag = error_flag;
    a.seed = seed; a.call = call_index; a.call_counter = call_counter;
    const int threads = 128, blocks = (batch + threads - 1) / threads;
    if(layout->index_bytes == 4) gather_sequences_kernel<uint32_t><<<blocks, threads, 0, (cudaStream_t)stream>>>(a);
    else gather_sequences_kernel<unsigned long long><<<blocks, threads, 0, (cudaStream_t)stream>>>(a);
    B200RL_LAUNCH_CHECK("gather_sequences");
    return B200RL_OK;
}

extern "C" int b200rl_replay_counters(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int32_t* position, uint8_t* full,
                                      b200rl_stream_t stream){
    if(!replay_buffers || !layout || !position || !full || n_envs < 0 || (layout->index_bytes != 4 && layout->index_bytes != 8)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    const int threads = 128, blocks = (n_envs + threads - 1) / threads;
    cudaStream_t s = (cudaStream_t)stream;
    if(layout->index_bytes == 4) replay_counters_kernel<uint32_t><<<blocks, threads, 0, s>>>(n_envs, static_cast<const unsigned char*>(replay_buffers), *layout, position, full);
    else replay_counters_kernel<unsigned long long><<<blocks, threads, 0, s>>>(n_envs, static_cast<const unsigned char*>(replay_buffers), *layout, position, full);
    B200RL_LAUNCH_CHECK("replay_counters");
    return B200RL_OK;
}

static int gather_launch(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim,
                         int action_dim, const int32_t* env_index, const int32_t* sample_offset, int batch, float* oa_base, int ld_oa,
                         float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                         uint8_t* next_final_step_mask_base, int* error_flag, DeviceRng rng, b200rl_stream_t stream,
                         const unsigned long long* call_counter = nullptr){
    if(!replay_buffers || !layout || (!rng.enabled && (!env_index || !sample_offset)) || !oa_base || !rewards || !terminated || !reset || !next_reset_base || !final_step_mask ||
       !next_final_step_mask_base || n_envs < 1 || batch < 0 || obs_dim < 1 || action_dim < 1 || max_episode_length < 0)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(layout->capacity < 1 || layout->ld_data < 2 * obs_dim + action_dim + 3 || ld_oa < obs_dim + action_dim || (layout->index_bytes != 4 && layout->index_bytes != 8))
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    GatherArgs a{};
    a.replay = static_cast<const unsigned char*>(replay_buffers); a.L = *layout; a.n_envs = n_envs; a.max_episode_length = max_episode_length; a.batch = batch;
    a.obs_dim = obs_dim; a.action_dim = action_dim; a.env_index = env_index; a.sample_offset = sample_offset; a.oa_base = oa_base; a.ld_oa = ld_oa;
    a.rewards = rewards; a.terminated = terminated; a.reset = reset; a.next_reset_base = next_reset_base; a.final_step_mask = final_step_mask;
    a.next_final_step_mask_base = next_final_step_mask_base; a.error_flag = error_flag;
    a.device_rng = rng.enabled; a.seed = rng.seed; a.call = rng.step0; a.call_counter = call_counter;
    const int threads = 128, blocks = (int)(((size_t)batch * 32 + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    if(layout->index_bytes == 4) gather_batch_kernel<uint32_t><<<blocks, threads, 0, s>>>(a);
    else gather_batch_kernel<unsigned long long><<<blocks, threads, 0, s>>>(a);
    B200RL_LAUNCH_CHECK("gather_batch");
    return B200RL_OK;
}

extern "C" int b200rl_gather_batch(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim,
                                   int action_dim, const int32_t* env_index, const int32_t* sample_offset, int batch, float* oa_base, int ld_oa,
                                   float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                                   uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream){
    return gather_launch(replay_buffers, layout, n_envs, max_episode_length, obs_dim, action_dim, env_index, sample_offset, batch, oa_base, ld_oa, rewards,
                         terminated, reset, next_reset_base, final_step_mask, next_final_step_mask_base, error_flag, DeviceRng{0, 0, 0}, stream);
}

extern "C" int b200rl_gather_batch_device_rng(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim,
                                              int action_dim, unsigned long long seed, unsigned long long call_index, int batch, float* oa_base, int ld_oa,
                                              float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                                              uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream){
    return gather_launch(replay_buffers, layout, n_envs, max_episode_length, obs_dim, action_dim, nullptr, nullptr, batch, oa_base, ld_oa, rewards,
                         terminated, reset, next_reset_base, final_step_mask, next_final_step_mask_base, error_flag, DeviceRng{1, seed, call_index}, stream);
}

// ---------------------------------------------------------------------------------------------------------------
// Randomness that lives entirely on the device, for update loops captured in a CUDA graph: a device-resident 64-bit call counter
// feeds the Philox counters of the sampling kernel above and of the normal generator below, and is advanced by its own launch, so that
// every replay of the same graph draws fresh numbers.
// ---------------------------------------------------------------------------------------------------------------
namespace b200rl {
__global__ void counter_advance_kernel(unsigned long long* counter, unsigned long long increment){ *counter += increment; }

// four standard normals per Philox block: counter (element / 4, call low, call high, 2 + stream_id), Box-Muller on word pairs
__global__ void randn_kernel(float* __restrict__ dst, size_t n, unsigned long long seed, uint32_t stream_id, unsigned long long call,
                             const unsigned long long* __restrict__ call_counter){
    const size_t q = blockIdx.x * (size_t)blockDim.x + threadIdx.x;
    if(q * 4 >= n) return;
    call += call_counter ? *call_counter : 0ull;
    uint32_t c[4] = {(uint32_t)q, (uint32_t)call, (uint32_t)(call >> 32), 2u + stream_id};
    Philox::block(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    float out[4];
#pragma unroll
    for(int h = 0; h < 2; h++){
        const float radius = sqrtf(-2.0f * logf(unit_uniform(c[2 * h])));
        float sn, cs;
        sincospif(2.0f * unit_uniform(c[2 * h + 1]), &sn, &cs);
        out[2 * h] = radius * cs; out[2 * h + 1] = radius * sn;
    }
    for(int i = 0; i < 4 && q * 4 + i < n; i++) dst[q * 4 + i] = out[i];
}
}  // namespace b200rl

extern "C" int b200rl_counter_advance(unsigned long long* counter, unsigned long long increment, b200rl_stream_t stream){
    if(!counter) return B200RL_ERR_INVALID_ARGUMENT;
    counter_advance_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(counter, increment);
    B200RL_LAUNCH_CHECK("counter_advance");
    return B200RL_OK;
}

extern "C" int b200rl_randn_device_rng(float* dst, size_t n, unsigned long long seed, unsigned int stream_id, unsigned long long call_index,
                                       const unsigned long long* call_counter, b200rl_stream_t stream){
    if(!dst || n > ((size_t)1 << 33)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    const size_t quads = (n + 3) / 4;
    randn_kernel<<<(unsigned)((quads + 127) / 128), 128, 0, (cudaStream_t)stream>>>(dst, n, seed, stream_id, call_index, call_counter);
    B200RL_LAUNCH_CHECK("randn_device_rng");
    return B200RL_OK;
}

extern "C" int b200rl_gather_batch_device_counter(const void* replay_buffers, const b200rl_replay_layout* layout, int n_envs, int max_episode_length, int obs_dim,
                                                  int action_dim, unsigned long long seed, const unsigned long long* call_counter, int batch, float* oa_base,
                                                  int ld_oa, float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                                                  uint8_t* next_final_step_mask_base, int* error_flag, b200rl_stream_t stream){
    if(!call_counter) return B200RL_ERR_INVALID_ARGUMENT;
    return gather_launch(replay_buffers, layout, n_envs, max_episode_length, obs_dim, action_dim, nullptr, nullptr, batch, oa_base, ld_oa, rewards,
                         terminated, reset, next_reset_base, final_step_mask, next_final_step_mask_base, error_flag, DeviceRng{1, seed, 0}, stream, call_counter);
}
