// Fused rollout for environments given as device-function policies: reset-if-truncated, observe, actor forward
// (OBS_DIM -> H -> H -> 1, H one of 16 / 32 / 64 / 128), environment step, reward and episode counters for T steps in ONE launch, one thread per
// environment, the runner state in registers between steps, the actor's weights in shared memory (read as warp broadcasts).
// This CUDA-core kernel serves the hidden widths other than 64; width 64 runs on the tensor-core kernel (rollout_tc.cu), which takes the
// same environment policies (envs.cuh).
#include "common.cuh"
#include "envs.cuh"
#include "rollout.cuh"

namespace b200rl {

struct EnvRolloutArgs {
    const float* params;        // actor arena: W1[H,OBS] b1[H] W2[H,H] b2[H] W3[1,H] b3[1]
    float* states;              // [n_envs, STATE_DIM]
    int32_t* episode_step; uint8_t* truncated; float* episode_return;
    const float* reset_states;  // [n_reset_rounds, n_envs, RESET_DIM]
    uint8_t* terminated;        // [n_steps * n_envs] or NULL
    int n_reset_rounds, n_envs, n_steps, step_limit;
    float* obs; float* act; float* rew;         // [n_steps * n_envs, OBS_DIM | 1 | 1], row = step * n_envs + env
    int* error_flag;
    int acts[3];
};

template <typename ENV, int H>
__global__ void __launch_bounds__(128, H <= 64 ? 4 : 2) rollout_env_kernel(EnvRolloutArgs a){
    constexpr int S = ENV::STATE_DIM, O = ENV::OBS_DIM;
    extern __shared__ __align__(16) float smem[];
    float* W1 = smem;                 // [H][O]
    float* b1 = W1 + H * O;
    float* W2 = b1 + H;               // [H][H]
    float* b2 = W2 + H * H;
    float* W3 = b2 + H;
    float* b3 = W3 + H;
    constexpr int NPARAMS = H * O + H + H * H + H + H + 1;
    for(int i = threadIdx.x; i < NPARAMS; i += blockDim.x) smem[i] = __ldg(a.params + i);
    __syncthreads();
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= a.n_envs) return;
    float state[S];
#pragma unroll
    for(int k = 0; k < S; k++) state[k] = a.states[(size_t)e * S + k];
    int es = a.episode_step[e];
    bool trunc = a.truncated[e] != 0;
    float er = a.episode_return[e];
    int resets = 0;
    for(int t = 0; t < a.n_steps; t++){
        if(trunc){                                   // prologue: rl/components/off_policy_runner/operations_generic_per_env.h:8-61
            if(a.reset_states != nullptr && resets < a.n_reset_rounds){
                const float* rsp = a.reset_states + ((size_t)resets * a.n_envs + e) * ENV::RESET_DIM;      // scalar loads: the table may be a view at any 4-byte offset
                float draws[ENV::RESET_DIM];
#pragma unroll
                for(int k = 0; k < ENV::RESET_DIM; k++) draws[k] = __ldg(rsp + k);
                ENV::reset(state, draws);
            }
            else if(a.error_flag) *a.error_flag = 1;
            resets++; es = 0; er = 0.0f;
        }
        float o[O];
        ENV::observe(state, o);
        const size_t row = (size_t)t * a.n_envs + e;
#pragma unroll
        for(int k = 0; k < O; k++) a.obs[row * O + k] = o[k];
        float h1[H];                                 // exact fp32 FMA chain in the reference's summation order (bias first, inputs ascending)
#pragma unroll
        for(int j = 0; j < H; j++){
            float acc = b1[j];
#pragma unroll
            for(int k = 0; k < O; k++) acc = fmaf(W1[j * O + k], o[k], acc);
            h1[j] = activation_rt(acc, a.acts[0]);
        }
        float out = b3[0];
#pragma unroll 2
        for(int j = 0; j < H; j++){
            float acc = b2[j];
            const float4* w = reinterpret_cast<const float4*>(W2 + j * H);
#pragma unroll
            for(int k = 0; k < H / 4; k++){
                const float4 w4 = w[k];
                acc = fmaf(w4.x, h1[4 * k + 0], acc); acc = fmaf(w4.y, h1[4 * k + 1], acc);
                acc = fmaf(w4.z, h1[4 * k + 2], acc); acc = fmaf(w4.w, h1[4 * k + 3], acc);
            }
            out = fmaf(W3[j], activation_rt(acc, a.acts[1]), out);
        }
        const float action = activation_rt(out, a.acts[2]);
        float next[S];
        const float r = ENV::transition(state, action, next);        // epilogue: operations_generic_per_env.h:62-108
        es += 1; er = __fadd_rn(er, r);
        const bool term = ENV::TERMINATES && ENV::terminated(next);
        trunc = term || (es == a.step_limit);                        // operations_generic_per_env.h:93-97
        a.act[row] = action; a.rew[row] = r;
        if(a.terminated) a.terminated[row] = term ? 1 : 0;
#pragma unroll
        for(int k = 0; k < S; k++) state[k] = next[k];
    }
#pragma unroll
    for(int k = 0; k < S; k++) a.states[(size_t)e * S + k] = state[k];
    a.episode_step[e] = es; a.truncated[e] = trunc ? 1 : 0; a.episode_return[e] = er;
}

template <typename ENV, int H>
static int launch_env_width(const EnvRolloutArgs& a, cudaStream_t s){
    constexpr int THREADS = 128;
    constexpr size_t SMEM = sizeof(float) * (H * ENV::OBS_DIM + H + H * H + H + H + 1);
    if(SMEM > 48 * 1024) B200RL_CUDA_TRY(cudaFuncSetAttribute(rollout_env_kernel<ENV, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    rollout_env_kernel<ENV, H><<<(a.n_envs + THREADS - 1) / THREADS, THREADS, SMEM, s>>>(a);
    B200RL_LAUNCH_CHECK("rollout_env");
    return B200RL_OK;
}

// the hidden width is a template parameter (the first layer's activations live in registers): the widths of the reference's example
// policies are instantiated (64 runs on the tensor-core kernel instead), any other is refused
template <typename ENV>
static int launch_env(const EnvRolloutArgs& a, int hidden, cudaStream_t s){
    switch(hidden){
        case 16:  return launch_env_width<ENV, 16>(a, s);
        case 32:  return launch_env_width<ENV, 32>(a, s);
        case 128: return launch_env_width<ENV, 128>(a, s);
        default:  return B200RL_ERR_UNSUPPORTED;
    }
}

}  // namespace b200rl
using namespace b200rl;

extern "C" int b200rl_env_observation_dim(int env){ return env == B200RL_ENV_PENDULUM ? 3 : (env == B200RL_ENV_ACROBOT_SWINGUP || env == B200RL_ENV_ACROBOT) ? 6 : 0; }
extern "C" int b200rl_env_state_dim(int env){ return env == B200RL_ENV_PENDULUM ? 2 : (env == B200RL_ENV_ACROBOT_SWINGUP || env == B200RL_ENV_ACROBOT) ? 4 : 0; }
extern "C" int b200rl_env_reset_dim(int env){ return env == B200RL_ENV_ACROBOT ? 4 : (env == B200RL_ENV_PENDULUM || env == B200RL_ENV_ACROBOT_SWINGUP) ? 2 : 0; }

extern "C" int b200rl_env_rollout(int env, const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step, uint8_t* truncated,
                                  float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps, int step_limit, float* obs,
                                  float* act, float* rew, int* error_flag, b200rl_stream_t stream){
    return b200rl_env_rollout_flags(env, actor, actor_params, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds, n_envs, n_steps, step_limit,
                                    obs, act, rew, nullptr, error_flag, stream);
}
extern "C" int b200rl_env_rollout_flags(int env, const b200rl_mlp_shape* actor, const float* actor_params, float* states, int32_t* episode_step, uint8_t* truncated,
                                        float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps, int step_limit, float* obs,
                                        float* act, float* rew, uint8_t* terminated, int* error_flag, b200rl_stream_t stream){
    const int O = b200rl_env_observation_dim(env);
    if(O == 0 || !actor) return B200RL_ERR_INVALID_ARGUMENT;
    if(actor->n_layers != 3 || actor->input_dim != O || actor->dims[0] != actor->dims[1] || actor->dims[2] != 1) return B200RL_ERR_UNSUPPORTED;
    const int H = actor->dims[0];
    if(H != 16 && H != 32 && H != 64 && H != 128) return B200RL_ERR_UNSUPPORTED;
    for(int l = 0; l < 3; l++) if(!valid_activation(actor->acts[l])) return B200RL_ERR_INVALID_ARGUMENT;
    if(!actor_params || !states || !episode_step || !truncated || !episode_return || !obs || !act || !rew || n_envs < 0 || n_steps < 0 || n_reset_rounds < 0 || step_limit < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(reset_states == nullptr && n_reset_rounds != 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0 || n_steps == 0) return B200RL_OK;
    if(H == 64){           // the tensor-core kernel: second layer as split-fp16 MMAs, the environment as its compile-time policy
        RolloutArgs t{};
        t.params = actor_params; t.states = states; t.episode_step = episode_step; t.truncated = truncated; t.episode_return = episode_return;
        t.reset_states = reset_states; t.n_reset_rounds = n_reset_rounds; t.n_envs = n_envs; t.env_begin = 0; t.env_count = n_envs;
        t.n_steps = n_steps; t.step_limit = step_limit; t.obs = obs; t.act = act; t.rew = rew; t.terminated = terminated; t.error_flag = error_flag;
        for(int l = 0; l < 3; l++) t.acts[l] = actor->acts[l];
        return launch_env_rollout_tc(env, t, (cudaStream_t)stream);
    }
    EnvRolloutArgs a{};
    a.params = actor_params; a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return;
    a.reset_states = reset_states; a.n_reset_rounds = n_reset_rounds; a.n_envs = n_envs; a.n_steps = n_steps; a.step_limit = step_limit;
    a.obs = obs; a.act = act; a.rew = rew; a.terminated = terminated; a.error_flag = error_flag;
    for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
    if(env == B200RL_ENV_PENDULUM) return launch_env<PendulumEnv>(a, H, (cudaStream_t)stream);
    if(env == B200RL_ENV_ACROBOT) return launch_env<AcrobotEnv>(a, H, (cudaStream_t)stream);
    return launch_env<AcrobotSwingupEnv>(a, H, (cudaStream_t)stream);
}
