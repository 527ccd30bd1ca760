// Argument block shared by the rollout kernels and the host-buffer pipeline.
#pragma once
#include "common.cuh"

namespace b200rl {

struct RolloutArgs {
    const float* params;        // actor arena: W1[H,OBS] b1[H] W2[H,H] b2[H] W3[1,H] b3[1]
    float* states;              // [n_envs, STATE_DIM] (Pendulum: 2)
    int32_t* episode_step;      // [n_envs]
    uint8_t* truncated;         // [n_envs]
    float* episode_return;      // [n_envs]
    const float* reset_states;  // [n_reset_rounds, n_envs, RESET_DIM] or null
    int n_reset_rounds;
    int32_t* reset_count;       // [n_envs] resets already consumed per env (in/out), or null = all zero
    int n_envs;                 // row pitch of the outputs: row = t * n_envs + env
    int env_begin, env_count;   // the slab of environments this launch owns
    int n_steps, step_limit;
    float* obs; float* act; float* rew;
    uint8_t* terminated;        // [n_steps * n_envs] the environment's terminated flag per transition, or null
    int* error_flag;            // device int, may be null: 1 = reset table exhausted, 2 = a bounded tensor-core wait timed out
    int acts[3];
    // on-policy collect (dataset != null): rows of the runner's dataset matrix instead of obs / act / rew
    float* dataset;             // [(n_steps + 1) * n_envs, ld_dataset], columns as in CollectColumns
    int ld_dataset;
    const float* noise;         // [n_steps, n_envs] standard-normal draws in the reference engine's order
    const float* log_std;       // device scalar: the actor's state-independent log standard deviation
    float neg_half_log_2pi;     // (float)(-0.5 * logf(2 pi)), evaluated on the host like the reference does
    // device-side random numbers (device_rng != 0): resets and action noise come from a counter-based generator keyed by
    // (rng_seed, environment, rng_step0 + step) instead of the host draw tables; reset_states and noise are then unused
    int device_rng;
    unsigned long long rng_seed, rng_step0;
};

// Philox-4x32-10 (Salmon, Moraes, Dror, Shaw: "Parallel random numbers: as easy as 1, 2, 3", SC'11): a counter-based generator, so the
// draw of (environment, step) does not depend on how the environments are sharded over launches or GPUs.
struct Philox {
    static constexpr uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
    __host__ __device__ static inline void block(uint32_t (&c)[4], uint32_t k0, uint32_t k1){
#pragma unroll
        for(int round = 0; round < 10; round++){
            const unsigned long long p0 = (unsigned long long)M0 * c[0], p1 = (unsigned long long)M1 * c[2];
            const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c[1] ^ k0, n1 = (uint32_t)p1, n2 = (uint32_t)(p0 >> 32) ^ c[3] ^ k1, n3 = (uint32_t)p0;
            c[0] = n0; c[1] = n1; c[2] = n2; c[3] = n3;
            k0 += W0; k1 += W1;
        }
    }
};
// One block per (environment, step): words 0-1 -> one standard normal (Box-Muller, cosine branch), words 2-3 -> the two uniforms of
// an initial state. u = ((word >> 9) + 0.5) * 2^-23 is exact in fp32 and lies strictly inside (0, 1).
struct StepDraws { float normal, u_theta, u_theta_dot; };
__device__ __forceinline__ float unit_uniform(uint32_t word){ return ((float)(word >> 9) + 0.5f) * 1.1920928955078125e-7f; }   // 2^-23
__device__ __forceinline__ StepDraws step_draws(unsigned long long seed, unsigned long long step, uint32_t env){
    uint32_t c[4] = {env, (uint32_t)step, (uint32_t)(step >> 32), 0u};
    Philox::block(c, (uint32_t)seed, (uint32_t)(seed >> 32));
    const float u1 = unit_uniform(c[0]), u2 = unit_uniform(c[1]);
    StepDraws d;
    d.normal = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
    d.u_theta = unit_uniform(c[2]);
    d.u_theta_dot = unit_uniform(c[3]);
    return d;
}

// Columns of the on-policy dataset for Pendulum (observation 3, action 1; rl/components/on_policy_runner/on_policy_runner.h:38-72)
enum CollectColumns { COL_OBS = 0, COL_ACTION_MEAN = 3, COL_ACTION = 4, COL_LOG_PROB = 5, COL_REWARD = 6, COL_TERMINATED = 7,
                      COL_TRUNCATED = 8, COL_RESET = 9, COL_VALUE = 10, COL_ADVANTAGE = 11, COL_TARGET_VALUE = 12, COLLECT_DATA_DIM = 13 };

// Gaussian policy head of the rollout (on_policy_runner/operations_generic_per_env.h:46-60, random/operations_cpu.h:40-48,
// random/operations_generic.h:87-97) with the reference's rounding sequence: action = eps * std + mean as separate multiply
// and add; log_prob = (neg_half_log_2pi - log_std) - 0.5 * ((action - mean) / std)^2, where the reference takes the square
// term and the subtraction in double: here the square is an exact float pair and the difference is rounded to float once
// (no double-precision instruction on the per-step path, see pendulum.cuh).
struct GaussianHead {
    float log_std, std;
    __device__ __forceinline__ void init(const float* log_std_ptr){
        log_std = __ldg(log_std_ptr);
        std = (float)exp((double)log_std);       // double exp rounded once = the host's correctly rounded expf
    }
    __device__ __forceinline__ float sample(float mean, float eps) const { return __fadd_rn(__fmul_rn(eps, std), mean); }
    __device__ __forceinline__ float log_prob(float mean, float action, float neg_half_log_2pi) const {
        const float p = __fdiv_rn(__fsub_rn(action, mean), std);
        const float h = __fmul_rn(p, p), l = __fmaf_rn(p, p, -h);                      // p^2 = h + l exactly
        const float a = __fsub_rn(neg_half_log_2pi, log_std), hh = __fmul_rn(0.5f, h);
        const float t = __fsub_rn(a, hh), tb = __fsub_rn(t, a);
        const float te = __fsub_rn(__fsub_rn(a, __fsub_rn(t, tb)), __fadd_rn(hh, tb)); // a - hh = t + te exactly
        return __fadd_rn(t, __fmaf_rn(-0.5f, l, te));
    }
};

int validate_actor(const b200rl_mlp_shape* actor);
int launch_rollout_tc(const RolloutArgs& a, cudaStream_t s);     // tensor-core kernel, H == 64, Pendulum
int launch_env_rollout_tc(int env, const RolloutArgs& a, cudaStream_t s);     // tensor-core kernel, H == 64, environment B200RL_ENV_*
int rollout_dispatch(const b200rl_mlp_shape* actor, const RolloutArgs& a, cudaStream_t s);

}  // namespace b200rl
