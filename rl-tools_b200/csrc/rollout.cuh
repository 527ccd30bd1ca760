// Argument block shared by the rollout kernels and the host-buffer pipeline.
#pragma once
#include "common.cuh"

namespace b200rl {

struct RolloutArgs {
    const float* params;        // actor arena: W1[H,3] b1[H] W2[H,H] b2[H] W3[1,H] b3[1]
    float* states;              // [n_envs, 2]
    int32_t* episode_step;      // [n_envs]
    uint8_t* truncated;         // [n_envs]
    float* episode_return;      // [n_envs]
    const float* reset_states;  // [n_reset_rounds, n_envs, 2] or null
    int n_reset_rounds;
    int32_t* reset_count;       // [n_envs] resets already consumed per env (in/out), or null = all zero
    int n_envs;                 // row pitch of the outputs: row = t * n_envs + env
    int env_begin, env_count;   // the slab of environments this launch owns
    int n_steps, step_limit;
    float* obs; float* act; float* rew;
    int* error_flag;            // device int, may be null: 1 = reset table exhausted, 2 = a bounded tensor-core wait timed out
    int acts[3];
};

int validate_actor(const b200rl_mlp_shape* actor);
int launch_rollout_simt(const RolloutArgs& a, int H, cudaStream_t s);
int launch_rollout_tc(const RolloutArgs& a, cudaStream_t s);     // tensor-core kernel, H == 64
int rollout_dispatch(const b200rl_mlp_shape* actor, const RolloutArgs& a, cudaStream_t s);

}  // namespace b200rl
