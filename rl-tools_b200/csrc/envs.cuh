// Environments as compile-time policies of the rollout kernels. An environment provides
//   STATE_DIM, OBS_DIM, RESET_DIM
//   reset(state, draws)                       the initial state from the RESET_DIM values of the reset table
//   observe(state, obs)                       the observation the actor sees
//   transition(state, action, next)           returns the reward of the transition (the reference's step + reward)
//   transition_obs(state, obs, action, next)  the same, given the observation of `state` (saves re-evaluating what both need)
//   TERMINATES, terminated(next)              whether the transition ended the episode (evaluated on the next state, as the runner does)
#pragma once
#include "common.cuh"
#include "pendulum.cuh"
#include "acrobot.cuh"

namespace b200rl {

struct PendulumEnv {          // rl/environments/pendulum/operations_generic.h
    static constexpr int STATE_DIM = 2, OBS_DIM = 3, RESET_DIM = 2;
    static constexpr bool TERMINATES = false;
    __device__ static bool terminated(const float (&)[2]){ return false; }
    __device__ static void reset(float (&s)[2], const float (&u)[2]){ s[0] = u[0]; s[1] = u[1]; }
    __device__ static void observe(const float (&s)[2], float (&o)[3]){ sincosf(s[0], &o[1], &o[0]); o[2] = s[1]; }
    __device__ static float transition(const float (&s)[2], float action, float (&next)[2]){
        pendulum::step(s[0], s[1], sinf(s[0]), action, next[0], next[1]);
        return pendulum::reward(s[0], s[1], action);
    }
    // the same transition given the observation of s (its second component is sin(theta), which the dynamics need again)
    __device__ static float transition_obs(const float (&s)[2], const float (&o)[3], float action, float (&next)[2]){
        pendulum::step(s[0], s[1], o[1], action, next[0], next[1]);
        return pendulum::reward(s[0], s[1], action);
    }
};
struct AcrobotSwingupEnv {    // rl/environments/acrobot/operations_generic.h
    static constexpr int STATE_DIM = 4, OBS_DIM = 6, RESET_DIM = 2;
    static constexpr bool TERMINATES = false;
    __device__ static bool terminated(const float (&)[4]){ return false; }
    __device__ static void reset(float (&s)[4], const float (&u)[2]){ s[0] = u[0]; s[1] = u[1]; s[2] = 0.0f; s[3] = 0.0f; }       // :46-53
    __device__ static void observe(const float (&s)[4], float (&o)[6]){                                                   // :180-191
        sincosf(s[0], &o[1], &o[0]); sincosf(s[1], &o[3], &o[2]); o[4] = s[2]; o[5] = s[3];
    }
    __device__ static float transition(const float (&s)[4], float action, float (&next)[4]){
        acrobot::step(s, action, next);
        return acrobot::swingup_reward(next);
    }
    __device__ static float transition_obs(const float (&s)[4], const float (&)[6], float action, float (&next)[4]){ return transition(s, action, next); }
};

struct AcrobotEnv: AcrobotSwingupEnv {    // rl::environments::Acrobot: the variant that terminates
    static constexpr int RESET_DIM = 4;
    static constexpr bool TERMINATES = true;
    __device__ static bool terminated(const float (&next)[4]){ return acrobot::terminated(next); }                         // :193-195
    __device__ static void reset(float (&s)[4], const float (&u)[4]){ s[0] = u[0]; s[1] = u[1]; s[2] = u[2]; s[3] = u[3]; }    // :38-44
    __device__ static float transition(const float (&s)[4], float action, float (&next)[4]){ acrobot::step(s, action, next); return -1.0f; }   // reward :154-156
    __device__ static float transition_obs(const float (&s)[4], const float (&)[6], float action, float (&next)[4]){ return transition(s, action, next); }
};

}  // namespace b200rl
