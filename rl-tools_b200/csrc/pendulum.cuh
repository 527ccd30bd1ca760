// Pendulum dynamics, reward and observation as device functions with the reference's exact arithmetic
// (rl/environments/pendulum/operations_generic.h). The reference mixes float and double: the literal 3.0 in the
// velocity update and 0.1 / 0.001 in the reward promote those expressions to double, and the CPU oracle build keeps
// multiply and add separate. Explicit *_rn intrinsics pin the same rounding sequence here, so that for identical
// sin/cos/action inputs the next state and the reward are bit-identical to the CPU path.
#pragma once
#include "common.cuh"

namespace b200rl { namespace pendulum {

constexpr float PI_F = 3.14159265358979323846f;      // math::PI<float>
constexpr float G = 10.0f, MAX_SPEED = 8.0f, MAX_TORQUE = 2.0f, DT = 0.05f, MASS = 1.0f, LENGTH = 1.0f;   // pendulum.h:11-25

__device__ __forceinline__ float clip(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }

// operations_generic.h:14-22
__device__ __forceinline__ float angle_normalize(float x){
    const float a = __fadd_rn(x, PI_F), b = 2.0f * PI_F;
    return __fsub_rn(__fsub_rn(a, __fmul_rn(b, floorf(__fdiv_rn(a, b)))), PI_F);
}
// operations_generic.h:78-101; sin_theta = sinf(theta) is passed in because the observation needs it too
__device__ __forceinline__ void step(float theta, float theta_dot, float sin_theta, float action, float& next_theta, float& next_theta_dot){
    float u = __fmul_rn(MAX_TORQUE, clip(action, -1.0f, 1.0f));
    u = clip(u, -MAX_TORQUE, MAX_TORQUE);
    const float gravity_term = __fmul_rn(3.0f * G / (2.0f * LENGTH), sin_theta);               // float
    const double bracket = __dadd_rn((double)gravity_term, __dmul_rn(3.0 / (double)(MASS * LENGTH * LENGTH), (double)u));
    float newthdot = (float)__dadd_rn((double)theta_dot, __dmul_rn(bracket, (double)DT));
    newthdot = clip(newthdot, -MAX_SPEED, MAX_SPEED);
    next_theta = __fadd_rn(theta, __fmul_rn(newthdot, DT));
    next_theta_dot = newthdot;
}
// operations_generic.h:130-139: unclamped action, pre-step state
__device__ __forceinline__ float reward(float theta, float theta_dot, float action){
    const float an = angle_normalize(theta);
    const float u = __fmul_rn(MAX_TORQUE, action);
    double costs = __dadd_rn((double)__fmul_rn(an, an), __dmul_rn(__dmul_rn(0.1, (double)theta_dot), (double)theta_dot));
    costs = __dadd_rn(costs, __dmul_rn(0.001, (double)__fmul_rn(u, u)));
    return -(float)costs;
}

}}  // namespace b200rl::pendulum
