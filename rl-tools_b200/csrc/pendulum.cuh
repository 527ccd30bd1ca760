// Pendulum dynamics, reward and observation as device functions following the reference's arithmetic
// (rl/environments/pendulum/operations_generic.h). The reference mixes float and double: the literal 3.0 in the velocity
// update and 0.1 / 0.001 in the reward promote those expressions to double. Double-precision instructions are avoided
// here on purpose: on this GPU they queue behind tensor-core work, and the handful of them per environment step made the
// fused rollout 24 % slower (0.864 -> 0.695 ms per 65,536 x 200 rollout). Instead
//   - the velocity update, which feeds back into the (chaotic) trajectory, carries its intermediate results as unevaluated
//     sums of two floats (error-free products and sums built from fused multiply-adds), i.e. with ~48 significant bits, and
//     rounds to float once at the end: the result equals the reference's double computation rounded to float except when
//     that lies within ~2^-46 relative of a rounding boundary;
//   - the reward (an output, not fed back) is evaluated in float with fused multiply-adds: within 2 ulp of the reference.
// Explicit *_rn intrinsics keep the compiler from contracting or reordering the error-free sequences.
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
    // newthdot = (float)(theta_dot + (gravity_term + 3.0 * u) * dt), evaluated on float pairs:
    const float ph = __fmul_rn(3.0f / (MASS * LENGTH * LENGTH), u), pl = __fmaf_rn(3.0f / (MASS * LENGTH * LENGTH), u, -ph);     // 3 u = ph + pl exactly
    const float s = __fadd_rn(gravity_term, ph), sb = __fsub_rn(s, gravity_term);
    const float se = __fadd_rn(__fsub_rn(gravity_term, __fsub_rn(s, sb)), __fsub_rn(ph, sb));                                   // gravity_term + ph = s + se exactly
    const float bl = __fadd_rn(se, pl);                                                                                           // bracket = s + bl
    const float qh = __fmul_rn(s, DT), ql = __fmaf_rn(bl, DT, __fmaf_rn(s, DT, -qh));                                             // bracket * dt = qh + ql
    const float t = __fadd_rn(theta_dot, qh), tb = __fsub_rn(t, theta_dot);
    const float te = __fadd_rn(__fsub_rn(theta_dot, __fsub_rn(t, tb)), __fsub_rn(qh, tb));                                        // theta_dot + qh = t + te exactly
    float newthdot = __fadd_rn(t, __fadd_rn(te, ql));
    newthdot = clip(newthdot, -MAX_SPEED, MAX_SPEED);
    next_theta = __fadd_rn(theta, __fmul_rn(newthdot, DT));
    next_theta_dot = newthdot;
}
// operations_generic.h:130-139: unclamped action, pre-step state
__device__ __forceinline__ float reward(float theta, float theta_dot, float action){
    const float an = angle_normalize(theta);
    const float u = __fmul_rn(MAX_TORQUE, action);
    return -__fmaf_rn(0.001f, __fmul_rn(u, u), __fmaf_rn(__fmul_rn(0.1f, theta_dot), theta_dot, __fmul_rn(an, an)));
}

}}  // namespace b200rl::pendulum
