// AcrobotSwingup dynamics, reward and observation as device functions with the reference's arithmetic
// (rl/environments/acrobot/operations_generic.h, parameters acrobot.h:11-27). The reference mixes float and double: the
// unqualified cos / sin calls inside dsdt take their float argument promoted to double and make the surrounding products
// double, as do the literals 2.0, 6.0, 1.0 and 0.02; every intermediate assigned to a T variable rounds to float. Explicit
// *_rn intrinsics pin that rounding sequence (no contraction into fused multiply-adds). The unit masses, lengths and moments
// of inertia of the default parameters are folded into constants where the product with 1 is exact.
#pragma once
#include "common.cuh"

namespace b200rl { namespace acrobot {

constexpr float PI_F = 3.14159265358979323846f;      // math::PI<float>
constexpr float DT = 0.2f, MIN_TORQUE = -5.0f, MAX_TORQUE = 5.0f, MAX_VEL_1 = 4 * PI_F, MAX_VEL_2 = 9 * PI_F;
constexpr float G = 9.8f;                            // T g = 9.8
constexpr float HALF_G = 0.5f * G;                   // m2 * lc2 * g, float
constexpr float M_L_G = 1.5f * G;                    // (m1 * lc1 + m2 * l1) * g, float

__device__ __forceinline__ float clip(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }

// operations_generic.h:15-23
__device__ __forceinline__ float angle_normalize(float x){
    const float a = __fadd_rn(x, PI_F), b = 2.0f * PI_F;
    return __fsub_rn(__fsub_rn(a, __fmul_rn(b, floorf(__fdiv_rn(a, b)))), PI_F);
}

// operations_generic.h:60-99
__device__ __forceinline__ void dsdt(const float (&s)[4], float action, float (&d)[4]){
    const float theta1 = s[0], theta2 = s[1], dtheta1 = s[2], dtheta2 = s[3];
    const double cos2 = cos((double)theta2), sin2 = sin((double)theta2);
    // d1 = m1 lc1^2 + m2 (l1^2 + lc2^2 + 2 l1 lc2 cos(theta2)) + I1 + I2
    const double inner = __dadd_rn(1.25, cos2);
    const float d1 = (float)__dadd_rn(__dadd_rn(__dadd_rn(0.25, inner), 1.0), 1.0);
    // d2 = m2 (lc2^2 + l1 lc2 cos(theta2)) + I2
    const float d2 = (float)__dadd_rn(__dadd_rn(0.25, __dmul_rn(0.5, cos2)), 1.0);
    // phi2 = m2 lc2 g cos(theta1 + theta2 - pi / 2.0)
    const float phi2 = (float)__dmul_rn((double)HALF_G, cos(__dsub_rn((double)__fadd_rn(theta1, theta2), (double)PI_F / 2.0)));
    // phi1 = -m2 l1 lc2 dtheta2^2 sin(theta2) - 2 m2 l1 lc2 dtheta2 dtheta1 sin(theta2) + (m1 lc1 + m2 l1) g cos(theta1 - pi / 2) + phi2
    const double term1 = __dmul_rn((double)__fmul_rn(__fmul_rn(-0.5f, dtheta2), dtheta2), sin2);
    const double term2 = __dmul_rn((double)__fmul_rn(dtheta2, dtheta1), sin2);
    const double term3 = __dmul_rn((double)M_L_G, cos((double)__fsub_rn(theta1, PI_F / 2)));
    const float phi1 = (float)__dadd_rn(__dadd_rn(__dsub_rn(term1, term2), term3), (double)phi2);
    // ddtheta2 = (action + d2 / d1 phi1 - m2 l1 lc2 dtheta1^2 sin(theta2) - phi2) / (m2 lc2^2 + I2 - d2^2 / d1)
    const float head = __fadd_rn(action, __fmul_rn(__fdiv_rn(d2, d1), phi1));
    const double numerator = __dsub_rn(__dsub_rn((double)head, __dmul_rn((double)__fmul_rn(__fmul_rn(0.5f, dtheta1), dtheta1), sin2)), (double)phi2);
    const float denominator = __fsub_rn(1.25f, __fdiv_rn(__fmul_rn(d2, d2), d1));
    const float ddtheta2 = (float)__ddiv_rn(numerator, (double)denominator);
    const float ddtheta1 = __fdiv_rn(-__fadd_rn(__fmul_rn(d2, ddtheta2), phi1), d1);
    d[0] = dtheta1; d[1] = dtheta2; d[2] = ddtheta1; d[3] = ddtheta2;
}

// operations_generic.h:101-124
__device__ __forceinline__ void rk4(const float (&s)[4], float action, float (&next)[4], float dt){
    float k1[4], k2[4], k3[4], k4[4], y[4];
    const float dt2 = (float)((double)dt / 2.0);
    dsdt(s, action, k1);
#pragma unroll
    for(int i = 0; i < 4; i++) y[i] = __fadd_rn(s[i], __fmul_rn(dt2, k1[i]));
    dsdt(y, action, k2);
#pragma unroll
    for(int i = 0; i < 4; i++) y[i] = __fadd_rn(s[i], __fmul_rn(dt2, k2[i]));
    dsdt(y, action, k3);
#pragma unroll
    for(int i = 0; i < 4; i++) y[i] = __fadd_rn(s[i], __fmul_rn(dt, k3[i]));
    dsdt(y, action, k4);
    const double sixth = (double)dt / 6.0;
#pragma unroll
    for(int i = 0; i < 4; i++){
        const float sum = __fadd_rn(__fadd_rn(__fadd_rn(k1[i], __fmul_rn(2.0f, k2[i])), __fmul_rn(2.0f, k3[i])), k4[i]);
        next[i] = (float)__dadd_rn((double)s[i], __dmul_rn(sixth, (double)sum));
    }
}

// operations_generic.h:126-151
__device__ __forceinline__ void step(const float (&s)[4], float action, float (&next)[4]){
    const float clamped = clip(action, -1.0f, 1.0f);
    const double unit = __ddiv_rn(__dadd_rn((double)clamped, 1.0), 2.0);
    const float scaled = (float)__dadd_rn(__dmul_rn(unit, (double)(MAX_TORQUE - MIN_TORQUE)), (double)MIN_TORQUE);
    rk4(s, scaled, next, DT);
    next[0] = angle_normalize(next[0]);
    next[1] = angle_normalize(next[1]);
    next[2] = clip(next[2], -MAX_VEL_1, MAX_VEL_1);
    next[3] = clip(next[3], -MAX_VEL_2, MAX_VEL_2);
}

// operations_generic.h:157-178: the swing-up reward looks at the NEXT state only
__device__ __forceinline__ float swingup_reward(const float (&next)[4]){
    const float a = fabsf(angle_normalize(__fsub_rn(next[0], PI_F)));
    const float b = fabsf(angle_normalize(next[1]));
    const float scaled = __fmul_rn(__fdiv_rn(__fsub_rn(-a, b), 100.0f), DT);
    return (float)__ddiv_rn((double)scaled, 0.02);
}

// the terminating variant, operations_generic.h:193-195: (-cos(theta_1) - cos(theta_2 + theta_1)) > 1.0, the unqualified cos of a float
// argument, i.e. evaluated in double on the float-rounded sum
__device__ __forceinline__ bool terminated(const float (&s)[4]){
    return __dsub_rn(-cos((double)s[0]), cos((double)__fadd_rn(s[1], s[0]))) > 1.0;
}

}}  // namespace b200rl::acrobot
