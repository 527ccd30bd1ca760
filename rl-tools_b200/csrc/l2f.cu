// L2F quadrotor in the configuration of the reference's own GPU throughput harness (src/rl/environments/l2f/cuda/benchmark.cu:31-60): state =
// StateRotors<StateRandomForce<StateBase>> -- position 3, orientation quaternion 4 (w first), linear velocity 3, angular velocity 3, a constant
// disturbance force 3 and torque 3, rotor speeds 4 = 23 floats -- advanced by step() (rl/environments/l2f/operations_generic.h:93-131): action
// clamp and map to the rotor-speed range, one RK4 step (utils/generic/integrators.h:20-49) of the rigid-body + rotor dynamics
// (operations_generic/60_dynamics.h:17-110), post_integration (70_post_integration.h:17-35, 127-150). One thread per quadrotor, the state in
// registers for all steps of a launch, the parameter set in the kernel's argument block (constant bank).
// This file is compiled WITHOUT multiply-add contraction (see the package's per-source flags): every expression below keeps the reference's
// association, division and square root are IEEE, so a step gives the reference's CPU bits.
#include "common.cuh"

namespace b200rl {

struct L2fState { float position[3], orientation[4], linear_velocity[3], angular_velocity[3], force[3], torque[3], rpm[4]; };
struct L2fDynamics { float rotor_positions[4][3], rotor_thrust_directions[4][3], rotor_torque_directions[4][3], rotor_thrust_coefficients[4][3], rotor_torque_constants[4],
                     rotor_time_constants_rising[4], rotor_time_constants_falling[4], mass, gravity[3], J[3][3], J_inv[3][3], hovering_throttle_relative, action_min, action_max; };
static_assert(sizeof(L2fDynamics) == 85 * sizeof(float) && sizeof(L2fState) == 23 * sizeof(float), "the layouts of the C ABI");
struct L2fArgs { L2fDynamics p; float dt, limit_position, limit_velocity, limit_angular_velocity; };

__device__ __forceinline__ void l2f_cross(const float* a, const float* b, float* out){
    out[0] = a[1] * b[2] - a[2] * b[1]; out[1] = a[2] * b[0] - a[0] * b[2]; out[2] = a[0] * b[1] - a[1] * b[0];
}
__device__ __forceinline__ void l2f_matvec(const float (&A)[3][3], const float* v, float* out){
#pragma unroll
    for(int i = 0; i < 3; i++){
        out[i] = 0;
#pragma unroll
        for(int j = 0; j < 3; j++) out[i] += A[i][j] * v[j];
    }
}
__device__ __forceinline__ float l2f_clamp(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }

// 60_dynamics.h: the rotor speeds in the state drive the body, the set-points drive the rotors
__device__ __forceinline__ void l2f_dynamics(const L2fDynamics& p, const L2fState& s, const float (&setpoint)[4], L2fState& d){
    float thrust[3] = {0, 0, 0}, torque[3] = {0, 0, 0};
#pragma unroll
    for(int r = 0; r < 4; r++){
        const float rpm = s.rpm[r];
        const float magnitude = p.rotor_thrust_coefficients[r][0] + p.rotor_thrust_coefficients[r][1] * rpm + p.rotor_thrust_coefficients[r][2] * rpm * rpm;
        float rotor_thrust[3];
#pragma unroll
        for(int i = 0; i < 3; i++){ rotor_thrust[i] = p.rotor_thrust_directions[r][i] * magnitude; thrust[i] += rotor_thrust[i]; }
        const float reaction = magnitude * p.rotor_torque_constants[r];
#pragma unroll
        for(int i = 0; i < 3; i++) torque[i] += p.rotor_torque_directions[r][i] * reaction;
        const float* a = p.rotor_positions[r];
        torque[0] += a[1] * rotor_thrust[2] - a[2] * rotor_thrust[1];
        torque[1] += a[2] * rotor_thrust[0] - a[0] * rotor_thrust[2];
        torque[2] += a[0] * rotor_thrust[1] - a[1] * rotor_thrust[0];
    }
#pragma unroll
    for(int i = 0; i < 3; i++) d.position[i] = s.linear_velocity[i];
    const float* q = s.orientation; const float* w = s.angular_velocity;
    d.orientation[0] = -q[1] * w[0] - q[2] * w[1] - q[3] * w[2];                  // quaternion_helper.h:11-19
    d.orientation[1] =  q[0] * w[0] + q[2] * w[2] - q[3] * w[1];
    d.orientation[2] =  q[0] * w[1] + q[3] * w[0] - q[1] * w[2];
    d.orientation[3] =  q[0] * w[2] + q[1] * w[1] - q[2] * w[0];
#pragma unroll
    for(int i = 0; i < 4; i++) d.orientation[i] *= 0.5f;
    float var[3], rotated[3];                                                     // rotate_vector_by_quaternion, :22-36
    l2f_cross(q + 1, thrust, var);
#pragma unroll
    for(int i = 0; i < 3; i++) var[i] *= 2.0f;
    l2f_cross(q + 1, var, rotated);
#pragma unroll
    for(int i = 0; i < 3; i++) rotated[i] += var[i] * q[0];
#pragma unroll
    for(int i = 0; i < 3; i++) rotated[i] += thrust[i];
    const float inverse_mass = 1 / p.mass;
#pragma unroll
    for(int i = 0; i < 3; i++) d.linear_velocity[i] = rotated[i] * inverse_mass;
#pragma unroll
    for(int i = 0; i < 3; i++) d.linear_velocity[i] += p.gravity[i];
    float v1[3], v2[3];
    l2f_matvec(p.J, w, v1);
    l2f_cross(w, v1, v2);
#pragma unroll
    for(int i = 0; i < 3; i++) v1[i] = torque[i] - v2[i];
    l2f_matvec(p.J_inv, v1, d.angular_velocity);
#pragma unroll
    for(int i = 0; i < 3; i++) d.linear_velocity[i] += s.force[i] / p.mass;      // StateRandomForce, 60_dynamics.h:77-88
    float extra[3];
    l2f_matvec(p.J_inv, s.torque, extra);
#pragma unroll
    for(int i = 0; i < 3; i++) d.angular_velocity[i] += extra[i];
#pragma unroll
    for(int r = 0; r < 4; r++){                                                  // StateRotors, :89-101
        const float tau = setpoint[r] >= s.rpm[r] ? p.rotor_time_constants_rising[r] : p.rotor_time_constants_falling[r];
        d.rpm[r] = (setpoint[r] - s.rpm[r]) * 1 / tau;
    }
}
// scalar_multiply_accumulate over the integrated components (50_state_algebra.h)
__device__ __forceinline__ void l2f_axpy(const L2fState& k, float scalar, L2fState& out){
#pragma unroll
    for(int i = 0; i < 3; i++){
        out.position[i] += scalar * k.position[i]; out.orientation[i] += scalar * k.orientation[i];
        out.linear_velocity[i] += scalar * k.linear_velocity[i]; out.angular_velocity[i] += scalar * k.angular_velocity[i];
    }
    out.orientation[3] += scalar * k.orientation[3];
#pragma unroll
    for(int i = 0; i < 4; i++) out.rpm[i] += scalar * k.rpm[i];
}

__global__ void __launch_bounds__(128) l2f_steps_kernel(L2fArgs a, float* __restrict__ states, const float* __restrict__ actions, int n, int n_steps){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n) return;
    const L2fDynamics& p = a.p;
    L2fState s;
    {
        const float* row = states + (size_t)e * 23;
        float* dst = reinterpret_cast<float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) dst[k] = row[k];
    }
    float setpoint[4];
    const float half_range = (p.action_max - p.action_min) / 2;                  // operations_generic.h:103-109; the default action noise is 0
#pragma unroll
    for(int i = 0; i < 4; i++){
        float act = __ldg(actions + (size_t)e * 4 + i);
        act += 0.0f;
        act = l2f_clamp(act, -1.0f, 1.0f);
        setpoint[i] = act * half_range + p.action_min + half_range;
    }
    const float dt = a.dt;
    for(int step = 0; step < n_steps; step++){
        L2fState k1 = s, k2 = s, k3 = s, k4 = s, t;
        l2f_dynamics(p, s, setpoint, k1);
        t = s; l2f_axpy(k1, dt / 2, t); l2f_dynamics(p, t, setpoint, k2);
        t = s; l2f_axpy(k2, dt / 2, t); l2f_dynamics(p, t, setpoint, k3);
        t = s; l2f_axpy(k3, dt, t);     l2f_dynamics(p, t, setpoint, k4);
        L2fState next = s;
        l2f_axpy(k1, dt / 6, next); l2f_axpy(k2, dt / 3, next); l2f_axpy(k3, dt / 3, next); l2f_axpy(k4, dt / 6, next);
        float norm = 0;                                                          // 70_post_integration.h:21-34
#pragma unroll
        for(int i = 0; i < 4; i++) norm += next.orientation[i] * next.orientation[i];
        norm = sqrtf(norm);
#pragma unroll
        for(int i = 0; i < 4; i++) next.orientation[i] /= norm;
#pragma unroll
        for(int i = 0; i < 3; i++){
            next.position[i] = l2f_clamp(next.position[i], -a.limit_position, a.limit_position);
            next.linear_velocity[i] = l2f_clamp(next.linear_velocity[i], -a.limit_velocity, a.limit_velocity);
            next.angular_velocity[i] = l2f_clamp(next.angular_velocity[i], -a.limit_angular_velocity, a.limit_angular_velocity);
        }
#pragma unroll
        for(int i = 0; i < 4; i++) next.rpm[i] = l2f_clamp(next.rpm[i], p.action_min, p.action_max);      // :137-139
        s = next;
    }
    {
        float* row = states + (size_t)e * 23;
        const float* src = reinterpret_cast<const float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) row[k] = src[k];
    }
}

}  // namespace b200rl
using namespace b200rl;

extern "C" int b200rl_l2f_steps(const b200rl_l2f_parameters* parameters, float* states, const float* actions, int n, int n_steps, b200rl_stream_t stream){
    if(!parameters || n < 0 || n_steps < 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0 || n_steps == 0) return B200RL_OK;
    if(!states || !actions) return B200RL_ERR_INVALID_ARGUMENT;
    L2fArgs a;
    static_assert(sizeof(parameters->dynamics) == sizeof(L2fDynamics), "b200rl_l2f_parameters::dynamics");
    memcpy(&a.p, parameters->dynamics, sizeof(L2fDynamics));
    a.dt = parameters->dt; a.limit_position = parameters->state_limit_position; a.limit_velocity = parameters->state_limit_velocity;
    a.limit_angular_velocity = parameters->state_limit_angular_velocity;
    l2f_steps_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(a, states, actions, n, n_steps);
    B200RL_LAUNCH_CHECK("l2f_steps");
    return B200RL_OK;
}
