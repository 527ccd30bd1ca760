// L2F quadrotor in the configuration of the reference's own GPU throughput harness (src/rl/environments/l2f/cuda/benchmark.cu:31-60): state =
// StateRotors<StateRandomForce<StateBase>> -- position 3, orientation quaternion 4 (w first), linear velocity 3, angular velocity 3, a constant
// disturbance force 3 and torque 3, rotor speeds 4 = 23 floats -- advanced by step() (rl/environments/l2f/operations_generic.h:93-131): action
// clamp and map to the rotor-speed range, one RK4 step (utils/generic/integrators.h:20-49) of the rigid-body + rotor dynamics
// (operations_generic/60_dynamics.h:17-110), post_integration (70_post_integration.h:17-35, 127-150). One thread per quadrotor, the state in
// registers for all steps of a launch, the parameter set in the kernel's argument block (constant bank).
// This file is compiled WITHOUT multiply-add contraction (see the package's per-source flags): every expression below keeps the reference's
// association, division and square root are IEEE, so a step gives the reference's CPU bits.
#include "common.cuh"
#include "rollout.cuh"

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

// one step() of the environment: action clamp and rotor-range map (operations_generic.h:103-109; the default action noise is 0), RK4, post_integration
__device__ __forceinline__ void l2f_step(const L2fArgs& a, const L2fState& s, const float (&action)[4], L2fState& next){
    const L2fDynamics& p = a.p;
    float setpoint[4];
    const float half_range = (p.action_max - p.action_min) / 2;
#pragma unroll
    for(int i = 0; i < 4; i++){
        float act = action[i];
        act += 0.0f;
        act = l2f_clamp(act, -1.0f, 1.0f);
        setpoint[i] = act * half_range + p.action_min + half_range;
    }
    const float dt = a.dt;
    L2fState k1 = s, k2 = s, k3 = s, k4 = s, t;
    l2f_dynamics(p, s, setpoint, k1);
    t = s; l2f_axpy(k1, dt / 2, t); l2f_dynamics(p, t, setpoint, k2);
    t = s; l2f_axpy(k2, dt / 2, t); l2f_dynamics(p, t, setpoint, k3);
    t = s; l2f_axpy(k3, dt, t);     l2f_dynamics(p, t, setpoint, k4);
    next = s;
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
}

__global__ void __launch_bounds__(128) l2f_steps_kernel(L2fArgs a, float* __restrict__ states, const float* __restrict__ actions, int n, int n_steps){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n) return;
    L2fState s;
    {
        const float* row = states + (size_t)e * 23;
        float* dst = reinterpret_cast<float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) dst[k] = row[k];
    }
    float action[4];
#pragma unroll
    for(int i = 0; i < 4; i++) action[i] = __ldg(actions + (size_t)e * 4 + i);
    for(int step = 0; step < n_steps; step++){
        L2fState next;
        l2f_step(a, s, action, next);
        s = next;
    }
    {
        float* row = states + (size_t)e * 23;
        const float* src = reinterpret_cast<const float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) row[k] = src[k];
    }
}

// ---------------------------------------------------------------------------------------------------------------
// The runner loop on this environment, fused like the other environments' rollouts (one thread per quadrotor, runner state in registers,
// the actor 18 -> H -> H -> 4 in shared memory): reset-if-truncated from the table, observe (40_observe.h:42-147: position, rotation matrix,
// velocities; the default observation noise is 0), actor forward as fp32 FMA chains in the reference's order (bias first, inputs
// ascending), step, reward (reward_functions/squared/operations_generic.h:12-103, desired state at the origin), terminated on the NEXT
// state (operations_generic.h:143-158), counters (operations_generic_per_env.h:62-108).
// mdp: non_negative, scale, constant, termination penalty, weights position, position clip, orientation, linear / angular velocity,
// linear / angular acceleration, action, d_action, position error integral; termination enabled, position / velocity / angular thresholds.
// ---------------------------------------------------------------------------------------------------------------
struct L2fRolloutArgs {
    L2fArgs env; float mdp[18];
    const float* params; float* states; int32_t* episode_step; uint8_t* truncated; float* episode_return;
    const float* reset_states; int n_reset_rounds, n_envs, n_steps, step_limit;
    float* obs; float* act; float* rew; uint8_t* terminated; int* error_flag; int acts[3];
    // device_rng != 0: a reset draws its initial state in the kernel (keyed by rng_seed, the environment and rng_step0 + step) from `init`
    int device_rng; unsigned long long rng_seed, rng_step0; float init[12];
};

// sample_initial_state of the harness' state (operations_generic/30_sample_initial_state.h:19-207) as a function of its draws: u[17] uniforms
// in [0, 1) (guidance; position 3; orientation u, v, angle; linear velocity 3; angular velocity 3; rotor speeds 4), nrm[6] standard normals
// (force 3, torque 3; the third torque component has std / 100). init: guidance, max_position, max_angle, max_linear_velocity,
// max_angular_velocity, relative_rpm, min_rpm, max_rpm, force mean / std, torque mean / std. The reference writes 2.0 / 1.0 / 0.5 as double
// literals in sample_orientation: those products are taken in double here too (a reset is rare next to a step).
__device__ __forceinline__ void l2f_initial_state(const float (&init)[12], float action_min, float action_max, const float (&u)[17], const float (&nrm)[6], L2fState& s){
    const bool guidance = u[0] < init[0];
#pragma unroll
    for(int i = 0; i < 3; i++){
        s.position[i] = guidance ? 0.0f : u[1 + i] * (init[1] - (-init[1])) + (-init[1]);
        s.linear_velocity[i] = guidance ? 0.0f : u[7 + i] * (init[3] - (-init[3])) + (-init[3]);
        s.angular_velocity[i] = guidance ? 0.0f : u[10 + i] * (init[4] - (-init[4])) + (-init[4]);
    }
    if(init[2] > 0 && !guidance){
        const float phi = (float)(2.0 * (double)3.14159265358979323846f * (double)u[4]);
        const float cos_theta = (float)(1.0 - 2.0 * (double)u[5]);
        const float sin_theta = (float)sqrt(1.0 - (double)(cos_theta * cos_theta));
        const float x = sin_theta * cosf(phi), y = sin_theta * sinf(phi), z = cos_theta;
        const float half = (float)(0.5 * (double)u[6]);
        const float sn = sinf(half);
        s.orientation[0] = cosf(half); s.orientation[1] = x * sn; s.orientation[2] = y * sn; s.orientation[3] = z * sn;
    }
    else { s.orientation[0] = 1; s.orientation[1] = 0; s.orientation[2] = 0; s.orientation[3] = 0; }
#pragma unroll
    for(int i = 0; i < 3; i++){
        const float fs = init[9], ts = i == 2 ? init[11] / 100 : init[11];
        s.force[i] = fs == 0 ? init[8] : nrm[i] * fs + init[8];
        s.torque[i] = ts == 0 ? init[10] : nrm[3 + i] * ts + init[10];
    }
    float min_rpm, max_rpm;
    if(init[5] != 0.0f){
        min_rpm = (init[6] + 1) / 2 * (action_max - action_min) + action_min;
        max_rpm = (init[7] + 1) / 2 * (action_max - action_min) + action_min;
    }
    else{
        min_rpm = init[6] < 0 ? action_min : init[6];
        max_rpm = init[7] < 0 ? action_max : init[7];
        if(max_rpm > action_max) max_rpm = action_max;
        if(min_rpm > max_rpm) min_rpm = max_rpm;
    }
#pragma unroll
    for(int i = 0; i < 4; i++) s.rpm[i] = u[13 + i] * (max_rpm - min_rpm) + min_rpm;
}
// The draws of one reset: six Philox-4x32-10 blocks keyed by the seed, counter (environment, step, block + 1): words 0-16 the uniforms,
// words 17-22 three Box-Muller pairs (both branches) for the six normals, which are only evaluated when a disturbance has a spread.
__device__ __forceinline__ void l2f_reset_draws(unsigned long long seed, unsigned long long step, uint32_t env, bool want_normals, float (&u)[17], float (&nrm)[6]){
    uint32_t w[24];
#pragma unroll
    for(int b = 0; b < 6; b++){
        uint32_t c[4] = {env, (uint32_t)step, (uint32_t)(step >> 32), (uint32_t)(b + 1)};
        Philox::block(c, (uint32_t)seed, (uint32_t)(seed >> 32));
#pragma unroll
        for(int k = 0; k < 4; k++) w[4 * b + k] = c[k];
    }
#pragma unroll
    for(int i = 0; i < 17; i++) u[i] = unit_uniform(w[i]);
#pragma unroll
    for(int i = 0; i < 3; i++){
        if(want_normals){
            const float r = sqrtf(-2.0f * logf(unit_uniform(w[17 + 2 * i]))), a = 2.0f * unit_uniform(w[18 + 2 * i]);
            nrm[2 * i] = r * cospif(a); nrm[2 * i + 1] = r * sinpif(a);
        }
        else { nrm[2 * i] = 0.0f; nrm[2 * i + 1] = 0.0f; }
    }
}
__global__ void l2f_initial_states_kernel(L2fRolloutArgs a, const float* __restrict__ u, const float* __restrict__ nrm, float* __restrict__ states, int n){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n) return;
    float uu[17], nn[6];
#pragma unroll
    for(int i = 0; i < 17; i++) uu[i] = u[(size_t)e * 17 + i];
#pragma unroll
    for(int i = 0; i < 6; i++) nn[i] = nrm[(size_t)e * 6 + i];
    L2fState s;
    l2f_initial_state(a.init, a.env.p.action_min, a.env.p.action_max, uu, nn, s);
    const float* src = reinterpret_cast<const float*>(&s);
#pragma unroll
    for(int k = 0; k < 23; k++) states[(size_t)e * 23 + k] = src[k];
}
__device__ __forceinline__ void l2f_observe(const L2fState& s, float (&o)[18]){
    const float* q = s.orientation;
#pragma unroll
    for(int i = 0; i < 3; i++){ o[i] = s.position[i]; o[12 + i] = s.linear_velocity[i]; o[15 + i] = s.angular_velocity[i]; }
    o[3]  = (1 - 2 * q[2] * q[2] - 2 * q[3] * q[3]); o[4]  = (2 * q[1] * q[2] - 2 * q[0] * q[3]); o[5]  = (2 * q[1] * q[3] + 2 * q[0] * q[2]);
    o[6]  = (2 * q[1] * q[2] + 2 * q[0] * q[3]); o[7]  = (1 - 2 * q[1] * q[1] - 2 * q[3] * q[3]); o[8]  = (2 * q[2] * q[3] - 2 * q[0] * q[1]);
    o[9]  = (2 * q[1] * q[3] - 2 * q[0] * q[2]); o[10] = (2 * q[2] * q[3] + 2 * q[0] * q[1]); o[11] = (1 - 2 * q[1] * q[1] - 2 * q[2] * q[2]);
}
__device__ __forceinline__ bool l2f_terminated(const float (&mdp)[18], const L2fState& s){
    if(mdp[14] != 0.0f){
#pragma unroll
        for(int i = 0; i < 3; i++)
            if(fabsf(s.position[i]) > mdp[15] || fabsf(s.linear_velocity[i]) > mdp[16] || fabsf(s.angular_velocity[i]) > mdp[17]) return true;
    }
    return false;
}
__device__ __forceinline__ float l2f_reward(const L2fArgs& a, const float (&mdp)[18], const L2fState& s, const float (&action)[4], const L2fState& next, bool terminated){
    const float orientation_cost = 2 * acosf(1 - fabsf(s.orientation[3]));
    float position_cost = sqrtf(s.position[0] * s.position[0] + s.position[1] * s.position[1] + s.position[2] * s.position[2]);
    if(mdp[5] > 0) position_cost = fminf(position_cost, mdp[5]);
    const float linear_vel_cost = sqrtf(s.linear_velocity[0] * s.linear_velocity[0] + s.linear_velocity[1] * s.linear_velocity[1] + s.linear_velocity[2] * s.linear_velocity[2]);
    const float angular_vel_cost = sqrtf(s.angular_velocity[0] * s.angular_velocity[0] + s.angular_velocity[1] * s.angular_velocity[1] + s.angular_velocity[2] * s.angular_velocity[2]);
    float la[3], aa[3];
#pragma unroll
    for(int i = 0; i < 3; i++){ la[i] = next.linear_velocity[i] - s.linear_velocity[i]; aa[i] = next.angular_velocity[i] - s.angular_velocity[i]; }
    const float linear_acc_cost = sqrtf(la[0] * la[0] + la[1] * la[1] + la[2] * la[2]) / a.dt;
    const float angular_acc_cost = sqrtf(aa[0] * aa[0] + aa[1] * aa[1] + aa[2] * aa[2]) / a.dt;
    float acc = 0;
#pragma unroll
    for(int i = 0; i < 4; i++){
        const float diff = (action[i] + 1.0f) / 2.0f - a.p.hovering_throttle_relative;
        acc += diff * diff;
    }
    float action_cost = sqrtf(acc);
    action_cost *= action_cost;
    float weighted = 0;
    weighted += mdp[4] * position_cost; weighted += mdp[6] * orientation_cost; weighted += mdp[7] * linear_vel_cost; weighted += mdp[8] * angular_vel_cost;
    weighted += mdp[9] * linear_acc_cost; weighted += mdp[10] * angular_acc_cost; weighted += mdp[11] * action_cost; weighted += mdp[12] * 0.0f; weighted += mdp[13] * 0.0f;
    const float scaled = mdp[1] * weighted;
    if(terminated) return mdp[3];
    const float reward = -scaled + mdp[2];
    return (reward > 0 || mdp[0] == 0.0f) ? reward : 0.0f;
}

// One CTA of 14 warps per SM: 448 quadrotors, so 65536 of them (443 per SM) are resident at once. A lane owns one quadrotor for the
// environment part (reset, observe, step, reward) and, for the two hidden layers, a register tile of 8 quadrotors x H/8 units of its warp's
// 32 x H product: operands come from shared memory as 16-byte loads that each feed 32 multiply-adds (one broadcast weight per multiply-add,
// as a thread-per-quadrotor layer would load it, leaves the kernel bound by shared-memory wavefronts). Every unit still accumulates
// bias + sum over k in ascending k with fused multiply-adds, so the actor's values are those of a plain per-sample loop.
constexpr int L2F_ROLLOUT_WARPS = 14, L2F_ROLLOUT_THREADS = 32 * L2F_ROLLOUT_WARPS;
template <int H>
struct L2fRolloutLayout {
    static constexpr int O = 18, A = 4;
    static constexpr int JPT = H / 8;                         // units per lane: unit j = og + 8 * jj for the lane's column group og = lane & 7
    static constexpr int VW = JPT < 4 ? JPT : 4, NV = JPT / VW;  // a lane's weights per k arrive as NV vectors of VW floats
    static constexpr int PITCH = 36;                          // row pitch of the hidden tile: rows og, og + 8, .. of eight lanes land on distinct banks
    // floats from the start of shared memory; the first two layers transposed ([k][slot]), the last as [unit][4]
    static constexpr int W1T = 0, B1 = W1T + O * H, W2T = B1 + H, B2 = W2T + H * H, W3T = B2 + H, B3 = W3T + A * H, WARP0 = B3 + A;
    static constexpr int OBS_TILE = O * 32, HID_TILE = H * PITCH, PER_WARP = OBS_TILE + HID_TILE;
    static constexpr size_t BYTES = sizeof(float) * (WARP0 + L2F_ROLLOUT_WARPS * PER_WARP);
    __host__ __device__ static constexpr int slot(int j){ return ((j / 8) / VW) * (8 * VW) + (j % 8) * VW + (j / 8) % VW; }
};

// acc[ee][jj] += sum over k of act[k][8 eg + ee] * wT[k][slot(og + 8 jj)], k ascending; act rows have the pitch ACT_PITCH. Two units advance
// with one packed multiply-add (each half is the same fused multiply-add as before; the kernel is bound by instruction issue).
template <int H, int K, int ACT_PITCH>
__device__ __forceinline__ void l2f_tile_layer(const float* __restrict__ act_tile, const float* __restrict__ wT, int eg, int og, float2 (&acc)[8][H / 16]){
    using L = L2fRolloutLayout<H>;
#pragma unroll 2
    for(int k = 0; k < K; k++){
        float x[8];
        float2 w[L::JPT / 2];
        const float4 x0 = *reinterpret_cast<const float4*>(act_tile + k * ACT_PITCH + eg * 8), x1 = *reinterpret_cast<const float4*>(act_tile + k * ACT_PITCH + eg * 8 + 4);
        x[0] = x0.x; x[1] = x0.y; x[2] = x0.z; x[3] = x0.w; x[4] = x1.x; x[5] = x1.y; x[6] = x1.z; x[7] = x1.w;
#pragma unroll
        for(int v = 0; v < L::NV; v++){
            const float* src = wT + k * H + v * (8 * L::VW) + og * L::VW;
            if constexpr (L::VW == 4){ const float4 t = *reinterpret_cast<const float4*>(src); w[2 * v] = make_float2(t.x, t.y); w[2 * v + 1] = make_float2(t.z, t.w); }
            else w[0] = *reinterpret_cast<const float2*>(src);
        }
#pragma unroll
        for(int ee = 0; ee < 8; ee++){
            const float2 xx = make_float2(x[ee], x[ee]);
#pragma unroll
            for(int jp = 0; jp < L::JPT / 2; jp++) acc[ee][jp] = __ffma2_rn(w[jp], xx, acc[ee][jp]);
        }
    }
}
// bias in, activation out: the lane's tile goes to the hidden tile as rows [unit][quadrotor of the warp]
template <int H>
__device__ __forceinline__ void l2f_tile_store(float* hid, float2 (&acc)[8][H / 16], int eg, int og, int act){
    using L = L2fRolloutLayout<H>;
#pragma unroll
    for(int jj = 0; jj < L::JPT; jj++){
        float* row = hid + (og + 8 * jj) * L::PITCH + eg * 8;
        float v[8];
#pragma unroll
        for(int ee = 0; ee < 8; ee++) v[ee] = activation_rt((jj & 1) ? acc[ee][jj / 2].y : acc[ee][jj / 2].x, act);
        *reinterpret_cast<float4*>(row) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4*>(row + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
}

template <int H>
__global__ void __launch_bounds__(L2F_ROLLOUT_THREADS, 1) l2f_rollout_kernel(L2fRolloutArgs a){
    using L = L2fRolloutLayout<H>;
    constexpr int O = L::O, A = L::A;
    extern __shared__ __align__(16) float smem[];
    {
        constexpr int W1_END = O * H, B1_END = W1_END + H, W2_END = B1_END + H * H, B2_END = W2_END + H, W3_END = B2_END + A * H;
        for(int i = threadIdx.x; i < W3_END + A; i += blockDim.x){
            const float v = __ldg(a.params + i);
            int dst = i;                                                                       // biases keep their place
            if(i < W1_END) dst = L::W1T + (i % O) * H + L::slot(i / O);                        // W1[j][k]
            else if(i >= B1_END && i < W2_END){ const int r = i - B1_END; dst = L::W2T + (r % H) * H + L::slot(r / H); }     // W2[j][k]
            else if(i >= B2_END && i < W3_END){ const int r = i - B2_END; dst = L::W3T + (r % H) * A + r / H; }             // W3[c][j]
            smem[dst] = v;
        }
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, eg = lane >> 3, og = lane & 7;
    float* obs_tile = smem + L::WARP0 + warp * L::PER_WARP;
    float* hid = obs_tile + L::OBS_TILE;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    const bool active = e < a.n_envs;                     // idle lanes of the last warp still take part in the warp's tiles
    L2fState s;
    {
        float* dst = reinterpret_cast<float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) dst[k] = active ? a.states[(size_t)e * 23 + k] : 0.0f;
    }
    int es = active ? a.episode_step[e] : 0, resets = 0;
    bool trunc = active ? a.truncated[e] != 0 : false;
    float er = active ? a.episode_return[e] : 0.0f;
    for(int t = 0; t < a.n_steps; t++){
        const size_t row = (size_t)t * a.n_envs + e;
        if(active){
            if(trunc){                                   // operations_generic_per_env.h:8-61
                if(a.device_rng){
                    float uu[17], nn[6];
                    l2f_reset_draws(a.rng_seed, a.rng_step0 + (unsigned long long)t, (uint32_t)e, a.init[9] != 0.0f || a.init[11] != 0.0f, uu, nn);
                    l2f_initial_state(a.init, a.env.p.action_min, a.env.p.action_max, uu, nn, s);
                }
                else if(a.reset_states != nullptr && resets < a.n_reset_rounds){
                    const float* src = a.reset_states + ((size_t)resets * a.n_envs + e) * 23;
                    float* dst = reinterpret_cast<float*>(&s);
#pragma unroll
                    for(int k = 0; k < 23; k++) dst[k] = __ldg(src + k);
                }
                else if(a.error_flag) *a.error_flag = 1;
                resets++; es = 0; er = 0.0f;
            }
            float o[O];
            l2f_observe(s, o);
#pragma unroll
            for(int k = 0; k < O; k++){ a.obs[row * O + k] = o[k]; obs_tile[k * 32 + lane] = o[k]; }
        }
        else {
#pragma unroll
            for(int k = 0; k < O; k++) obs_tile[k * 32 + lane] = 0.0f;
        }
        __syncwarp();
        {
            float2 acc[8][L::JPT / 2];
#pragma unroll
            for(int jp = 0; jp < L::JPT / 2; jp++){
                const float2 b = make_float2(smem[L::B1 + og + 16 * jp], smem[L::B1 + og + 16 * jp + 8]);
#pragma unroll
                for(int ee = 0; ee < 8; ee++) acc[ee][jp] = b;
            }
            l2f_tile_layer<H, O, 32>(obs_tile, smem + L::W1T, eg, og, acc);
            l2f_tile_store<H>(hid, acc, eg, og, a.acts[0]);
        }
        __syncwarp();
        {
            float2 acc[8][L::JPT / 2];
#pragma unroll
            for(int jp = 0; jp < L::JPT / 2; jp++){
                const float2 b = make_float2(smem[L::B2 + og + 16 * jp], smem[L::B2 + og + 16 * jp + 8]);
#pragma unroll
                for(int ee = 0; ee < 8; ee++) acc[ee][jp] = b;
            }
            l2f_tile_layer<H, H, L::PITCH>(hid, smem + L::W2T, eg, og, acc);
            __syncwarp();                                // every lane has read the first hidden layer before the second overwrites it
            l2f_tile_store<H>(hid, acc, eg, og, a.acts[1]);
        }
        __syncwarp();
        float out[A];
#pragma unroll
        for(int c = 0; c < A; c++) out[c] = smem[L::B3 + c];
#pragma unroll 8
        for(int j = 0; j < H; j++){
            const float h2 = hid[j * L::PITCH + lane];
            const float4 w3 = *reinterpret_cast<const float4*>(smem + L::W3T + j * A);
            out[0] = fmaf(w3.x, h2, out[0]); out[1] = fmaf(w3.y, h2, out[1]); out[2] = fmaf(w3.z, h2, out[2]); out[3] = fmaf(w3.w, h2, out[3]);
        }
        __syncwarp();                                    // the tiles are free for the next step
        if(active){
            float action[A];
#pragma unroll
            for(int c = 0; c < A; c++){ action[c] = activation_rt(out[c], a.acts[2]); a.act[row * A + c] = action[c]; }
            L2fState next;
            l2f_step(a.env, s, action, next);
            const bool term = l2f_terminated(a.mdp, next);
            const float r = l2f_reward(a.env, a.mdp, s, action, next, term);
            es += 1; er = __fadd_rn(er, r);
            trunc = term || (es == a.step_limit);
            a.rew[row] = r;
            if(a.terminated) a.terminated[row] = term ? 1 : 0;
            s = next;
        }
    }
    if(active){
        float* dst = a.states + (size_t)e * 23;
        const float* src = reinterpret_cast<const float*>(&s);
#pragma unroll
        for(int k = 0; k < 23; k++) dst[k] = src[k];
        a.episode_step[e] = es; a.truncated[e] = trunc ? 1 : 0; a.episode_return[e] = er;
    }
}

template <int H>
static int launch_l2f_rollout(const L2fRolloutArgs& a, cudaStream_t s){
    constexpr size_t SMEM = L2fRolloutLayout<H>::BYTES;
    B200RL_CUDA_TRY(cudaFuncSetAttribute(l2f_rollout_kernel<H>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM));
    l2f_rollout_kernel<H><<<(a.n_envs + L2F_ROLLOUT_THREADS - 1) / L2F_ROLLOUT_THREADS, L2F_ROLLOUT_THREADS, SMEM, s>>>(a);
    B200RL_LAUNCH_CHECK("l2f_rollout");
    return B200RL_OK;
}

// ---------------------------------------------------------------------------------------------------------------
// The off-policy runner step on this environment in two halves around ANY policy, like the Pendulum's (the reference's CUDA runner:
// prologue kernel, evaluate(policy), epilogue kernel; rl/components/off_policy_runner/operations_cuda.h:184-204 around
// operations_generic_per_env.h:8-61 and :62-108), with the replay-buffer append of rl/components/replay_buffer/operations_generic.h:54-79:
// row = observation 18 | action 4 | reward | next observation 18 | terminated | truncated.
// ---------------------------------------------------------------------------------------------------------------
template <typename INDEX>
__device__ __forceinline__ void l2f_replay_append(int e, const float (&obs)[18], const float (&action)[4], float reward, const float (&next_obs)[18], bool term, bool trunc,
                                                  bool was_truncated, unsigned char* replay, const b200rl_replay_layout& L){
    constexpr int O = 18, A = 4, COL_REWARD = O + A, COL_NEXT = O + A + 1, COL_TERMINATED = 2 * O + A + 1, COL_TRUNCATED = 2 * O + A + 2;
    unsigned char* rb = replay + (size_t)e * L.env_stride;
    float* data = reinterpret_cast<float*>(rb + L.off_data);
    INDEX* episode_start = reinterpret_cast<INDEX*>(rb + L.off_episode_start);
    INDEX& position_ref = *reinterpret_cast<INDEX*>(rb + L.off_position);
    INDEX& ces_ref = *reinterpret_cast<INDEX*>(rb + L.off_current_episode_start);
    unsigned char& full_ref = *(rb + L.off_full);
    INDEX position = position_ref, ces = ces_ref;
    bool full = full_ref != 0;
    if(was_truncated && (full || position > 0)){               // the environment was reset at the start of this step (operations_generic_per_env.h:41-52)
        const INDEX prev = position == 0 ? (INDEX)(L.capacity - 1) : position - 1;
        data[(size_t)prev * L.ld_data + COL_TRUNCATED] = 1.0f;
        ces = position;
    }
    float* row = data + (size_t)position * L.ld_data;
#pragma unroll
    for(int k = 0; k < O; k++){ row[k] = obs[k]; row[COL_NEXT + k] = next_obs[k]; }
#pragma unroll
    for(int k = 0; k < A; k++) row[O + k] = action[k];
    row[COL_REWARD] = reward; row[COL_TERMINATED] = term ? 1.0f : 0.0f; row[COL_TRUNCATED] = trunc ? 1.0f : 0.0f;
    episode_start[position] = ces;
    position = (position + 1) % (INDEX)L.capacity;
    if(trunc) ces = position;
    if(position == 0 && !full) full = true;
    position_ref = position; ces_ref = ces; full_ref = full ? 1 : 0;
}

// prologue: reset-if-truncated (from reset_states [n, 23], or drawn in the kernel from `init`), counters of a fresh episode, observation
__global__ void __launch_bounds__(128) l2f_offpolicy_prologue_kernel(L2fRolloutArgs a, const unsigned long long* __restrict__ call_counter, float* __restrict__ observations,
                                                                     uint8_t* __restrict__ was_truncated){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= a.n_envs) return;
    L2fState s;
    float* sf = reinterpret_cast<float*>(&s);
#pragma unroll
    for(int k = 0; k < 23; k++) sf[k] = a.states[(size_t)e * 23 + k];
    const bool trunc = a.truncated[e] != 0;
    was_truncated[e] = trunc ? 1 : 0;
    if(trunc){
        if(a.reset_states){
#pragma unroll
            for(int k = 0; k < 23; k++) sf[k] = __ldg(a.reset_states + (size_t)e * 23 + k);
        }
        else{
            float uu[17], nn[6];
            l2f_reset_draws(a.rng_seed, a.rng_step0 + (call_counter ? *call_counter : 0ull), (uint32_t)e, a.init[9] != 0.0f || a.init[11] != 0.0f, uu, nn);
            l2f_initial_state(a.init, a.env.p.action_min, a.env.p.action_max, uu, nn, s);
        }
#pragma unroll
        for(int k = 0; k < 23; k++) a.states[(size_t)e * 23 + k] = sf[k];
        a.episode_step[e] = 0; a.episode_return[e] = 0.0f;
    }
    float o[18];
    l2f_observe(s, o);
#pragma unroll
    for(int k = 0; k < 18; k++) observations[(size_t)e * 18 + k] = o[k];
}
// epilogue: step with the given actions, reward, termination, counters, next observation, replay-buffer append
template <typename INDEX>
__global__ void __launch_bounds__(128) l2f_offpolicy_epilogue_kernel(L2fRolloutArgs a, const float* __restrict__ actions, float* __restrict__ next_observations,
                                                                     const uint8_t* __restrict__ was_truncated, unsigned char* replay, b200rl_replay_layout L){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= a.n_envs) return;
    L2fState s, next;
    float* sf = reinterpret_cast<float*>(&s);
#pragma unroll
    for(int k = 0; k < 23; k++) sf[k] = a.states[(size_t)e * 23 + k];
    float action[4], o[18], no[18];
#pragma unroll
    for(int k = 0; k < 4; k++) action[k] = actions[(size_t)e * 4 + k];
    l2f_observe(s, o);
    l2f_step(a.env, s, action, next);
    const bool term = l2f_terminated(a.mdp, next);
    const float r = l2f_reward(a.env, a.mdp, s, action, next, term);
    const int es = a.episode_step[e] + 1;
    const bool trunc = term || es == a.step_limit;             // operations_generic_per_env.h:93-97
    l2f_observe(next, no);
    const float* nf = reinterpret_cast<const float*>(&next);
#pragma unroll
    for(int k = 0; k < 23; k++) a.states[(size_t)e * 23 + k] = nf[k];
#pragma unroll
    for(int k = 0; k < 18; k++) next_observations[(size_t)e * 18 + k] = no[k];
    a.episode_step[e] = es; a.episode_return[e] = __fadd_rn(a.episode_return[e], r); a.truncated[e] = trunc ? 1 : 0;
    l2f_replay_append<INDEX>(e, o, action, r, no, term, trunc, was_truncated[e] != 0, replay, L);
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

static int l2f_rollout_impl(const b200rl_l2f_parameters* parameters, const float* mdp, const float* init, const b200rl_mlp_shape* actor, const float* actor_params, float* states,
                            int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds, int device_rng,
                            unsigned long long seed, unsigned long long first_step, int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew,
                            uint8_t* terminated, int* error_flag, cudaStream_t stream){
    if(!parameters || !mdp || !actor || (device_rng && !init)) return B200RL_ERR_INVALID_ARGUMENT;
    if(actor->n_layers != 3 || actor->input_dim != 18 || actor->dims[0] != actor->dims[1] || actor->dims[2] != 4) return B200RL_ERR_UNSUPPORTED;
    const int H = actor->dims[0];
    if(H != 16 && H != 32 && H != 64) return B200RL_ERR_UNSUPPORTED;
    for(int l = 0; l < 3; l++) if(!valid_activation(actor->acts[l])) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs < 0 || n_steps < 0 || n_reset_rounds < 0 || step_limit < 1 || (reset_states == nullptr && n_reset_rounds != 0)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0 || n_steps == 0) return B200RL_OK;
    if(!actor_params || !states || !episode_step || !truncated || !episode_return || !obs || !act || !rew) return B200RL_ERR_INVALID_ARGUMENT;
    L2fRolloutArgs a{};
    memcpy(&a.env.p, parameters->dynamics, sizeof(L2fDynamics));
    a.env.dt = parameters->dt; a.env.limit_position = parameters->state_limit_position; a.env.limit_velocity = parameters->state_limit_velocity;
    a.env.limit_angular_velocity = parameters->state_limit_angular_velocity;
    memcpy(a.mdp, mdp, sizeof(a.mdp));
    a.params = actor_params; a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return;
    a.reset_states = reset_states; a.n_reset_rounds = n_reset_rounds; a.n_envs = n_envs; a.n_steps = n_steps; a.step_limit = step_limit;
    a.obs = obs; a.act = act; a.rew = rew; a.terminated = terminated; a.error_flag = error_flag;
    a.device_rng = device_rng; a.rng_seed = seed; a.rng_step0 = first_step;
    if(init) memcpy(a.init, init, sizeof(a.init));
    for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
    if(H == 16) return launch_l2f_rollout<16>(a, stream);
    if(H == 32) return launch_l2f_rollout<32>(a, stream);
    return launch_l2f_rollout<64>(a, stream);
}

extern "C" int b200rl_l2f_rollout(const b200rl_l2f_parameters* parameters, const float* mdp, const b200rl_mlp_shape* actor, const float* actor_params, float* states,
                                  int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int n_reset_rounds, int n_envs, int n_steps,
                                  int step_limit, float* obs, float* act, float* rew, uint8_t* terminated, int* error_flag, b200rl_stream_t stream){
    return l2f_rollout_impl(parameters, mdp, nullptr, actor, actor_params, states, episode_step, truncated, episode_return, reset_states, n_reset_rounds, 0, 0, 0, n_envs, n_steps,
                            step_limit, obs, act, rew, terminated, error_flag, (cudaStream_t)stream);
}

extern "C" int b200rl_l2f_rollout_device_rng(const b200rl_l2f_parameters* parameters, const float* mdp, const float* init, const b200rl_mlp_shape* actor, const float* actor_params,
                                             float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return, unsigned long long seed,
                                             unsigned long long first_step, int n_envs, int n_steps, int step_limit, float* obs, float* act, float* rew, uint8_t* terminated,
                                             b200rl_stream_t stream){
    if(!init) return B200RL_ERR_INVALID_ARGUMENT;
    return l2f_rollout_impl(parameters, mdp, init, actor, actor_params, states, episode_step, truncated, episode_return, nullptr, 0, 1, seed, first_step, n_envs, n_steps,
                            step_limit, obs, act, rew, terminated, nullptr, (cudaStream_t)stream);
}

extern "C" int b200rl_l2f_initial_states_from_draws(const b200rl_l2f_parameters* parameters, const float* init, const float* uniforms, const float* normals, float* states, int n,
                                                    b200rl_stream_t stream){
    if(!parameters || !init || n < 0) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    if(!uniforms || !normals || !states) return B200RL_ERR_INVALID_ARGUMENT;
    L2fRolloutArgs a{};
    memcpy(&a.env.p, parameters->dynamics, sizeof(L2fDynamics));
    memcpy(a.init, init, sizeof(a.init));
    l2f_initial_states_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(a, uniforms, normals, states, n);
    B200RL_LAUNCH_CHECK("l2f_initial_states");
    return B200RL_OK;
}

static void l2f_fill_args(L2fRolloutArgs& a, const b200rl_l2f_parameters* parameters){
    memcpy(&a.env.p, parameters->dynamics, sizeof(L2fDynamics));
    a.env.dt = parameters->dt; a.env.limit_position = parameters->state_limit_position; a.env.limit_velocity = parameters->state_limit_velocity;
    a.env.limit_angular_velocity = parameters->state_limit_angular_velocity;
}

extern "C" int b200rl_l2f_offpolicy_prologue(const b200rl_l2f_parameters* parameters, const float* init, float* states, int32_t* episode_step, const uint8_t* truncated,
                                             float* episode_return, const float* reset_states, unsigned long long seed, unsigned long long call,
                                             const unsigned long long* call_counter, int n_envs, float* observations, uint8_t* was_truncated_scratch, b200rl_stream_t stream){
    if(!parameters || (!init && !reset_states) || !states || !episode_step || !truncated || !episode_return || !observations || !was_truncated_scratch || n_envs < 0)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    L2fRolloutArgs a{};
    l2f_fill_args(a, parameters);
    if(init) memcpy(a.init, init, sizeof(a.init));
    a.states = states; a.episode_step = episode_step; a.truncated = const_cast<uint8_t*>(truncated); a.episode_return = episode_return; a.reset_states = reset_states;
    a.n_envs = n_envs; a.rng_seed = seed; a.rng_step0 = call;
    l2f_offpolicy_prologue_kernel<<<(n_envs + 127) / 128, 128, 0, (cudaStream_t)stream>>>(a, call_counter, observations, was_truncated_scratch);
    B200RL_LAUNCH_CHECK("l2f_offpolicy_prologue");
    return B200RL_OK;
}

extern "C" int b200rl_l2f_offpolicy_epilogue(const b200rl_l2f_parameters* parameters, const float* mdp, float* states, int32_t* episode_step, uint8_t* truncated,
                                             float* episode_return, int n_envs, int step_limit, const float* actions, float* next_observations, void* replay_buffers,
                                             const b200rl_replay_layout* layout, const uint8_t* was_truncated_scratch, b200rl_stream_t stream){
    if(!parameters || !mdp || !states || !episode_step || !truncated || !episode_return || !actions || !next_observations || !replay_buffers || !layout ||
       !was_truncated_scratch || n_envs < 0 || step_limit < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(layout->capacity < 1 || layout->ld_data < 2 * 18 + 4 + 3 || (layout->index_bytes != 4 && layout->index_bytes != 8)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0) return B200RL_OK;
    L2fRolloutArgs a{};
    l2f_fill_args(a, parameters);
    memcpy(a.mdp, mdp, sizeof(a.mdp));
    a.states = states; a.episode_step = episode_step; a.truncated = truncated; a.episode_return = episode_return; a.n_envs = n_envs; a.step_limit = step_limit;
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = (n_envs + 127) / 128;
    if(layout->index_bytes == 4)
        l2f_offpolicy_epilogue_kernel<uint32_t><<<blocks, 128, 0, s>>>(a, actions, next_observations, was_truncated_scratch, static_cast<unsigned char*>(replay_buffers), *layout);
    else
        l2f_offpolicy_epilogue_kernel<unsigned long long><<<blocks, 128, 0, s>>>(a, actions, next_observations, was_truncated_scratch, static_cast<unsigned char*>(replay_buffers), *layout);
    B200RL_LAUNCH_CHECK("l2f_offpolicy_epilogue");
    return B200RL_OK;
}
