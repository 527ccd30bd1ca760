// SAC update pieces that are not dense layers: the sample-and-squash policy head (forward with external noise, backward with the
// entropy term and the log_alpha gradient), the critic target and the actor's choice between the two critics' input gradients.
// All are per-sample element-wise passes over a minibatch (a few hundred rows): latency-bound launches, one thread per sample.
// The transcendental functions are evaluated in double and rounded once: the host libm's expf and logf, which the reference computes
// with, are correctly rounded, its tanhf is within one ulp of that.
#include "common.cuh"

namespace b200rl {

constexpr float SAS_LOG_STD_LOW = -20.0f, SAS_LOG_STD_HIGH = 2.0f, SAS_EPS = 1e-6f;      // nn/layers/sample_and_squash/layer.h:27-36

__device__ __forceinline__ float exp_once(float x){ return (float)exp((double)x); }
__device__ __forceinline__ float log_once(float x){ return (float)log((double)x); }
__device__ __forceinline__ float tanh_once(float x){ return (float)tanh((double)x); }
__device__ __forceinline__ float clampf(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }

// random/operations_generic.h:87-120 with the reference's promotions: the -0.5 factors are double literals
struct NormalTerms {
    float log_prob, d_mean, d_log_std, d_sample;
    __device__ __forceinline__ NormalTerms(float mean, float log_std, float value, float neg_half_log_2pi){
        const float diff = __fsub_rn(value, mean), std = exp_once(log_std), pre_square = __fdiv_rn(diff, std);
        const double sq = __dmul_rn(__dmul_rn(0.5, (double)pre_square), (double)pre_square);
        log_prob = (float)__dsub_rn((double)__fsub_rn(neg_half_log_2pi, log_std), sq);
        d_mean = __fdiv_rn(pre_square, std);
        d_log_std = __fadd_rn(-1.0f, __fmul_rn(pre_square, pre_square));
        d_sample = __fdiv_rn(-pre_square, std);
    }
};

// forward_per_sample (nn/layers/sample_and_squash/operations_generic.h:212-260) and evaluate_per_sample (:149-195), external noise
__global__ void sas_forward_kernel(const float* __restrict__ input, int ld_in, const float* __restrict__ noise, int ld_noise, int B, int A,
                                   float* __restrict__ pre_squashing, float* __restrict__ output, int ld_out, float* __restrict__ log_probs,
                                   float neg_half_log_2pi){
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if(b >= B) return;
    float log_prob = 0.0f;
    for(int a = 0; a < A; a++){
        const float mean = input[(size_t)b * ld_in + a];
        const float log_std = clampf(input[(size_t)b * ld_in + A + a], SAS_LOG_STD_LOW, SAS_LOG_STD_HIGH);
        const float std = exp_once(log_std);
        const float sample = __fadd_rn(mean, __fmul_rn(noise[(size_t)b * ld_noise + a], std));
        const float squashed = tanh_once(sample);
        if(pre_squashing) pre_squashing[(size_t)b * A + a] = sample;
        output[(size_t)b * ld_out + a] = squashed;
        const float one_minus = __fadd_rn(__fsub_rn(1.0f, __fmul_rn(squashed, squashed)), SAS_EPS);
        const NormalTerms n(mean, log_std, sample, neg_half_log_2pi);
        log_prob = __fadd_rn(log_prob, __fsub_rn(n.log_prob, log_once(one_minus)));
    }
    if(log_probs) log_probs[b] = log_prob;
}

// backward_full_per_sample (:290-357)
__global__ void sas_backward_kernel(const float* __restrict__ input, int ld_in, const float* __restrict__ noise, int ld_noise, const float* __restrict__ pre_squashing,
                                    const float* __restrict__ output, int ld_out, const float* __restrict__ d_output, int ld_dout, const float* __restrict__ log_alpha,
                                    float target_entropy, int B, int A, float* __restrict__ d_input, int ld_din, float* __restrict__ d_log_alpha_per_sample,
                                    float neg_half_log_2pi){
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if(b >= B) return;
    const float alpha = exp_once(__ldg(log_alpha));
    const float alpha_over_batch = __fdiv_rn(alpha, (float)B);
    float entropy = 0.0f;
    for(int a = 0; a < A; a++){
        const float action = output[(size_t)b * ld_out + a];
        const float d_tanh = __fmul_rn(d_output[(size_t)b * ld_dout + a], __fsub_rn(1.0f, __fmul_rn(action, action)));
        const float nz = noise[(size_t)b * ld_noise + a];
        const float d_std = __fmul_rn(d_tanh, nz);
        const float log_std_raw = input[(size_t)b * ld_in + A + a];
        const float log_std = clampf(log_std_raw, SAS_LOG_STD_LOW, SAS_LOG_STD_HIGH);
        const float std = exp_once(log_std);
        const float mu = input[(size_t)b * ld_in + a];
        const float sample = pre_squashing[(size_t)b * A + a];
        const NormalTerms n(mu, log_std, sample, neg_half_log_2pi);
        const float two_action = __fmul_rn(2.0f, action);
        const float d_mu = __fadd_rn(d_tanh, __fmul_rn(alpha_over_batch, __fadd_rn(__fadd_rn(n.d_mean, n.d_sample), two_action)));
        const float inner = __fadd_rn(__fadd_rn(n.d_log_std, __fmul_rn(__fmul_rn(n.d_sample, nz), std)), __fmul_rn(__fmul_rn(two_action, nz), std));
        const float d_log_std_clamped = __fadd_rn(__fmul_rn(std, d_std), __fmul_rn(alpha_over_batch, inner));
        d_input[(size_t)b * ld_din + a] = d_mu;
        d_input[(size_t)b * ld_din + A + a] = (log_std_raw < SAS_LOG_STD_LOW || log_std_raw > SAS_LOG_STD_HIGH) ? 0.0f : d_log_std_clamped;
        const float one_minus = __fadd_rn(__fsub_rn(1.0f, __fmul_rn(action, action)), SAS_EPS);
        entropy = __fadd_rn(entropy, -__fsub_rn(n.log_prob, log_once(one_minus)));
    }
    d_log_alpha_per_sample[b] = __fmul_rn(alpha, __fsub_rn(entropy, target_entropy));
}

// backward_full (:384-397): the per-sample terms summed in sample order (one warp: coalesced loads, lane 0 adds in order), divided by the
// batch size (the number of resets at sequence length 1) and added to the gradient
__global__ void sas_log_alpha_gradient_kernel(const float* __restrict__ per_sample, int B, float* __restrict__ gradient){
    const int lane = threadIdx.x;
    float acc = 0.0f;
    for(int base = 0; base < B; base += 32){
        const float v = base + lane < B ? per_sample[base + lane] : 0.0f;
        const int n = min(32, B - base);
        for(int i = 0; i < n; i++){
            const float x = __shfl_sync(0xffffffffu, v, i);
            acc = __fadd_rn(acc, x);
        }
    }
    if(lane == 0) *gradient = __fadd_rn(*gradient, __fdiv_rn(acc, (float)B));
}

// target_action_values_per_sample (rl/algorithms/sac/operations_generic.h:133-163)
__global__ void sac_target_kernel(const float* __restrict__ q1, int ld_q1, const float* __restrict__ q2, int ld_q2, const float* __restrict__ rewards,
                                  const uint8_t* __restrict__ terminated, const float* __restrict__ next_log_probs, const float* __restrict__ log_alpha,
                                  float gamma, int ignore_termination, int entropy_bonus, int entropy_bonus_next_step, float* __restrict__ target,
                                  int ld_target, int B){
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if(b >= B) return;
    const float alpha = exp_once(__ldg(log_alpha));
    float min_next = fminf(q1[(size_t)b * ld_q1], q2[(size_t)b * ld_q2]);
    const float bonus = __fmul_rn(-alpha, next_log_probs[b]);
    if(entropy_bonus && entropy_bonus_next_step) min_next = __fadd_rn(min_next, bonus);
    const float future = (ignore_termination || !terminated[b]) ? __fmul_rn(gamma, min_next) : 0.0f;
    float value = __fadd_rn(rewards[b], future);
    if(entropy_bonus && !entropy_bonus_next_step) value = __fadd_rn(value, bonus);
    target[(size_t)b * ld_target] = value;
}

// min_value_d_output_per_sample (:341-365): the action part of the input gradient of whichever critic has the smaller value
__global__ void sac_min_value_kernel(const float* __restrict__ q1, int ld_q1, const float* __restrict__ q2, int ld_q2, const float* __restrict__ d_in_1,
                                     const float* __restrict__ d_in_2, int ld_d_in, int action_offset, int A, float* __restrict__ d_actor_output, int ld_out, int B){
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if(i >= B * A) return;
    const int b = i / A, a = i - b * A;
    const bool first = q1[(size_t)b * ld_q1] < q2[(size_t)b * ld_q2];
    d_actor_output[(size_t)b * ld_out + a] = (first ? d_in_1 : d_in_2)[(size_t)b * ld_d_in + action_offset + a];
}

static float neg_half_log_2pi_host(){ return (float)(-0.5 * logf(2 * 3.14159265358979323846f)); }      // random/operations_generic.h:89, on the host's libm

}  // namespace b200rl
using namespace b200rl;

extern "C" {

int b200rl_sample_and_squash_forward(const float* input, int ld_in, const float* noise, int ld_noise, int batch, int action_dim, float* pre_squashing,
                                     float* output, int ld_out, float* log_probs, b200rl_stream_t stream){
    if(!input || !noise || !output || batch < 0 || action_dim < 1 || ld_in < 2 * action_dim || ld_noise < action_dim || ld_out < action_dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    sas_forward_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(input, ld_in, noise, ld_noise, batch, action_dim, pre_squashing, output, ld_out, log_probs,
                                                                           neg_half_log_2pi_host());
    B200RL_LAUNCH_CHECK("sample_and_squash_forward");
    return B200RL_OK;
}

int b200rl_sample_and_squash_backward(const float* input, int ld_in, const float* noise, int ld_noise, const float* pre_squashing, const float* output, int ld_out,
                                      const float* d_output, int ld_dout, const float* log_alpha, float target_entropy, int batch, int action_dim, float* d_input,
                                      int ld_din, float* d_log_alpha_per_sample, float* log_alpha_gradient, b200rl_stream_t stream){
    if(!input || !noise || !pre_squashing || !output || !d_output || !log_alpha || !d_input || !d_log_alpha_per_sample || batch < 0 || action_dim < 1 ||
       ld_in < 2 * action_dim || ld_noise < action_dim || ld_out < action_dim || ld_dout < action_dim || ld_din < 2 * action_dim)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    cudaStream_t s = (cudaStream_t)stream;
    sas_backward_kernel<<<(batch + 127) / 128, 128, 0, s>>>(input, ld_in, noise, ld_noise, pre_squashing, output, ld_out, d_output, ld_dout, log_alpha, target_entropy,
                                                            batch, action_dim, d_input, ld_din, d_log_alpha_per_sample, neg_half_log_2pi_host());
    B200RL_LAUNCH_CHECK("sample_and_squash_backward");
    if(log_alpha_gradient){
        sas_log_alpha_gradient_kernel<<<1, 32, 0, s>>>(d_log_alpha_per_sample, batch, log_alpha_gradient);
        B200RL_LAUNCH_CHECK("sample_and_squash_log_alpha_gradient");
    }
    return B200RL_OK;
}

int b200rl_sac_target_action_values(const float* q1_next, int ld_q1, const float* q2_next, int ld_q2, const float* rewards, const uint8_t* terminated,
                                    const float* next_log_probs, const float* log_alpha, float gamma, int ignore_termination, int entropy_bonus,
                                    int entropy_bonus_next_step, float* target, int ld_target, int batch, b200rl_stream_t stream){
    if(!q1_next || !q2_next || !rewards || !terminated || !next_log_probs || !log_alpha || !target || batch < 0 || ld_q1 < 1 || ld_q2 < 1 || ld_target < 1)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    sac_target_kernel<<<(batch + 127) / 128, 128, 0, (cudaStream_t)stream>>>(q1_next, ld_q1, q2_next, ld_q2, rewards, terminated, next_log_probs, log_alpha, gamma,
                                                                          ignore_termination, entropy_bonus, entropy_bonus_next_step, target, ld_target, batch);
    B200RL_LAUNCH_CHECK("sac_target_action_values");
    return B200RL_OK;
}

int b200rl_sac_min_value_d_output(const float* q1, int ld_q1, const float* q2, int ld_q2, const float* d_critic_1_input, const float* d_critic_2_input, int ld_d_input,
                                  int action_offset, int action_dim, float* d_actor_output, int ld_out, int batch, b200rl_stream_t stream){
    if(!q1 || !q2 || !d_critic_1_input || !d_critic_2_input || !d_actor_output || batch < 0 || action_dim < 1 || action_offset < 0 || ld_q1 < 1 || ld_q2 < 1 ||
       ld_d_input < action_offset + action_dim || ld_out < action_dim)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    const int n = batch * action_dim;
    sac_min_value_kernel<<<(n + 127) / 128, 128, 0, (cudaStream_t)stream>>>(q1, ld_q1, q2, ld_q2, d_critic_1_input, d_critic_2_input, ld_d_input, action_offset, action_dim,
                                                                         d_actor_output, ld_out, batch);
    B200RL_LAUNCH_CHECK("sac_min_value_d_output");
    return B200RL_OK;
}

}
