// PPO update pieces that the reference runs as host scalar loops (rl/algorithms/ppo/operations_generic.h): generalized
// advantage estimation (one backward scan per environment) and the minibatch loss gradient with respect to the actor
// output and log_std (advantage normalisation, clipped surrogate, entropy bonus). All are HBM/latency-bound
// element-wise or scan kernels over columns of the on-policy dataset, addressed with an element pitch so that they work
// directly on the reference's row-major dataset matrix (row = step * N_ENVIRONMENTS + env) as well as on SoA arrays.
#include "common.cuh"

namespace b200rl {

// rl/algorithms/ppo/operations_generic.h:59-95. One thread per environment; consecutive threads read consecutive rows.
__global__ void gae_kernel(const float* __restrict__ rewards, long long ld_r, const float* __restrict__ all_values, long long ld_v,
                           const float* __restrict__ terminated, long long ld_te, const float* __restrict__ truncated, long long ld_tr,
                           float* advantages, long long ld_a, float* target_values, long long ld_t, int n_envs, int steps, float gamma, float lambda, int ignore_termination){
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if(e >= n_envs) return;
    float previous_value = all_values[((long long)steps * n_envs + e) * ld_v];
    float previous_advantage = 0.0f;
    const float lambda_gamma = __fmul_rn(lambda, gamma);
    for(int sb = steps - 1; sb >= 0; sb--){
        const long long pos = (long long)sb * n_envs + e;
        const bool term = terminated[pos * ld_te] != 0.0f, trunc = truncated[pos * ld_tr] != 0.0f;
        const float current = all_values[pos * ld_v];
        const float next = (term && !ignore_termination) ? 0.0f : previous_value;
        float td = __fsub_rn(__fadd_rn(rewards[pos * ld_r], __fmul_rn(gamma, next)), current);
        if(trunc){ if(!term) td = 0.0f; previous_advantage = 0.0f; }
        const float adv = __fadd_rn(__fmul_rn(lambda_gamma, previous_advantage), td);
        advantages[pos * ld_a] = adv;
        target_values[pos * ld_t] = __fadd_rn(adv, current);
        previous_advantage = adv; previous_value = current;
    }
}

// random/operations_generic.h:87-121 with the reference's float/double promotions
struct GaussianTerms { float log_prob, d_mean, d_log_std; };
__device__ __forceinline__ GaussianTerms gaussian_terms(float mean, float log_std, float value){
    const float neg_log_sqrt_pi = (float)(-0.5 * (double)logf(2.0f * 3.14159265358979323846f));
    const float diff = __fsub_rn(value, mean);
    const float std = expf(log_std);
    const float pre_square = __fdiv_rn(diff, std);
    GaussianTerms t;
    // (neg_log_sqrt_pi - log_std) - 0.5 * pre_square^2, which the reference takes in double and rounds to float: here the square is an exact
    // float pair and the difference is rounded to float once (no double-precision instruction: they issue at 1/64 rate on this part and were
    // most of this kernel's time), as in the rollout's Gaussian head
    {
        const float h = __fmul_rn(pre_square, pre_square), l = __fmaf_rn(pre_square, pre_square, -h);          // pre_square^2 = h + l exactly
        const float a = __fsub_rn(neg_log_sqrt_pi, log_std), hh = __fmul_rn(0.5f, h);
        const float d = __fsub_rn(a, hh), db = __fsub_rn(d, a);
        const float de = __fsub_rn(__fsub_rn(a, __fsub_rn(d, db)), __fadd_rn(hh, db));                         // a - hh = d + de exactly
        t.log_prob = __fadd_rn(d, __fmaf_rn(-0.5f, l, de));
    }
    t.d_mean = __fdiv_rn(pre_square, std);
    t.d_log_std = __fadd_rn(-1.0f, __fmul_rn(pre_square, pre_square));
    return t;
}

// the same d_mean and d_log_std without the log-probability (no double-precision instruction)
__device__ __forceinline__ GaussianTerms gaussian_derivatives(float mean, float log_std, float value){
    const float diff = __fsub_rn(value, mean);
    const float std = expf(log_std);
    const float pre_square = __fdiv_rn(diff, std);
    GaussianTerms t;
    t.log_prob = 0.0f;
    t.d_mean = __fdiv_rn(pre_square, std);
    t.d_log_std = __fadd_rn(-1.0f, __fmul_rn(pre_square, pre_square));
    return t;
}

// :173-184: mean and std of the minibatch advantages -> stats[0], stats[1]
__global__ void __launch_bounds__(1024) ppo_adv_stats_kernel(const float* __restrict__ adv, long long ld, int B, float* stats){
    __shared__ float s_sum[32], s_sq[32];
    float sum = 0.0f, sq = 0.0f;
    for(int b = threadIdx.x; b < B; b += blockDim.x){ const float a = adv[b * ld]; sum += a; sq = fmaf(a, a, sq); }
    for(int o = 16; o > 0; o >>= 1){ sum += __shfl_xor_sync(0xffffffffu, sum, o); sq += __shfl_xor_sync(0xffffffffu, sq, o); }
    if((threadIdx.x & 31) == 0){ s_sum[threadIdx.x >> 5] = sum; s_sq[threadIdx.x >> 5] = sq; }
    __syncthreads();
    if(threadIdx.x == 0){
        float ts = 0.0f, tq = 0.0f;
        for(int w = 0; w < (int)(blockDim.x >> 5); w++){ ts += s_sum[w]; tq += s_sq[w]; }
        const float mean = ts / B, msq = tq / B;
        stats[0] = mean; stats[1] = sqrtf(fmaxf(0.0f, msq - mean * mean));
    }
}

struct PpoArgs {
    const float* current_actions; long long ld_cur;
    const float* rollout_actions; long long ld_roll;
    const float* log_std;
    const float* rollout_log_probs; long long ld_lp;
    const float* advantages; long long ld_adv;
    float* d_actions; long long ld_d;
    const float* stats; float* partial;       // partial[block][A]
    int B, A;
    float epsilon_clip, advantage_epsilon; int normalize_advantage, learn_action_std;
};
constexpr int PPO_THREADS = 256, PPO_MAX_ACTION_DIM = 64;

// :214-296, one thread per sample; per-block partial sums of the log_std gradient (warp shuffle + shared memory)
__global__ void __launch_bounds__(PPO_THREADS) ppo_gradient_kernel(PpoArgs a){
    __shared__ float s_part[PPO_MAX_ACTION_DIM][PPO_THREADS / 32];
    const int b = blockIdx.x * PPO_THREADS + threadIdx.x;
    const bool valid = b < a.B;
    float d_loss_d_lp = 0.0f;
    if(valid){
        float action_log_prob = 0.0f;
        for(int i = 0; i < a.A; i++){
            const GaussianTerms t = gaussian_terms(a.current_actions[b * a.ld_cur + i], a.log_std[i], a.rollout_actions[b * a.ld_roll + i]);
            action_log_prob = __fadd_rn(action_log_prob, t.log_prob);
        }
        float advantage = a.advantages[b * a.ld_adv];
        if(a.normalize_advantage) advantage = __fdiv_rn(__fsub_rn(advantage, a.stats[0]), __fadd_rn(a.stats[1], a.advantage_epsilon));
        const float ratio = expf(__fsub_rn(action_log_prob, a.rollout_log_probs[b * a.ld_lp]));
        const float lo = 1.0f - a.epsilon_clip, hi = 1.0f + a.epsilon_clip;
        const float clipped_ratio = ratio < lo ? lo : (ratio > hi ? hi : ratio);
        const bool clipped = ratio != clipped_ratio;
        const bool ratio_min_switch = __fsub_rn(__fmul_rn(ratio, advantage), __fmul_rn(clipped_ratio, advantage)) <= 0.0f;
        const float d_surrogate_d_ratio = ratio_min_switch ? advantage : (clipped ? 0.0f : advantage);
        d_loss_d_lp = __fmul_rn(__fmul_rn(-1.0f / (float)a.B, d_surrogate_d_ratio), ratio);
    }
    // second pass over the actions: only the float terms of the Gaussian (the double-precision log-probability is not needed again); the
    // warps' sums of the log_std gradient meet in shared memory once, after the loop
    for(int i = 0; i < a.A; i++){
        float contrib = 0.0f;
        if(valid){
            const GaussianTerms t = gaussian_derivatives(a.current_actions[b * a.ld_cur + i], a.log_std[i], a.rollout_actions[b * a.ld_roll + i]);
            a.d_actions[b * a.ld_d + i] = __fmul_rn(t.d_mean, d_loss_d_lp);
            contrib = __fmul_rn(d_loss_d_lp, t.d_log_std);
        }
        if(a.learn_action_std){
            for(int o = 16; o > 0; o >>= 1) contrib += __shfl_xor_sync(0xffffffffu, contrib, o);
            if((threadIdx.x & 31) == 0) s_part[i][threadIdx.x >> 5] = contrib;
        }
    }
    if(a.learn_action_std){
        __syncthreads();
        for(int i = threadIdx.x; i < a.A; i += PPO_THREADS){
            float t = 0.0f;
            for(int w = 0; w < PPO_THREADS / 32; w++) t += s_part[i][w];
            a.partial[(long long)blockIdx.x * a.A + i] = t;
        }
    }
}
// d_log_std[i] += sum over blocks (fixed order) + B * (-coefficient / B) (the entropy bonus of every sample, :262-266)
__global__ void ppo_log_std_reduce_kernel(float* d_log_std, const float* __restrict__ partial, int blocks, int A, int B, float entropy_coefficient){
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if(i >= A) return;
    float t = 0.0f;
    for(int k = 0; k < blocks; k++) t += partial[(long long)k * A + i];
    const float d_entropy = -1.0f / (float)B * entropy_coefficient;
    d_log_std[i] += t + (float)B * d_entropy;
}

}  // namespace b200rl
using namespace b200rl;

extern "C" {

int b200rl_gae(const float* rewards, int ld_rewards, const float* all_values, int ld_values, const float* terminated, int ld_terminated,
               const float* truncated, int ld_truncated, float* advantages, int ld_advantages, float* target_values, int ld_targets,
               int n_envs, int steps, float gamma, float lambda, int ignore_termination, b200rl_stream_t stream){
    if(!rewards || !all_values || !terminated || !truncated || !advantages || !target_values || n_envs < 0 || steps < 0 ||
       ld_rewards < 1 || ld_values < 1 || ld_terminated < 1 || ld_truncated < 1 || ld_advantages < 1 || ld_targets < 1) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0 || steps == 0) return B200RL_OK;
    gae_kernel<<<(n_envs + 63) / 64, 64, 0, (cudaStream_t)stream>>>(rewards, ld_rewards, all_values, ld_values, terminated, ld_terminated, truncated, ld_truncated,
                                                                  advantages, ld_advantages, target_values, ld_targets, n_envs, steps, gamma, lambda, ignore_termination);
    B200RL_LAUNCH_CHECK("gae");
    return B200RL_OK;
}

size_t b200rl_ppo_scratch_bytes(int batch, int action_dim){
    if(batch < 1 || action_dim < 1) return 0;
    return sizeof(float) * (2 + (size_t)((batch + PPO_THREADS - 1) / PPO_THREADS) * action_dim);
}

int b200rl_ppo_policy_gradient(const float* current_actions, int ld_current, const float* rollout_actions, int ld_rollout, const float* log_std,
                               const float* rollout_log_probs, int ld_log_probs, const float* advantages, int ld_advantages, float* d_actions, int ld_d,
                               float* d_log_std, int batch, int action_dim, float epsilon_clip, float entropy_coefficient, float advantage_epsilon,
                               int normalize_advantage, int learn_action_std, void* scratch, size_t scratch_bytes, b200rl_stream_t stream){
    if(!current_actions || !rollout_actions || !log_std || !rollout_log_probs || !advantages || !d_actions || batch < 0 || action_dim < 1 ||
       ld_current < action_dim || ld_rollout < action_dim || ld_d < action_dim || ld_log_probs < 1 || ld_advantages < 1) return B200RL_ERR_INVALID_ARGUMENT;
    if(learn_action_std && !d_log_std) return B200RL_ERR_INVALID_ARGUMENT;
    if(action_dim > PPO_MAX_ACTION_DIM) return B200RL_ERR_UNSUPPORTED;
    if(batch == 0) return B200RL_OK;
    if(!scratch || scratch_bytes < b200rl_ppo_scratch_bytes(batch, action_dim)) return B200RL_ERR_INVALID_ARGUMENT;
    cudaStream_t s = (cudaStream_t)stream;
    float* stats = reinterpret_cast<float*>(scratch);
    const int blocks = (batch + PPO_THREADS - 1) / PPO_THREADS;
    if(normalize_advantage){
        ppo_adv_stats_kernel<<<1, 1024, 0, s>>>(advantages, ld_advantages, batch, stats);
        B200RL_LAUNCH_CHECK("ppo_adv_stats");
    }
    PpoArgs a{current_actions, ld_current, rollout_actions, ld_rollout, log_std, rollout_log_probs, ld_log_probs, advantages, ld_advantages, d_actions, ld_d,
              stats, stats + 2, batch, action_dim, epsilon_clip, advantage_epsilon, normalize_advantage, learn_action_std};
    ppo_gradient_kernel<<<blocks, PPO_THREADS, 0, s>>>(a);
    B200RL_LAUNCH_CHECK("ppo_gradient");
    if(learn_action_std){
        ppo_log_std_reduce_kernel<<<1, PPO_MAX_ACTION_DIM, 0, s>>>(d_log_std, stats + 2, blocks, action_dim, batch, entropy_coefficient);
        B200RL_LAUNCH_CHECK("ppo_log_std_reduce");
    }
    return B200RL_OK;
}

}

// ---------------------------------------------------------------------------------------------------------------
// Epoch shuffle: apply a row permutation to selected columns of the dataset matrix (gather into scratch, write back).
// ---------------------------------------------------------------------------------------------------------------
namespace b200rl {
template <bool GATHER>
__global__ void permute_rows_kernel(float* __restrict__ data, int ld, int n_rows, const int32_t* __restrict__ perm, unsigned long long mask, int n_cols,
                                    float* __restrict__ scratch){
    const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if(idx >= (long long)n_rows * n_cols) return;
    const int row = (int)(idx / n_cols), c = (int)(idx % n_cols);
    // column index of the c-th set bit of the mask
    unsigned long long m = mask;
    for(int k = 0; k < c; k++) m &= m - 1;
    const int col = __ffsll((long long)m) - 1;
    if(GATHER) scratch[idx] = data[(size_t)perm[row] * ld + col];
    else data[(size_t)row * ld + col] = scratch[idx];
}
}  // namespace b200rl

extern "C" size_t b200rl_permute_rows_scratch_bytes(int n_rows, unsigned long long column_mask){
    return sizeof(float) * (size_t)(n_rows > 0 ? n_rows : 0) * (size_t)__builtin_popcountll(column_mask);
}

extern "C" int b200rl_permute_rows(float* data, int ld, int n_rows, const int32_t* perm, unsigned long long column_mask, void* scratch, size_t scratch_bytes,
                                   b200rl_stream_t stream){
    const int n_cols = __builtin_popcountll(column_mask);
    if(!data || !perm || n_rows < 0 || ld < 1 || (ld < 64 && (column_mask >> ld) != 0)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n_rows == 0 || n_cols == 0) return B200RL_OK;
    if(!scratch || scratch_bytes < b200rl_permute_rows_scratch_bytes(n_rows, column_mask)) return B200RL_ERR_INVALID_ARGUMENT;
    const long long total = (long long)n_rows * n_cols;
    const int threads = 256;
    const unsigned blocks = (unsigned)((total + threads - 1) / threads);
    cudaStream_t s = (cudaStream_t)stream;
    b200rl::permute_rows_kernel<true><<<blocks, threads, 0, s>>>(data, ld, n_rows, perm, column_mask, n_cols, static_cast<float*>(scratch));
    b200rl::permute_rows_kernel<false><<<blocks, threads, 0, s>>>(data, ld, n_rows, perm, column_mask, n_cols, static_cast<float*>(scratch));
    B200RL_LAUNCH_CHECK("permute_rows");
    return B200RL_OK;
}
