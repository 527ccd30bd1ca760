// Observation normalisation: the running normaliser's update (per-column batch mean and standard deviation folded into running values)
// and the standardize layer that applies them. HBM-bound passes over the observation matrix: the update reads it twice (mean, then the
// squared deviations about that mean, as the reference does), the layer reads and writes it once.
#include "common.cuh"

namespace b200rl {

__device__ __forceinline__ double block_sum(double v, double* shared){
    for(int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, n_warps = blockDim.x >> 5;
    __syncthreads();                           // `shared` may still be read from the previous call
    if(lane == 0) shared[warp] = v;
    __syncthreads();
    double total = 0.0;
    for(int w = 0; w < n_warps; w++) total += shared[w];      // the same order in every thread
    return total;
}

// rl/components/running_normalizer/operations_generic.h:27-47 with mean / std of containers/matrix/operations_generic.h:641-650, 674-691.
// One block per column. The reference sums in fp32 in row order; here the sums are taken in double (any order) and rounded to fp32 once,
// which is within the rounding error of the reference's own sum.
__global__ void __launch_bounds__(256) running_normalizer_update_kernel(const float* __restrict__ data, int ld, int rows, int dim, float* __restrict__ mean,
                                                                        float* __restrict__ std, float age){
    __shared__ double shared[8];
    const int c = blockIdx.x;
    double acc = 0.0;
    for(int r = threadIdx.x; r < rows; r += blockDim.x) acc += (double)data[(size_t)r * ld + c];
    const float data_mean = __fdiv_rn((float)block_sum(acc, shared), (float)rows);
    double sq = 0.0;
    for(int r = threadIdx.x; r < rows; r += blockDim.x){
        const float diff = __fsub_rn(data[(size_t)r * ld + c], data_mean);
        sq += (double)__fmul_rn(diff, diff);
    }
    const float sq_f = (float)block_sum(sq, shared);
    if(threadIdx.x == 0){
        const float data_std = sq_f < 1e-6 ? 0.0f : __fsqrt_rn(__fdiv_rn(sq_f, (float)(rows - 1)));
        mean[c] = __fadd_rn(mean[c], __fdiv_rn(__fsub_rn(data_mean, mean[c]), age));
        std[c] = __fadd_rn(std[c], __fdiv_rn(__fsub_rn(data_std, std[c]), age));
    }
}

// nn/layers/standardize/operations_generic.h:52-66
__global__ void standardize_set_statistics_kernel(const float* __restrict__ mean, const float* __restrict__ std, int dim, float* __restrict__ layer_mean,
                                                  float* __restrict__ layer_precision){
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if(c >= dim) return;
    layer_mean[c] = mean[c];
    layer_precision[c] = std[c] == 0.0f ? 0.0f : __fdiv_rn(1.0f, std[c]);
}

// :69-86
__global__ void __launch_bounds__(256) standardize_forward_kernel(const float* __restrict__ x, int ldx, const float* __restrict__ mean, const float* __restrict__ precision,
                                                                  float* __restrict__ y, int ldy, int rows, int dim){
    const size_t n = (size_t)rows * dim, stride = (size_t)gridDim.x * blockDim.x;
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride){
        const size_t r = i / dim; const int c = (int)(i - r * dim);
        float v = __fsub_rn(x[r * ldx + c], __ldg(mean + c));
        const float p = __ldg(precision + c);
        if(p != 0.0f) v = __fmul_rn(v, p);
        y[r * ldy + c] = v;
    }
}

static int grid_for(size_t n, int block){
    int sms = 148;
    size_t blocks = (n + block - 1) / block, cap = (size_t)sms * 8;
    if(blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

}  // namespace b200rl
using namespace b200rl;

extern "C" {

int b200rl_running_normalizer_update(const float* data, int ld, int rows, int dim, float* mean, float* std, unsigned long long age, b200rl_stream_t stream){
    if(!data || !mean || !std || rows < 2 || dim < 1 || ld < dim || age < 1) return B200RL_ERR_INVALID_ARGUMENT;
    running_normalizer_update_kernel<<<dim, 256, 0, (cudaStream_t)stream>>>(data, ld, rows, dim, mean, std, (float)age);
    B200RL_LAUNCH_CHECK("running_normalizer_update");
    return B200RL_OK;
}

int b200rl_standardize_set_statistics(const float* mean, const float* std, int dim, float* layer_mean, float* layer_precision, b200rl_stream_t stream){
    if(!mean || !std || !layer_mean || !layer_precision || dim < 1) return B200RL_ERR_INVALID_ARGUMENT;
    standardize_set_statistics_kernel<<<(dim + 127) / 128, 128, 0, (cudaStream_t)stream>>>(mean, std, dim, layer_mean, layer_precision);
    B200RL_LAUNCH_CHECK("standardize_set_statistics");
    return B200RL_OK;
}

int b200rl_standardize_forward(const float* x, int ldx, const float* mean, const float* precision, float* y, int ldy, int rows, int dim, b200rl_stream_t stream){
    if(!x || !mean || !precision || !y || rows < 0 || dim < 1 || ldx < dim || ldy < dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0) return B200RL_OK;
    standardize_forward_kernel<<<grid_for((size_t)rows * dim, 256), 256, 0, (cudaStream_t)stream>>>(x, ldx, mean, precision, y, ldy, rows, dim);
    B200RL_LAUNCH_CHECK("standardize_forward");
    return B200RL_OK;
}

}
