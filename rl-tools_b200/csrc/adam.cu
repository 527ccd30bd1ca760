// Fused Adam step over a flat parameter arena, MSE gradient, fill. All three are HBM-bandwidth-bound
// element-wise passes: 16-byte vector accesses, grid sized in multiples of the SM count.
#include "common.cuh"

namespace b200rl {

struct AdamState { uint32_t age; uint32_t ticket; float c1; float c2; };

// c = 1 / (1 - beta^age) with the power taken in double and rounded to float once, which reproduces the
// correctly-rounded powf the CPU reference gets from its libm (nn/optimizers/adam/operations_generic.h:49-59).
__device__ __forceinline__ float bias_correction(float beta, uint32_t age){
    float pw = (float)pow((double)beta, (double)(float)age);
    return 1.0f / (1.0f - pw);
}
__device__ __forceinline__ void adam_one(float& p, float g, float& m, float& v, const b200rl_adam_hyper& h, float c1, float c2){
    // utils/polyak/operations_generic.h:72-88 and nn/optimizers/adam/instance/operations_generic.h:25-61, no fused
    // multiply-add so every intermediate rounds like the reference's
    m = __fadd_rn(__fmul_rn(h.beta_1, m), __fmul_rn(1.0f - h.beta_1, g));
    v = __fadd_rn(__fmul_rn(h.beta_2, v), __fmul_rn(__fmul_rn(1.0f - h.beta_2, g), g));
    float pre_sqrt = fmaxf(__fmul_rn(v, c2), h.epsilon_sqrt);
    float update = __fdiv_rn(__fmul_rn(__fmul_rn(h.alpha, c1), m), __fadd_rn(__fsqrt_rn(pre_sqrt), h.epsilon));
    p = __fsub_rn(p, update);
}

__global__ void __launch_bounds__(256) adam_step_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v,
                                                        size_t n, b200rl_adam_hyper h, AdamState* state, int vec_ok){
    __shared__ float sc[2];
    if(threadIdx.x == 0){
        uint32_t age = *reinterpret_cast<volatile uint32_t*>(&state->age);
        sc[0] = bias_correction(h.beta_1, age);
        sc[1] = bias_correction(h.beta_2, age);
    }
    __syncthreads();
    const float c1 = sc[0], c2 = sc[1];
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    if(vec_ok){
        size_t n4 = n / 4;
        float4* p4 = reinterpret_cast<float4*>(p); const float4* g4 = reinterpret_cast<const float4*>(g);
        float4* m4 = reinterpret_cast<float4*>(m); float4* v4 = reinterpret_cast<float4*>(v);
        for(size_t i = tid; i < n4; i += stride){
            float4 pp = p4[i], gg = __ldg(g4 + i), mm = m4[i], vv = v4[i];
            adam_one(pp.x, gg.x, mm.x, vv.x, h, c1, c2); adam_one(pp.y, gg.y, mm.y, vv.y, h, c1, c2);
            adam_one(pp.z, gg.z, mm.z, vv.z, h, c1, c2); adam_one(pp.w, gg.w, mm.w, vv.w, h, c1, c2);
            p4[i] = pp; m4[i] = mm; v4[i] = vv;
        }
        for(size_t i = n4 * 4 + tid; i < n; i += stride) adam_one(p[i], g[i], m[i], v[i], h, c1, c2);
    }
    else{
        for(size_t i = tid; i < n; i += stride) adam_one(p[i], g[i], m[i], v[i], h, c1, c2);
    }
    // the last block to finish publishes c1/c2 and bumps the age: every block has read the old age by then
    __syncthreads();
    if(threadIdx.x == 0){
        __threadfence();
        uint32_t t = atomicAdd(&state->ticket, 1u);
        if(t == gridDim.x - 1){
            state->c1 = c1; state->c2 = c2;
            state->ticket = 0;
            state->age = state->age + 1;
        }
    }
}
__global__ void adam_advance_dev_kernel(const float* hyper9, uint32_t* age, float* c1, float* c2){
    const uint32_t a = *age;
    *c1 = bias_correction(hyper9[1], a);
    *c2 = bias_correction(hyper9[2], a);
    *age = a + 1;
}
__global__ void __launch_bounds__(256) adam_update_dev_kernel(float* __restrict__ p, const float* __restrict__ g, float* __restrict__ m, float* __restrict__ v, size_t n,
                                                              const float* __restrict__ hyper9, const float* __restrict__ c1p, const float* __restrict__ c2p){
    b200rl_adam_hyper h{hyper9[0], hyper9[1], hyper9[2], hyper9[3], hyper9[4]};
    const float c1 = *c1p, c2 = *c2p;
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) adam_one(p[i], g[i], m[i], v[i], h, c1, c2);
}
__global__ void adam_reset_kernel(AdamState* s){ s->age = 1; s->ticket = 0; s->c1 = 0.0f; s->c2 = 0.0f; }

__global__ void __launch_bounds__(256) mse_gradient_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ b, long long ldb, float* d, long long ldd,
                                                           int rows, int cols, float constant){
    long long n = (long long)rows * cols;
    for(long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x){
        long long r = i / cols; int c = (int)(i - r * cols);
        float diff = __fsub_rn(a[r * lda + c], b[r * ldb + c]);
        d[r * ldd + c] = __fmul_rn(diff, constant);
    }
}
// loss = loss_weight * sum (a - b)^2 / (rows * cols): one block, every thread a strided partial sum in double, then a fixed-order tree
// (the reference adds the squares in float in row-major order; the double sum rounded once lies within that sum's own rounding error)
__device__ float g_mse_value;
__global__ void __launch_bounds__(1024) mse_evaluate_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ b, long long ldb, int rows, int cols,
                                                            float loss_weight, float* out){
    __shared__ double part[1024];
    const long long n = (long long)rows * cols;
    double acc = 0.0;
    for(long long i = threadIdx.x; i < n; i += blockDim.x){
        const long long r = i / cols; const int c = (int)(i - r * cols);
        const float diff = __fsub_rn(a[r * lda + c], b[r * ldb + c]);
        acc += (double)__fmul_rn(diff, diff);
    }
    part[threadIdx.x] = acc;
    __syncthreads();
    for(int w = 512; w > 0; w >>= 1){
        if((int)threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w];
        __syncthreads();
    }
    if(threadIdx.x == 0) *out = __fdiv_rn(__fmul_rn((float)part[0], loss_weight), (float)n);     // acc * loss_weight / (ROWS * COLS)
}
__global__ void __launch_bounds__(256) fill_kernel(float* dst, size_t n, float value, int vec_ok){
    const size_t tid = blockIdx.x * (size_t)blockDim.x + threadIdx.x, stride = (size_t)gridDim.x * blockDim.x;
    if(vec_ok){
        size_t n4 = n / 4; float4 v4 = make_float4(value, value, value, value);
        for(size_t i = tid; i < n4; i += stride) reinterpret_cast<float4*>(dst)[i] = v4;
        for(size_t i = n4 * 4 + tid; i < n; i += stride) dst[i] = value;
    }
    else for(size_t i = tid; i < n; i += stride) dst[i] = value;
}

static int grid_for(size_t work_items, int per_block){
    size_t blocks = (work_items + per_block - 1) / per_block;
    size_t cap = (size_t)NUM_SMS * 8;
    if(blocks > cap) blocks = cap;
    if(blocks < 1) blocks = 1;
    return (int)blocks;
}
static bool aligned16(const void* p){ return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Target-network update (utils/polyak/operations_generic.h:10-24, 26-40; CUDA form operations_cuda.h:12-52):
// target = polyak * target + (1 - polyak) * source (source squared in the second form), the two products rounded separately.
template <bool SQUARE>
__global__ void __launch_bounds__(256) polyak_kernel(const float* __restrict__ source, int ld_source, float* __restrict__ target, int ld_target,
                                                     int rows, int cols, float polyak, float one_minus){
    const size_t n = (size_t)rows * cols, stride = (size_t)gridDim.x * blockDim.x;
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += stride){
        const size_t r = i / cols, c = i - r * cols;
        float s = source[r * ld_source + c];
        float* t = target + r * ld_target + c;
        if constexpr(SQUARE) *t = __fadd_rn(__fmul_rn(polyak, *t), __fmul_rn(__fmul_rn(one_minus, s), s));
        else *t = __fadd_rn(__fmul_rn(polyak, *t), __fmul_rn(one_minus, s));
    }
}

// ---- small tensor operations of the SAC update whose operands live in device memory ------------------------------------------------
// mse::gradient with the loss weight read from a one-element device tensor (nn/loss_functions/mse/operations_generic.h:66-79)
__global__ void __launch_bounds__(256) mse_gradient_dev_weight_kernel(const float* __restrict__ a, long long lda, const float* __restrict__ b, long long ldb, float* d,
                                                                      long long ldd, int rows, int cols, const float* __restrict__ loss_weight){
    const float constant = __fmul_rn(__fdiv_rn(2.0f, __fmul_rn((float)rows, (float)cols)), __ldg(loss_weight));
    long long n = (long long)rows * cols;
    for(long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x){
        long long r = i / cols; int c = (int)(i - r * cols);
        d[r * ldd + c] = __fmul_rn(__fsub_rn(a[r * lda + c], b[r * ldb + c]), constant);
    }
}
// cast_reduce_sum<float> of a mask (containers/tensor/operations_generic.h:838-845): the count is an integer, exact in float below 2^24
__global__ void __launch_bounds__(256) mask_count_kernel(const uint8_t* __restrict__ mask, size_t n, float* result){
    __shared__ unsigned int part[256];
    unsigned int count = 0;
    for(size_t i = threadIdx.x; i < n; i += blockDim.x) count += mask[i] != 0;
    part[threadIdx.x] = count;
    __syncthreads();
    for(int w = 128; w > 0; w >>= 1){ if((int)threadIdx.x < w) part[threadIdx.x] += part[threadIdx.x + w]; __syncthreads(); }
    if(threadIdx.x == 0) *result = (float)part[0];
}
// tensor::operations::unary::Scale (containers/tensor/operations_generic.h:433-445): x * scale, or (1 / x) * scale
__global__ void __launch_bounds__(256) scale_kernel(float* t, size_t n, float scale, int reciprocal){
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        t[i] = reciprocal ? __fmul_rn(__fdiv_rn(1.0f, t[i]), scale) : __fmul_rn(t[i], scale);
}
// set_all(tensor, one-element tensor) (containers/tensor/operations_generic.h:741-748)
__global__ void __launch_bounds__(256) fill_from_kernel(float* dst, size_t n, const float* __restrict__ value){
    const float v = __ldg(value);
    for(size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) dst[i] = v;
}
// mask_actions / mask_gradient (rl/algorithms/sac/operations_generic.h:180-232): rows whose mask (optionally inverted) is set receive the
// source row, or zeros when there is no source
__global__ void __launch_bounds__(256) mask_rows_kernel(const float* __restrict__ source, long long ld_source, float* target, long long ld_target,
                                                        const uint8_t* __restrict__ mask, int rows, int cols, int invert){
    long long n = (long long)rows * cols;
    for(long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x){
        long long r = i / cols; int c = (int)(i - r * cols);
        const bool take = (mask[r] != 0) != (invert != 0);
        if(take) target[r * ld_target + c] = source ? source[r * ld_source + c] : 0.0f;
    }
}

}  // namespace b200rl
using namespace b200rl;

extern "C" {

int b200rl_polyak_update(const float* source, int ld_source, float* target, int ld_target, int rows, int cols, float polyak, int square, b200rl_stream_t stream){
    if(!source || !target || rows < 0 || cols < 1 || ld_source < cols || ld_target < cols) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0) return B200RL_OK;
    const int grid = grid_for((size_t)rows * cols, 256);
    if(square) polyak_kernel<true><<<grid, 256, 0, (cudaStream_t)stream>>>(source, ld_source, target, ld_target, rows, cols, polyak, 1.0f - polyak);
    else polyak_kernel<false><<<grid, 256, 0, (cudaStream_t)stream>>>(source, ld_source, target, ld_target, rows, cols, polyak, 1.0f - polyak);
    B200RL_LAUNCH_CHECK("polyak_update");
    return B200RL_OK;
}

int b200rl_adam_reset(uint32_t* state, b200rl_stream_t stream){
    if(!state) return B200RL_ERR_INVALID_ARGUMENT;
    adam_reset_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(reinterpret_cast<AdamState*>(state));
    B200RL_LAUNCH_CHECK("adam_reset");
    return B200RL_OK;
}

int b200rl_adam_step(float* params, const float* grads, float* m, float* v, size_t n, b200rl_adam_hyper hyper, uint32_t* state, b200rl_stream_t stream){
    if(!params || !grads || !m || !v || !state) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    int vec_ok = aligned16(params) && aligned16(grads) && aligned16(m) && aligned16(v);
    int grid = grid_for(vec_ok ? (n + 3) / 4 : n, 256);
    adam_step_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(params, grads, m, v, n, hyper, reinterpret_cast<AdamState*>(state), vec_ok);
    B200RL_LAUNCH_CHECK("adam_step");
    return B200RL_OK;
}

int b200rl_adam_advance_dev(const float* hyper9, uint32_t* age, float* c1, float* c2, b200rl_stream_t stream){
    if(!hyper9 || !age || !c1 || !c2) return B200RL_ERR_INVALID_ARGUMENT;
    adam_advance_dev_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(hyper9, age, c1, c2);
    B200RL_LAUNCH_CHECK("adam_advance_dev");
    return B200RL_OK;
}
int b200rl_adam_update_dev(float* params, const float* grads, float* m, float* v, size_t n, const float* hyper9, const float* c1, const float* c2, b200rl_stream_t stream){
    if(!params || !grads || !m || !v || !hyper9 || !c1 || !c2) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    adam_update_dev_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(params, grads, m, v, n, hyper9, c1, c2);
    B200RL_LAUNCH_CHECK("adam_update_dev");
    return B200RL_OK;
}

int b200rl_mse_gradient(const float* a, int lda, const float* b, int ldb, float* d_a, int ldd, int rows, int cols, float loss_weight, b200rl_stream_t stream){
    if(!a || !b || !d_a || rows < 0 || cols < 1 || lda < cols || ldb < cols || ldd < cols) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0) return B200RL_OK;
    // nn/loss_functions/mse/operations_generic.h:49: (T)2 / ((T)ROWS * COLS) * loss_weight, evaluated in float
    float constant = 2.0f / ((float)rows * (float)cols) * loss_weight;
    mse_gradient_kernel<<<grid_for((size_t)rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(a, lda, b, ldb, d_a, ldd, rows, cols, constant);
    B200RL_LAUNCH_CHECK("mse_gradient");
    return B200RL_OK;
}

int b200rl_mse_evaluate(const float* a, int lda, const float* b, int ldb, int rows, int cols, float loss_weight, float* loss_host, b200rl_stream_t stream){
    if(!a || !b || !loss_host || rows < 1 || cols < 1 || lda < cols || ldb < cols) return B200RL_ERR_INVALID_ARGUMENT;
    float* slot = nullptr;
    B200RL_CUDA_TRY(cudaGetSymbolAddress((void**)&slot, g_mse_value));
    cudaStream_t s = (cudaStream_t)stream;
    mse_evaluate_kernel<<<1, 1024, 0, s>>>(a, lda, b, ldb, rows, cols, loss_weight, slot);
    B200RL_LAUNCH_CHECK("mse_evaluate");
    B200RL_CUDA_TRY(cudaMemcpyAsync(loss_host, slot, sizeof(float), cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaStreamSynchronize(s));
    return B200RL_OK;
}

int b200rl_fill(float* dst, size_t n, float value, b200rl_stream_t stream){
    if(!dst) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    int vec_ok = aligned16(dst);
    fill_kernel<<<grid_for(vec_ok ? (n + 3) / 4 : n, 256), 256, 0, (cudaStream_t)stream>>>(dst, n, value, vec_ok);
    B200RL_LAUNCH_CHECK("fill");
    return B200RL_OK;
}


int b200rl_mse_gradient_dev_weight(const float* a, int lda, const float* b, int ldb, float* d_a, int ldd, int rows, int cols, const float* loss_weight,
                                   b200rl_stream_t stream){
    if(!a || !b || !d_a || !loss_weight || rows < 0 || cols < 1 || lda < cols || ldb < cols || ldd < cols) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0) return B200RL_OK;
    mse_gradient_dev_weight_kernel<<<grid_for((size_t)rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(a, lda, b, ldb, d_a, ldd, rows, cols, loss_weight);
    B200RL_LAUNCH_CHECK("mse_gradient_dev_weight");
    return B200RL_OK;
}
int b200rl_mask_count(const uint8_t* mask, size_t n, float* result, b200rl_stream_t stream){
    if(!result || (n && !mask) || n >= ((size_t)1 << 24)) return B200RL_ERR_INVALID_ARGUMENT;
    mask_count_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(mask, n, result);
    B200RL_LAUNCH_CHECK("mask_count");
    return B200RL_OK;
}
int b200rl_scale(float* t, size_t n, float scale, int reciprocal, b200rl_stream_t stream){
    if(n && !t) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    scale_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(t, n, scale, reciprocal);
    B200RL_LAUNCH_CHECK("scale");
    return B200RL_OK;
}
int b200rl_fill_from_device(float* dst, size_t n, const float* value, b200rl_stream_t stream){
    if(!value || (n && !dst)) return B200RL_ERR_INVALID_ARGUMENT;
    if(n == 0) return B200RL_OK;
    fill_from_kernel<<<grid_for(n, 256), 256, 0, (cudaStream_t)stream>>>(dst, n, value);
    B200RL_LAUNCH_CHECK("fill_from_device");
    return B200RL_OK;
}
int b200rl_mask_rows(const float* source, int ld_source, float* target, int ld_target, const uint8_t* mask, int rows, int cols, int invert, b200rl_stream_t stream){
    if(!target || !mask || rows < 0 || cols < 1 || ld_target < cols || (source && ld_source < cols)) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0) return B200RL_OK;
    mask_rows_kernel<<<grid_for((size_t)rows * cols, 256), 256, 0, (cudaStream_t)stream>>>(source, ld_source, target, ld_target, mask, rows, cols, invert);
    B200RL_LAUNCH_CHECK("mask_rows");
    return B200RL_OK;
}

}
