// Whole-network kernels for SMALL networks at SMALL batches: one launch per forward pass, two per backward pass (the input-gradient chain,
// then all parameter gradients), instead of 1 / 3-5 launches per LAYER. For the actor / PPO shapes of the reference (3 -> 64 -> 64 -> 2 at
// batch 256, 27 -> 64 -> 64 -> 8 at minibatch 2048) a layer's arithmetic takes well under a microsecond; a pass through the per-layer kernels is
// then a chain of dependent launches of ~2.5 us each, and the chain, not the arithmetic, is what a step costs. Replaces, for these shapes,
// the per-layer recursion of nn_models/mlp/operations_generic.h:77-217 over nn/layers/dense/operations_cuda.h:236-446 (per layer:
// set_biases kernel, cublasSgemm, activation kernel; backward: d_activation + bias-gradient kernel and two cublasSgemm).
//
// Work split: a CTA owns ROWS consecutive batch rows and walks the layers with the activations (or the back-propagated gradient) of its
// rows in shared memory. ALL parameters of the network are brought into shared memory in one burst at the start of the kernel (one L2 round
// trip for the whole pass instead of one per layer), which is what limits the path to networks of at most FUSED_MAX_PARAMS weights: every
// CTA reads every weight, a few MB of L2 traffic per pass for the eligible shapes. Wider networks (the 256-wide SAC critic is 67 K
// weights, and 128 CTAs x 256 KB per layer would be 32 MB of L2 reads) stay on the per-layer kernels, which tile the weights over CTAs.
// Thread t owns output units t and t + 128 of every layer. Forward reads the weight row of its unit as float4; the rows lie at a pitch of
// an odd number of float4, so that the rows of consecutive threads start in different banks. The backward chain reads W[o][i] with i across
// the threads, which the arena's own row-major layout serves without conflicts.
// Parameter gradients are sums over the batch: 32 x 32 tiles of dW over all layers in one grid, the batch split over CTAs in slices of
// 256 rows whose partial tiles the last-arriving CTA of a tile adds up in slice order (deterministic; the arrival counters live in the
// caller's scratch and are zeroed by the chain kernel that runs before).
#include "common.cuh"
#include <atomic>

namespace b200rl {

constexpr int FUSED_MAX_WIDTH = 256;        // every layer width and the input width
constexpr int FUSED_MAX_PARAMS = 40000;     // padded weights + biases of the whole network, in floats (160 KB of shared memory)
constexpr int FUSED_THREADS = 128;
constexpr int FUSED_SLICE = 256;            // batch rows per gradient slice

// asynchronous global -> shared copies (no staging registers: a thread can have all of its copies of all layers in flight at once)
__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem){
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_4(void* smem, const void* gmem){
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" :: "r"((uint32_t)__cvta_generic_to_shared(smem)), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all(){ asm volatile("cp.async.commit_group;\ncp.async.wait_group 0;" ::: "memory"); }

// pitch of a weight row in shared memory, in float4: the row length rounded up to four inputs, made odd
__host__ __device__ inline int fused_pitch4(int input_dim){ const int q = (input_dim + 3) >> 2; return q | 1; }

struct FusedShape {
    int n_layers, input_dim, batch;
    int dims[B200RL_MAX_LAYERS], acts[B200RL_MAX_LAYERS];
    long long poff[B200RL_MAX_LAYERS];      // offset of W_l in the parameter arena (bias follows the weights)
    long long aoff[B200RL_MAX_LAYERS];      // offset of layer l in the per-layer activation arenas [batch, dims[l]]
    int woff[B200RL_MAX_LAYERS];            // forward kernel: offset of layer l's interleaved weights in shared memory (floats)
    int boff[B200RL_MAX_LAYERS];            // forward kernel: offset of layer l's bias in shared memory
    int smem_params;                        // forward kernel: floats of shared memory taken by the parameters
    int n_params;                           // parameters of the network (arena length)
    int tile_begin[B200RL_MAX_LAYERS + 1];  // gradient tiles: prefix sums over layers of ceil(O / 32) * ceil((I + 1) / 32)
};

// ---------------------------------------------------------------------------------------------------------------------------------------
// forward / evaluate: y_l = act_l(b_l + W_l y_{l-1}), bias first and inputs in ascending order as the reference sums them
// ---------------------------------------------------------------------------------------------------------------------------------------
template <int ROWS, bool SAVE>
__global__ void __launch_bounds__(FUSED_THREADS) mlp_fused_forward_kernel(FusedShape sh, const float* __restrict__ params, const float* __restrict__ x, long long ldx,
                                                                          float* __restrict__ pre, float* __restrict__ out, float* __restrict__ y, long long ldy){
    extern __shared__ __align__(16) float fused_smem[];
    float* s_par = fused_smem;
    float (*act)[ROWS][FUSED_MAX_WIDTH] = reinterpret_cast<float (*)[ROWS][FUSED_MAX_WIDTH]>(fused_smem + sh.smem_params);
    const int tid = threadIdx.x;
    const long long row0 = (long long)blockIdx.x * ROWS;
    // all parameters in one burst of asynchronous copies (about one L2 round trip for the whole network): every weight row into shared
    // memory at a pitch of an ODD number of float4 (rows of consecutive units then start in different banks: thread t reads float4 k4 of
    // row t without conflicts), zero-padded to a multiple of four inputs; biases behind; then the rows of the input.
    {
        int I = sh.input_dim;
        for(int l = 0; l < sh.n_layers; l++){
            const int O = sh.dims[l], I4 = (I + 3) & ~3, S4 = fused_pitch4(I);
            const float* W = params + sh.poff[l];
            float* sw = s_par + sh.woff[l];
            if((I & 3) == 0 && (reinterpret_cast<uintptr_t>(W) & 15u) == 0){
                const int q = I >> 2, n4 = O * q;
                for(int i4 = tid; i4 < n4; i4 += FUSED_THREADS){ const int o = i4 / q; cp_async_16(reinterpret_cast<float4*>(sw) + o * S4 + (i4 - o * q), reinterpret_cast<const float4*>(W) + i4); }
            }
            else{
                for(int idx = tid; idx < O * (I4 - I); idx += FUSED_THREADS){ const int o = idx / (I4 - I); sw[o * S4 * 4 + I + idx % (I4 - I)] = 0.0f; }
                for(int i = tid; i < O * I; i += FUSED_THREADS){ const int o = i / I; cp_async_4(sw + o * S4 * 4 + (i - o * I), W + i); }
            }
            for(int o = tid; o < O; o += FUSED_THREADS) cp_async_4(s_par + sh.boff[l] + o, W + (long long)O * I + o);
            I = O;
        }
        const int I4 = (sh.input_dim + 3) & ~3;
        for(int idx = tid; idx < ROWS * I4; idx += FUSED_THREADS){
            const int r = idx / I4, k = idx - r * I4;
            if(k < sh.input_dim && row0 + r < sh.batch) cp_async_4(&act[0][r][k], x + (row0 + r) * ldx + k);
            else act[0][r][k] = 0.0f;
        }
        cp_async_wait_all();
    }
    __syncthreads();
    int cur = 0, I = sh.input_dim;
    for(int l = 0; l < sh.n_layers; l++){
        const int O = sh.dims[l], a = sh.acts[l], I4 = (I + 3) & ~3, O4 = (O + 3) & ~3, S4 = fused_pitch4(I);
        const float* sw = s_par + sh.woff[l];
        const float* sb = s_par + sh.boff[l];
        const bool last = l == sh.n_layers - 1;
        const int o0 = tid, o1 = tid + FUSED_THREADS;
        const bool has0 = o0 < O, has1 = o1 < O;
        float acc0[ROWS], acc1[ROWS];
#pragma unroll
        for(int r = 0; r < ROWS; r++){ acc0[r] = has0 ? sb[o0] : 0.0f; acc1[r] = has1 ? sb[o1] : 0.0f; }
        if(has0){
            const float4* wa = reinterpret_cast<const float4*>(sw) + o0 * S4;
            const float4* wb = reinterpret_cast<const float4*>(sw) + (has1 ? o1 : o0) * S4;
#pragma unroll 4
            for(int k4 = 0; k4 < I4 / 4; k4++){
                const float4 a4 = wa[k4], b4 = wb[k4];
#pragma unroll
                for(int r = 0; r < ROWS; r++){
                    const float4 v = *reinterpret_cast<const float4*>(&act[cur][r][k4 * 4]);
                    acc0[r] = fmaf(a4.x, v.x, acc0[r]); acc0[r] = fmaf(a4.y, v.y, acc0[r]); acc0[r] = fmaf(a4.z, v.z, acc0[r]); acc0[r] = fmaf(a4.w, v.w, acc0[r]);
                    acc1[r] = fmaf(b4.x, v.x, acc1[r]); acc1[r] = fmaf(b4.y, v.y, acc1[r]); acc1[r] = fmaf(b4.z, v.z, acc1[r]); acc1[r] = fmaf(b4.w, v.w, acc1[r]);
                }
            }
        }
        const int nxt = cur ^ 1;
#pragma unroll
        for(int h = 0; h < 2; h++){
            const int o = h ? o1 : o0;
            if(o < O){
#pragma unroll
                for(int r = 0; r < ROWS; r++){
                    const float p = h ? acc1[r] : acc0[r];
                    const float v = activation_rt(p, a);
                    act[nxt][r][o] = v;
                    if(row0 + r < sh.batch){
                        if(SAVE){ pre[sh.aoff[l] + (row0 + r) * O + o] = p; out[sh.aoff[l] + (row0 + r) * O + o] = v; }
                        else if(last) y[(row0 + r) * ldy + o] = v;
                    }
                }
            }
            else if(o < O4){                                       // the zero padding the next layer's float4 reads run into
#pragma unroll
                for(int r = 0; r < ROWS; r++) act[nxt][r][o] = 0.0f;
            }
        }
        __syncthreads();
        cur = nxt; I = O;
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// backward, part 1: d_pre_l = act_l'(pre_l) * d_out_l and d_out_{l-1} = d_pre_l W_l down the layers. d_pre of every layer goes to `dpre`
// (per-layer arena layout); the last layer's is also written back into d_out, as the per-layer path does. d_input may be NULL.
// ---------------------------------------------------------------------------------------------------------------------------------------
template <int ROWS>
__global__ void __launch_bounds__(FUSED_THREADS) mlp_fused_backward_chain_kernel(FusedShape sh, const float* __restrict__ params, const float* __restrict__ pre,
                                                                                 float* d_out, long long ldd, float* __restrict__ dpre, float* d_input, long long ldi,
                                                                                 unsigned int* counters, int n_counters){
    extern __shared__ __align__(16) float fused_smem[];
    float* s_par = fused_smem;                                   // the parameter arena as it is: W_l row-major, b_l behind
    float (*d)[ROWS][FUSED_MAX_WIDTH] = reinterpret_cast<float (*)[ROWS][FUSED_MAX_WIDTH]>(fused_smem + ((sh.n_params + 3) & ~3));
    const int tid = threadIdx.x;
    const long long row0 = (long long)blockIdx.x * ROWS;
    if(counters) for(int i = blockIdx.x * FUSED_THREADS + tid; i < n_counters; i += gridDim.x * FUSED_THREADS) counters[i] = 0u;
    if((reinterpret_cast<uintptr_t>(params) & 15u) == 0){
        const int n4 = sh.n_params >> 2;
        for(int i = tid; i < n4; i += FUSED_THREADS) cp_async_16(reinterpret_cast<float4*>(s_par) + i, reinterpret_cast<const float4*>(params) + i);
        for(int i = (n4 << 2) + tid; i < sh.n_params; i += FUSED_THREADS) cp_async_4(s_par + i, params + i);
    }
    else{
        for(int i = tid; i < sh.n_params; i += FUSED_THREADS) cp_async_4(s_par + i, params + i);
    }
    const int L = sh.n_layers;
    {
        const int O = sh.dims[L - 1];
        for(int idx = tid; idx < ROWS * O; idx += FUSED_THREADS){
            const int r = idx / O, o = idx - r * O;
            d[0][r][o] = row0 + r < sh.batch ? d_out[(row0 + r) * ldd + o] : 0.0f;
        }
    }
    cp_async_wait_all();
    __syncthreads();
    int cur = 0;
    for(int l = L - 1; l >= 0; l--){
        const int O = sh.dims[l], I = l ? sh.dims[l - 1] : sh.input_dim, a = sh.acts[l];
        for(int idx = tid; idx < ROWS * O; idx += FUSED_THREADS){
            const int r = idx / O, o = idx - r * O;
            float v = 0.0f;
            if(row0 + r < sh.batch){
                v = d_activation_rt(pre[sh.aoff[l] + (row0 + r) * O + o], a) * d[cur][r][o];
                dpre[sh.aoff[l] + (row0 + r) * O + o] = v;
                if(l == L - 1) d_out[(row0 + r) * ldd + o] = v;
            }
            d[cur][r][o] = v;
        }
        __syncthreads();
        if(l == 0 && !d_input) break;
        const float* W = s_par + sh.poff[l];
        const int i0 = tid, i1 = tid + FUSED_THREADS;
        float acc0[ROWS], acc1[ROWS];
#pragma unroll
        for(int r = 0; r < ROWS; r++){ acc0[r] = 0.0f; acc1[r] = 0.0f; }
        if(i0 < I){
            const float* w0 = W + i0;
            const float* w1 = W + (i1 < I ? i1 : i0);
#pragma unroll 4
            for(int o = 0; o < O; o++){
                const float wa = w0[o * I], wb = w1[o * I];
#pragma unroll
                for(int r = 0; r < ROWS; r++){ const float v = d[cur][r][o]; acc0[r] = fmaf(v, wa, acc0[r]); acc1[r] = fmaf(v, wb, acc1[r]); }
            }
        }
        const int nxt = cur ^ 1;
#pragma unroll
        for(int h = 0; h < 2; h++){
            const int i = h ? i1 : i0;
            if(i < I){
#pragma unroll
                for(int r = 0; r < ROWS; r++){
                    const float v = h ? acc1[r] : acc0[r];
                    d[nxt][r][i] = v;
                    if(l == 0 && row0 + r < sh.batch) d_input[(row0 + r) * ldi + i] = v;
                }
            }
        }
        __syncthreads();
        cur = nxt;
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// backward, part 2: dW_l += d_pre_l^T in_l and db_l += column sums of d_pre_l, all layers in one grid. A tile is 32 outputs x 32 columns
// of the row-extended matrix [in_l | 1] (the column of ones yields the bias gradient); blockIdx.y is the batch slice.
// A CTA brings 128 rows of both operands into shared memory per round (16 loads in flight per thread and operand: two L2 round trips per
// 256-row slice instead of eight), its eight warps take interleaved rows with a 4 x 8 patch of the tile per lane (three 16-byte
// shared-memory loads per 32 multiply-adds), and the eight partial tiles are added in warp order.
// ---------------------------------------------------------------------------------------------------------------------------------------
constexpr int GRADS_ROWS = 128, GRADS_PITCH = 36;
__global__ void __launch_bounds__(256) mlp_fused_grads_kernel(FusedShape sh, const float* __restrict__ x, long long ldx, const float* __restrict__ outs,
                                                              const float* __restrict__ dpre, float* grads, float* partial, unsigned int* counters, int n_slices){
    __shared__ __align__(16) float s_all[2 * GRADS_ROWS * GRADS_PITCH];          // d_pre rows, then input rows; the eight partial tiles reuse it
    __shared__ bool is_last;
    float (*s_d)[GRADS_PITCH] = reinterpret_cast<float (*)[GRADS_PITCH]>(s_all);
    float (*s_in)[GRADS_PITCH] = s_d + GRADS_ROWS;
    static_assert(8 * 32 * 32 <= 2 * GRADS_ROWS * GRADS_PITCH, "partial tiles");
    const int tile = blockIdx.x, slice = blockIdx.y;
    int l = 0;
    while(l + 1 < sh.n_layers && tile >= sh.tile_begin[l + 1]) l++;
    const int O = sh.dims[l], I = l ? sh.dims[l - 1] : sh.input_dim;
    const int tiles_i = (I + 1 + 31) / 32;
    const int local = tile - sh.tile_begin[l];
    const int o_base = (local / tiles_i) * 32, i_base = (local % tiles_i) * 32;
    const float* in = l ? outs + sh.aoff[l - 1] : x;
    const long long ldin = l ? I : ldx;
    const float* dp = dpre + sh.aoff[l];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, rg = lane >> 2, cg = lane & 3;      // lane: outputs 4 rg .. + 3, columns 8 cg .. + 7
    float acc[4][8];
#pragma unroll
    for(int p = 0; p < 4; p++)
#pragma unroll
        for(int q = 0; q < 8; q++) acc[p][q] = 0.0f;
    const int b_begin = slice * FUSED_SLICE, b_end = min(sh.batch, b_begin + FUSED_SLICE);
    for(int b0 = b_begin; b0 < b_end; b0 += GRADS_ROWS){
        float rd[GRADS_ROWS * 32 / 256], ri[GRADS_ROWS * 32 / 256];
#pragma unroll
        for(int u = 0; u < GRADS_ROWS * 32 / 256; u++){
            const int idx = threadIdx.x + u * 256, bb = idx >> 5, c = idx & 31, b = b0 + bb, i = i_base + c;
            rd[u] = (b < b_end && o_base + c < O) ? dp[(long long)b * O + o_base + c] : 0.0f;
            ri[u] = b < b_end ? (i < I ? in[(long long)b * ldin + i] : (i == I ? 1.0f : 0.0f)) : 0.0f;
        }
        __syncthreads();                                  // the previous round's rows have been read
#pragma unroll
        for(int u = 0; u < GRADS_ROWS * 32 / 256; u++){
            const int idx = threadIdx.x + u * 256, bb = idx >> 5, c = idx & 31;
            s_d[bb][c] = rd[u]; s_in[bb][c] = ri[u];
        }
        __syncthreads();
#pragma unroll 4
        for(int bb = warp; bb < GRADS_ROWS; bb += 8){
            const float4 d = *reinterpret_cast<const float4*>(&s_d[bb][4 * rg]);
            const float4 v0 = *reinterpret_cast<const float4*>(&s_in[bb][8 * cg]), v1 = *reinterpret_cast<const float4*>(&s_in[bb][8 * cg + 4]);
            const float dv[4] = {d.x, d.y, d.z, d.w}, vv[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
            for(int p = 0; p < 4; p++)
#pragma unroll
                for(int q = 0; q < 8; q++) acc[p][q] = fmaf(dv[p], vv[q], acc[p][q]);
        }
    }
    __syncthreads();
    float* R = s_all;                                     // [warp][32 outputs][32 columns]
#pragma unroll
    for(int p = 0; p < 4; p++){
        float* row = R + (warp * 32 + 4 * rg + p) * 32 + 8 * cg;
        *reinterpret_cast<float4*>(row) = make_float4(acc[p][0], acc[p][1], acc[p][2], acc[p][3]);
        *reinterpret_cast<float4*>(row + 4) = make_float4(acc[p][4], acc[p][5], acc[p][6], acc[p][7]);
    }
    __syncthreads();
    const int to = threadIdx.x >> 3, ti = (threadIdx.x & 7) * 4;          // thread: output o_base + to, columns i_base + ti .. + 3
    float sum[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for(int w = 0; w < 8; w++){
        const float4 t = *reinterpret_cast<const float4*>(R + (w * 32 + to) * 32 + ti);
        sum[0] += t.x; sum[1] += t.y; sum[2] += t.z; sum[3] += t.w;
    }
    float* gW = grads + sh.poff[l];
    float* gb = gW + (long long)O * I;
    auto target = [&](int o, int i) -> float* { return i < I ? gW + (long long)o * I + i : gb + o; };
    const int o = o_base + to;
    if(n_slices == 1){
#pragma unroll
        for(int q = 0; q < 4; q++){
            const int i = i_base + ti + q;
            if(o < O && i <= I) *target(o, i) += sum[q];
        }
        return;
    }
    // several slices: park the partial tile, the last CTA to arrive for this tile adds the slices in order
    float* mine = partial + ((long long)tile * n_slices + slice) * 1024;
#pragma unroll
    for(int q = 0; q < 4; q++) mine[to * 32 + ti + q] = sum[q];          // scalar: the caller's scratch need not be 16-byte aligned
    __threadfence();
    __syncthreads();
    if(threadIdx.x == 0) is_last = atomicAdd(&counters[tile], 1u) == (unsigned int)(n_slices - 1);
    __syncthreads();
    if(!is_last) return;
    __threadfence();
    const float* all = partial + (long long)tile * n_slices * 1024;
    float t[4] = {0.0f, 0.0f, 0.0f, 0.0f};
    for(int sl = 0; sl < n_slices; sl++){
#pragma unroll
        for(int q = 0; q < 4; q++) t[q] += __ldcg(all + (long long)sl * 1024 + to * 32 + ti + q);
    }
#pragma unroll
    for(int q = 0; q < 4; q++){
        const int i = i_base + ti + q;
        if(o < O && i <= I) *target(o, i) += t[q];
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------------------------------
bool mlp_fused_eligible(const b200rl_mlp_shape* sh, int batch){
    if(batch < 1 || batch > 4096 || sh->input_dim > FUSED_MAX_WIDTH) return false;
    long long padded = 0; int I = sh->input_dim;
    for(int l = 0; l < sh->n_layers; l++){
        if(sh->dims[l] > FUSED_MAX_WIDTH) return false;
        padded += (long long)sh->dims[l] * fused_pitch4(I) * 4 + ((sh->dims[l] + 3) & ~3);
        I = sh->dims[l];
    }
    return padded <= FUSED_MAX_PARAMS;                     // the whole network has to fit into a CTA's shared memory
}

static FusedShape make_fused_shape(const b200rl_mlp_shape* sh, int batch){
    FusedShape f{};
    f.n_layers = sh->n_layers; f.input_dim = sh->input_dim; f.batch = batch;
    long long po = 0, ao = 0; int I = sh->input_dim, tiles = 0, so = 0;
    for(int l = 0; l < sh->n_layers; l++){
        f.dims[l] = sh->dims[l]; f.acts[l] = sh->acts[l]; f.poff[l] = po; f.aoff[l] = ao; f.tile_begin[l] = tiles;
        f.woff[l] = so; so += sh->dims[l] * fused_pitch4(I) * 4;
        f.boff[l] = so; so += (sh->dims[l] + 3) & ~3;
        tiles += ((sh->dims[l] + 31) / 32) * ((I + 1 + 31) / 32);
        po += (long long)sh->dims[l] * I + sh->dims[l]; ao += (long long)batch * sh->dims[l]; I = sh->dims[l];
    }
    f.tile_begin[sh->n_layers] = tiles;
    f.smem_params = so; f.n_params = (int)po;
    return f;
}

static int fused_rows(int batch){ return batch <= 512 ? 2 : (batch <= 1024 ? 4 : 8); }

// scratch of the fused backward: d_pre of all layers | partial tiles (when the batch has several slices) | arrival counters
struct FusedScratch { size_t dpre_floats, partial_floats, counters; size_t bytes; int slices, tiles; };
static FusedScratch fused_scratch(const b200rl_mlp_shape* sh, int batch){
    FusedScratch s{};
    const FusedShape f = make_fused_shape(sh, batch);
    for(int l = 0; l < sh->n_layers; l++) s.dpre_floats += (size_t)batch * sh->dims[l];
    s.dpre_floats = (s.dpre_floats + 3) / 4 * 4;
    s.slices = (batch + FUSED_SLICE - 1) / FUSED_SLICE;
    s.tiles = f.tile_begin[sh->n_layers];
    s.partial_floats = s.slices > 1 ? (size_t)s.tiles * s.slices * 1024 : 0;
    s.counters = s.slices > 1 ? (size_t)s.tiles : 0;
    s.bytes = (s.dpre_floats + s.partial_floats) * sizeof(float) + s.counters * sizeof(unsigned int);
    return s;
}
size_t mlp_fused_backward_scratch_bytes(const b200rl_mlp_shape* sh, int batch){ return mlp_fused_eligible(sh, batch) ? fused_scratch(sh, batch).bytes : 0; }

// dynamic shared memory above 48 KB has to be allowed per kernel and device
template <typename KERNEL>
static int allow_shared_memory(KERNEL kernel, std::atomic<int>* granted, size_t bytes){
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    if((size_t)granted[dev].load(std::memory_order_acquire) < bytes){
        B200RL_CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)((FUSED_MAX_PARAMS + 4 + 2 * 8 * FUSED_MAX_WIDTH) * sizeof(float))));
        granted[dev].store((int)((FUSED_MAX_PARAMS + 4 + 2 * 8 * FUSED_MAX_WIDTH) * sizeof(float)), std::memory_order_release);
    }
    return B200RL_OK;
}

template <int ROWS, bool SAVE>
static int launch_fused_forward(const FusedShape& f, const float* params, const float* x, int ldx, float* pre, float* out, float* y, int ldy, cudaStream_t s){
    static std::atomic<int> granted[MAX_DEVICES];
    const size_t bytes = ((size_t)f.smem_params + 2 * ROWS * FUSED_MAX_WIDTH) * sizeof(float);
    int rc = allow_shared_memory(mlp_fused_forward_kernel<ROWS, SAVE>, granted, bytes);
    if(rc) return rc;
    mlp_fused_forward_kernel<ROWS, SAVE><<<(f.batch + ROWS - 1) / ROWS, FUSED_THREADS, bytes, s>>>(f, params, x, ldx, pre, out, y, ldy);
    B200RL_LAUNCH_CHECK("mlp_fused_forward");
    return B200RL_OK;
}
template <int ROWS>
static int launch_fused_chain(const FusedShape& f, const float* params, const float* pre, float* d_out, int ldd, float* dpre, float* d_input, int ldi,
                              unsigned int* counters, int n_counters, cudaStream_t s){
    static std::atomic<int> granted[MAX_DEVICES];
    const size_t bytes = ((size_t)((f.n_params + 3) & ~3) + 2 * ROWS * FUSED_MAX_WIDTH) * sizeof(float);
    int rc = allow_shared_memory(mlp_fused_backward_chain_kernel<ROWS>, granted, bytes);
    if(rc) return rc;
    mlp_fused_backward_chain_kernel<ROWS><<<(f.batch + ROWS - 1) / ROWS, FUSED_THREADS, bytes, s>>>(f, params, pre, d_out, ldd, dpre, d_input, ldi, counters, n_counters);
    B200RL_LAUNCH_CHECK("mlp_fused_backward_chain");
    return B200RL_OK;
}

int mlp_fused_forward(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out, float* y, int ldy, int batch, cudaStream_t s){
    const FusedShape f = make_fused_shape(sh, batch);
    const int rows = fused_rows(batch);
    if(pre){
        if(rows == 2) return launch_fused_forward<2, true>(f, params, x, ldx, pre, out, nullptr, 0, s);
        if(rows == 4) return launch_fused_forward<4, true>(f, params, x, ldx, pre, out, nullptr, 0, s);
        return launch_fused_forward<8, true>(f, params, x, ldx, pre, out, nullptr, 0, s);
    }
    if(rows == 2) return launch_fused_forward<2, false>(f, params, x, ldx, nullptr, nullptr, y, ldy, s);
    if(rows == 4) return launch_fused_forward<4, false>(f, params, x, ldx, nullptr, nullptr, y, ldy, s);
    return launch_fused_forward<8, false>(f, params, x, ldx, nullptr, nullptr, y, ldy, s);
}

int mlp_fused_backward(const b200rl_mlp_shape* sh, const float* params, float* grads, const float* x, int ldx, const float* pre, const float* out, float* d_out,
                       float* d_input, int batch, void* scratch, size_t scratch_bytes, cudaStream_t s){
    const FusedScratch fs = fused_scratch(sh, batch);
    if(!scratch || scratch_bytes < fs.bytes) return B200RL_ERR_INVALID_ARGUMENT;
    const FusedShape f = make_fused_shape(sh, batch);
    float* dpre = reinterpret_cast<float*>(scratch);
    float* partial = dpre + fs.dpre_floats;
    unsigned int* counters = reinterpret_cast<unsigned int*>(partial + fs.partial_floats);
    const int rows = fused_rows(batch);
    const int ldd = sh->dims[sh->n_layers - 1];
    unsigned int* cnt = grads && fs.counters ? counters : nullptr;
    int rc;
    if(rows == 2) rc = launch_fused_chain<2>(f, params, pre, d_out, ldd, dpre, d_input, sh->input_dim, cnt, (int)fs.counters, s);
    else if(rows == 4) rc = launch_fused_chain<4>(f, params, pre, d_out, ldd, dpre, d_input, sh->input_dim, cnt, (int)fs.counters, s);
    else rc = launch_fused_chain<8>(f, params, pre, d_out, ldd, dpre, d_input, sh->input_dim, cnt, (int)fs.counters, s);
    if(rc) return rc;
    if(grads){
        mlp_fused_grads_kernel<<<dim3(fs.tiles, fs.slices), 256, 0, s>>>(f, x, ldx, out, dpre, grads, partial, counters, fs.slices);
        B200RL_LAUNCH_CHECK("mlp_fused_grads");
    }
    return B200RL_OK;
}

}  // namespace b200rl
