// Dense layer forward / backward for fp32 row-major operands with arbitrary row pitch, and the MLP chaining on a
// flat parameter arena.
//
// One tiled kernel template covers the three contractions of a dense layer; they differ only in which operand
// index is contiguous in memory:
//   forward : y[b][o]   = sum_i x[b][i]     * W[o][i]     (both operands contiguous along the summed index)
//   d_in    : d_in[b][i]= sum_o d_pre[b][o] * W[o][i]     (W strided along the summed index)
//   d_W     : dW[o][i] += sum_b d_pre[b][o] * x[b][i]     (both strided; summed index = batch, split across CTAs)
// Bias, pre-activation store and activation are fused into the forward epilogue; d_pre = act'(pre) * d_out and the
// bias gradient are one pass; split-batch partials of d_W / d_bias are reduced in a fixed order (deterministic).
#include "common.cuh"
#include "dense.cuh"
#include <math.h>
#include <mutex>

namespace b200rl {

constexpr int BM = 64, BN = 64, BK = 16, GEMM_THREADS = 256, PADM = 4;

// One k-step of an operand tile travels global -> registers -> shared memory, so that the loads of step k+1 are in flight while
// step k is multiplied (the batch-256 and 64-wide problems run on few CTAs and are bound by this latency, not by bandwidth).
// Tile element (k, r) = P(row0 + r, k0 + k), zero outside [0, rows) x [k0, k_end); T * KS / 256 elements per thread (T = tile edge, KS = k
// step). The 32-wide tiles take k steps of 64: they exist for problems that fill few SMs, where a tile's time is (number of k steps) x
// (one L2 round trip), so four times fewer, four times larger steps (8 loads in flight per thread and operand instead of 2).
template <int T, int KS, bool KCONTIG>
__device__ __forceinline__ void fetch_tile(float (&reg)[T * KS / GEMM_THREADS], const float* __restrict__ P, long long ld, int row0, int rows, int k0, int k_end, int tid){
    if constexpr(KCONTIG){
        const int k = tid % KS, r = tid / KS;            // KS consecutive k per row -> 64- or 256-byte segments
#pragma unroll
        for(int j = 0; j < T * KS / GEMM_THREADS; j++){
            const int gr = row0 + r + j * (GEMM_THREADS / KS), gk = k0 + k;
            reg[j] = (gr < rows && gk < k_end) ? __ldg(P + (long long)gr * ld + gk) : 0.0f;
        }
    }
    else{
        const int r = tid % T, k = tid / T;              // T consecutive rows (contiguous in memory) per k
#pragma unroll
        for(int j = 0; j < T * KS / GEMM_THREADS; j++){
            const int gr = row0 + r, gk = k0 + k + j * (GEMM_THREADS / T);
            reg[j] = (gr < rows && gk < k_end) ? __ldg(P + (long long)gk * ld + gr) : 0.0f;
        }
    }
}
template <int T, int KS, bool KCONTIG>
__device__ __forceinline__ void store_tile(float (*S)[T + PADM], const float (&reg)[T * KS / GEMM_THREADS], int tid){
    if constexpr(KCONTIG){
        const int k = tid % KS, r = tid / KS;
#pragma unroll
        for(int j = 0; j < T * KS / GEMM_THREADS; j++) S[k][r + j * (GEMM_THREADS / KS)] = reg[j];
    }
    else{
        const int r = tid % T, k = tid / T;
#pragma unroll
        for(int j = 0; j < T * KS / GEMM_THREADS; j++) S[k + j * (GEMM_THREADS / T)][r] = reg[j];
    }
}

// C tile T x T per CTA (T = 64, or 32 when 64-wide tiles would leave most SMs idle), 256 threads, (T/16)^2 outputs per thread.
template <int T, bool A_KCONTIG, bool B_KCONTIG, int EPI, int ACT>
__global__ void __launch_bounds__(GEMM_THREADS) gemm_kernel(GemmArgs a){
    static_assert(T == 64 || T == 32);
    constexpr int R = T / 16, KS = T == 64 ? BK : 4 * BK, NREG = T * KS / GEMM_THREADS;
    __shared__ __align__(16) float As[KS][T + PADM];
    __shared__ __align__(16) float Bs[KS][T + PADM];
    const int tid = threadIdx.x;
    const int m0 = blockIdx.y * T, n0 = blockIdx.x * T;
    const int k_begin = blockIdx.z * a.k_per_split;
    const int k_end = min(a.K, k_begin + a.k_per_split);
    const int tx = tid % 16, ty = tid / 16;
    float acc[R][R];
#pragma unroll
    for(int i = 0; i < R; i++)
#pragma unroll
        for(int j = 0; j < R; j++) acc[i][j] = 0.0f;

    float ra[NREG], rb[NREG];
    fetch_tile<T, KS, A_KCONTIG>(ra, a.A, a.lda, m0, a.M, k_begin, k_end, tid);
    fetch_tile<T, KS, B_KCONTIG>(rb, a.B, a.ldb, n0, a.N, k_begin, k_end, tid);
    for(int k0 = k_begin; k0 < k_end; k0 += KS){
        store_tile<T, KS, A_KCONTIG>(As, ra, tid);
        store_tile<T, KS, B_KCONTIG>(Bs, rb, tid);
        __syncthreads();
        if(k0 + KS < k_end){
            fetch_tile<T, KS, A_KCONTIG>(ra, a.A, a.lda, m0, a.M, k0 + KS, k_end, tid);
            fetch_tile<T, KS, B_KCONTIG>(rb, a.B, a.ldb, n0, a.N, k0 + KS, k_end, tid);
        }
#pragma unroll
        for(int k = 0; k < KS; k++){
            float am[R], bn[R];
            if constexpr(R == 4){
                const float4 av = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
                const float4 bv = *reinterpret_cast<const float4*>(&Bs[k][tx * 4]);
                am[0] = av.x; am[1] = av.y; am[2] = av.z; am[3] = av.w; bn[0] = bv.x; bn[1] = bv.y; bn[2] = bv.z; bn[3] = bv.w;
            }
            else{
                const float2 av = *reinterpret_cast<const float2*>(&As[k][ty * 2]);
                const float2 bv = *reinterpret_cast<const float2*>(&Bs[k][tx * 2]);
                am[0] = av.x; am[1] = av.y; bn[0] = bv.x; bn[1] = bv.y;
            }
#pragma unroll
            for(int i = 0; i < R; i++)
#pragma unroll
                for(int j = 0; j < R; j++) acc[i][j] = fmaf(am[i], bn[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for(int i = 0; i < R; i++){
        int m = m0 + ty * R + i;
        if(m >= a.M) continue;
#pragma unroll
        for(int j = 0; j < R; j++){
            int n = n0 + tx * R + j;
            if(n >= a.N) continue;
            float v = acc[i][j];
            if constexpr(EPI == EPI_FORWARD){
                v += __ldg(a.bias + n);
                if(a.pre) a.pre[(long long)m * a.ldpre + n] = v;
                a.C[(long long)m * a.ldc + n] = activation<ACT>(v);
            }
            else if constexpr(EPI == EPI_STORE){
                a.C[(long long)m * a.ldc + n] = v;
            }
            else{
                if(gridDim.z == 1) a.C[(long long)m * a.ldc + n] += v;
                else a.partial[((long long)blockIdx.z * a.M + m) * a.N + n] = v;
            }
        }
    }
}
// 32-wide tiles when 64-wide ones would occupy less than half of the SMs
static inline bool small_tiles(int M, int N, int splits){
    return (long long)((M + 63) / 64) * ((N + 63) / 64) * splits < NUM_SMS / 2;
}
#define B200RL_LAUNCH_SIMT_GEMM(AK, BKC, EPI, ACT, args, splits, stream)                                                            \
    do{                                                                                                                             \
        if(small_tiles((args).M, (args).N, (splits))){                                                                              \
            dim3 grid_(((args).N + 31) / 32, ((args).M + 31) / 32, (splits));                                                       \
            gemm_kernel<32, AK, BKC, EPI, ACT><<<grid_, GEMM_THREADS, 0, (stream)>>>(args);                                         \
        }                                                                                                                           \
        else{                                                                                                                       \
            dim3 grid_(((args).N + 63) / 64, ((args).M + 63) / 64, (splits));                                                       \
            gemm_kernel<64, AK, BKC, EPI, ACT><<<grid_, GEMM_THREADS, 0, (stream)>>>(args);                                         \
        }                                                                                                                           \
    } while(0)

// d_pre = act'(pre) * d_out written in place, plus per-column sums over a segment of rows.
// grid (ceil(O/32), n_seg), block (32, 8). n_seg == 1: d_bias += column sum; else bias_partial[seg][o] = column sum.
template <int ACT>
__global__ void __launch_bounds__(256) dpre_bias_kernel(const float* __restrict__ pre, long long ldpre, float* d_out, long long ldd, float* d_bias, float* bias_partial,
                                                       int B, int O, int rows_per_seg){
    __shared__ float red[8][33];
    int o = blockIdx.x * 32 + threadIdx.x;
    int r0 = blockIdx.y * rows_per_seg, r1 = min(B, r0 + rows_per_seg);
    float s = 0.0f;
    if(o < O){
        for(int r = r0 + threadIdx.y; r < r1; r += 8){
            float d = d_activation<ACT>(pre[(long long)r * ldpre + o]) * d_out[(long long)r * ldd + o];
            d_out[(long long)r * ldd + o] = d;
            s += d;
        }
    }
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if(threadIdx.y == 0 && o < O){
        float t = 0.0f;
#pragma unroll
        for(int y = 0; y < 8; y++) t += red[y][threadIdx.x];
        if(d_bias){
            if(gridDim.y == 1) d_bias[o] += t;
            else bias_partial[(long long)blockIdx.y * O + o] = t;
        }
    }
}
// Vector version for 16-byte aligned operands (O % 4 == 0, pitches % 4 == 0): a thread owns 4 adjacent columns, a block
// 128 columns x 8 row lanes, and each thread keeps 4 rows (8 independent 16-byte loads) in flight -- the scalar version
// above has one dependent load pair per thread in flight and reaches only a quarter of the HBM bandwidth.
template <int ACT>
__global__ void __launch_bounds__(256) dpre_bias_vec_kernel(const float* __restrict__ pre, long long ldpre, float* d_out, long long ldd, float* d_bias, float* bias_partial,
                                                           int B, int O, int rows_per_seg){
    __shared__ float4 red[8][32];
    const int cg = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int o = blockIdx.x * 128 + cg * 4;
    const int r0 = blockIdx.y * rows_per_seg, r1 = min(B, r0 + rows_per_seg);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    if(o < O){
        int r = r0 + ty;
        for(; r + 24 < r1; r += 32){
            float4 p[4], d[4];
#pragma unroll
            for(int k = 0; k < 4; k++){
                p[k] = *reinterpret_cast<const float4*>(pre + (long long)(r + 8 * k) * ldpre + o);
                d[k] = *reinterpret_cast<const float4*>(d_out + (long long)(r + 8 * k) * ldd + o);
            }
#pragma unroll
            for(int k = 0; k < 4; k++){
                d[k].x *= d_activation<ACT>(p[k].x); d[k].y *= d_activation<ACT>(p[k].y); d[k].z *= d_activation<ACT>(p[k].z); d[k].w *= d_activation<ACT>(p[k].w);
                *reinterpret_cast<float4*>(d_out + (long long)(r + 8 * k) * ldd + o) = d[k];
                s.x += d[k].x; s.y += d[k].y; s.z += d[k].z; s.w += d[k].w;
            }
        }
        for(; r < r1; r += 8){
            const float4 p = *reinterpret_cast<const float4*>(pre + (long long)r * ldpre + o);
            float4 d = *reinterpret_cast<const float4*>(d_out + (long long)r * ldd + o);
            d.x *= d_activation<ACT>(p.x); d.y *= d_activation<ACT>(p.y); d.z *= d_activation<ACT>(p.z); d.w *= d_activation<ACT>(p.w);
            *reinterpret_cast<float4*>(d_out + (long long)r * ldd + o) = d;
            s.x += d.x; s.y += d.y; s.z += d.z; s.w += d.w;
        }
    }
    red[ty][cg] = s;
    __syncthreads();
    if(ty == 0 && o < O && d_bias){
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for(int y = 0; y < 8; y++){ t.x += red[y][cg].x; t.y += red[y][cg].y; t.z += red[y][cg].z; t.w += red[y][cg].w; }
        float* dst = gridDim.y == 1 ? d_bias + o : bias_partial + (long long)blockIdx.y * O + o;
        if(gridDim.y == 1){ dst[0] += t.x; dst[1] += t.y; dst[2] += t.z; dst[3] += t.w; }
        else{ dst[0] = t.x; dst[1] = t.y; dst[2] = t.z; dst[3] = t.w; }
    }
}
// dst[i] += sum_s partial[s][i], s ascending (fixed order). Eight loads are issued before their (sequential, order-preserving) adds:
// with 74 splits of a 256 x 256 gradient a thread's chain of dependent load-add pairs was latency-bound (24 us per call).
__global__ void reduce_partials_kernel(float* dst, const float* __restrict__ partial, long long n, int splits){
    for(long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x){
        float s = 0.0f;
        int z = 0;
        for(; z + 8 <= splits; z += 8){
            float v[8];
#pragma unroll
            for(int j = 0; j < 8; j++) v[j] = __ldg(partial + (long long)(z + j) * n + i);
#pragma unroll
            for(int j = 0; j < 8; j++) s += v[j];
        }
        for(; z < splits; z++) s += __ldg(partial + (long long)z * n + i);
        dst[i] += s;
    }
}

// Bias gradient: dst[o] += sum_s partial[s][o] for few columns and many segments. One block per 32 columns, 8 lanes of segments
// (lane y takes s = y, y + 8, ... in ascending order), then the 8 lane sums in ascending order: a fixed summation order, and
// segs / 8 dependent steps instead of segs (the single-block, one-thread-per-column form took 31 us for 296 segments).
// (stride: floats from one segment's record to the next; O for densely packed segments)
__global__ void __launch_bounds__(256) reduce_strided_partials_kernel(float* dst, const float* __restrict__ partial, int O, long long stride, int segs){
    __shared__ float red[8][33];
    const int o = blockIdx.x * 32 + threadIdx.x;
    float s = 0.0f;
    if(o < O){
        int z = threadIdx.y;
        for(; z + 24 < segs; z += 32){
            const float v0 = __ldg(partial + (long long)z * stride + o), v1 = __ldg(partial + (long long)(z + 8) * stride + o);
            const float v2 = __ldg(partial + (long long)(z + 16) * stride + o), v3 = __ldg(partial + (long long)(z + 24) * stride + o);
            s += v0; s += v1; s += v2; s += v3;
        }
        for(; z < segs; z += 8) s += __ldg(partial + (long long)z * stride + o);
    }
    red[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if(threadIdx.y == 0 && o < O){
        float t = 0.0f;
#pragma unroll
        for(int y = 0; y < 8; y++) t += red[y][threadIdx.x];
        dst[o] += t;
    }
}

// The tensor-core kernel takes the contraction when there is enough work to fill its 128 x 256 tiles on a good part of the SMs:
// one tile costs ~30 us at K = 256 however few tiles there are, which the CUDA-core kernel's 64 x 64 tiles beat below ~2^27
// multiply-adds (batch-256 training steps, the 64-wide PPO networks).
static bool tc_eligible(long long M, long long N, long long K){
    return M >= 64 && N >= 16 && (double)M * N * K >= ldexp(1.0, 27);
}
static bool use_tensor_cores(const GemmArgs& a){ return tc_eligible(a.M, a.N, a.K); }

// one-pass backward of a layer with few outputs at a large batch (dense_skinny.cu)
bool skinny_backward_eligible(int B, int I, int O);
size_t skinny_backward_scratch_bytes(int I, int O, int ctas);
int skinny_backward_launch(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd, float* partial, float* d_in, int ldi,
                           int B, int I, int O, int act, int ctas, cudaStream_t s);
bool skinny_forward_eligible(const float* x, int ldx, int B, int I, int O);
int skinny_forward_launch(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy, int B, int I, int O, int act, int ctas, cudaStream_t s);
constexpr int SKINNY_CTAS = 2 * NUM_SMS;       // two resident CTAs per SM, one wave

// bytes: split-k and bias partial sums (required when gradients are wanted); wt_bytes: room behind them for the operand image of the
// transposed weights, which the input-gradient product of the tensor-core path copies in instead of re-splitting W^T per row tile
// (used when the scratch has it)
struct BackwardPlan { int splits; int k_per_split; int bias_segs; int rows_per_seg; size_t bytes; size_t wt_bytes; };
// budget: upper bound on p.bytes. The plan lowers the number of bias segments and of batch splits until the partial sums fit (fewer
// splits is slower but as correct and as deterministic; one split needs no partial sums at all).
static BackwardPlan plan_backward(int B, int I, int O, size_t budget = SIZE_MAX){
    BackwardPlan p;
    // weight gradient = contraction over the batch: split it so that every SM has work (tile shape of the kernel that will run)
    // fewer than 64 output rows (e.g. a 16-wide last layer): the tensor-core kernel computes dW^T instead (rows = input features)
    const bool tc_direct = tc_eligible(O, I, B), tc_swapped = !tc_direct && tc_eligible(I, O, B);
    const bool tc = tc_direct || tc_swapped;
    int tiles = tc_direct ? ((O + 127) / 128) * ((I + 255) / 256) : tc_swapped ? ((I + 127) / 128) * ((O + 255) / 256) : ((O + BM - 1) / BM) * ((I + BN - 1) / BN);
    int want = tc ? (NUM_SMS + tiles - 1) / tiles : (2 * NUM_SMS + tiles - 1) / tiles;
    // at least 256 batch rows per split for the tensor-core kernel (8 chunks amortise its tile setup), 64 for the CUDA-core kernel:
    // small batches (256 ... 2048 rows) would otherwise run on a handful of CTAs and be bound by the latency of their k loop
    int max_splits = tc ? (B + 255) / 256 : (B + 63) / 64;
    p.splits = want < 1 ? 1 : (want > max_splits ? max_splits : want);
    if(p.splits < 1) p.splits = 1;
    int col_blocks = (O + 127) / 128;                      // the vector kernel's blocks cover 128 columns
    int want_segs = (4 * NUM_SMS + col_blocks - 1) / col_blocks;
    int max_segs = (B + 63) / 64;
    p.bias_segs = want_segs > max_segs ? max_segs : want_segs;
    if(p.bias_segs < 1) p.bias_segs = 1;
    if(budget != SIZE_MAX){
        const size_t seg_bytes = sizeof(float) * (size_t)O, split_bytes = sizeof(float) * (size_t)O * I, usable = budget - (budget < 16 ? budget : 16);
        if((size_t)p.bias_segs * seg_bytes > usable / 4) p.bias_segs = (int)(usable / 4 / seg_bytes);     // at most a quarter for the bias partials
        if(p.bias_segs < 2) p.bias_segs = 1;
        const size_t left = usable - (p.bias_segs > 1 ? (size_t)p.bias_segs * seg_bytes : 0);
        if((size_t)p.splits * split_bytes > left) p.splits = (int)(left / split_bytes);
        if(p.splits < 2) p.splits = 1;
    }
    p.k_per_split = ((B + p.splits - 1) / p.splits + BK - 1) / BK * BK;
    p.splits = (B + p.k_per_split - 1) / p.k_per_split;
    p.rows_per_seg = (B + p.bias_segs - 1) / p.bias_segs;
    p.bias_segs = (B + p.rows_per_seg - 1) / p.rows_per_seg;
    p.bytes = 0;
    if(p.splits > 1) p.bytes += sizeof(float) * (size_t)p.splits * O * I;
    if(p.bias_segs > 1) p.bytes += sizeof(float) * (size_t)p.bias_segs * O;
    p.bytes = (p.bytes + 15) / 16 * 16;
    p.wt_bytes = tc_eligible(B, I, O) ? weight_image_bytes(I, O) : 0;
    return p;
}

// what b200rl_dense_backward_scratch_bytes reports: the tiled path's partial sums and operand image, or the one-pass kernel's per-CTA sums
static size_t backward_scratch_total(int B, int I, int O){
    const BackwardPlan p = plan_backward(B, I, O);
    const size_t tiled = p.bytes + p.wt_bytes, skinny = skinny_backward_eligible(B, I, O) ? skinny_backward_scratch_bytes(I, O, SKINNY_CTAS) : 0;
    return tiled > skinny ? tiled : skinny;
}

// workspace (optional): room for the weights' operand image, see b200rl_dense_forward_workspace_bytes
static size_t forward_workspace_bytes(int B, int I, int O){ return tc_eligible(B, O, I) ? weight_image_bytes(O, I) : 0; }
static int dense_forward_impl(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                              int B, int I, int O, int act, cudaStream_t s, void* workspace = nullptr, size_t workspace_bytes = 0){
    if(skinny_forward_eligible(x, ldx, B, I, O)) return skinny_forward_launch(W, bias, x, ldx, pre, ldpre, y, ldy, B, I, O, act, SKINNY_CTAS, s);
    GemmArgs a{};
    a.A = x; a.lda = ldx; a.B = W; a.ldb = I; a.M = B; a.N = O; a.K = I; a.k_per_split = I;
    a.bias = bias; a.pre = pre; a.ldpre = ldpre; a.C = y; a.ldc = ldy;
    if(use_tensor_cores(a)){
        int rc = B200RL_ERR_UNSUPPORTED;
        if(workspace != nullptr && workspace_bytes >= weight_image_bytes(O, I) && (reinterpret_cast<uintptr_t>(workspace) & 15u) == 0){
            // the weights are split into their tf32 parts ONCE per call (a few microseconds), not once per 128-row tile of the batch
            rc = launch_weight_image(W, I, O, I, false, static_cast<float*>(workspace), s);
            if(rc) return rc;
            GemmArgs g = a;
            g.B = static_cast<const float*>(workspace);
            rc = launch_gemm_tc(g, EPI_FORWARD, act, true, true, 1, s, true);
        }
        if(rc == B200RL_ERR_UNSUPPORTED) rc = launch_gemm_tc(a, EPI_FORWARD, act, true, true, 1, s);
        if(rc != B200RL_ERR_UNSUPPORTED) return rc;
    }
    B200RL_DISPATCH_ACT(act, B200RL_LAUNCH_SIMT_GEMM(true, true, EPI_FORWARD, ACT, a, 1, s));
    B200RL_LAUNCH_CHECK("dense_forward");
    return B200RL_OK;
}

// A second stream for the gradient branch of a captured backward pass, forked from `s` here and joined by the caller through *join.
// Every origin stream gets its own helper stream and event pair (created on first use, kept for the life of the process), so that two
// networks whose backward passes are captured on two streams do not serialise on one helper. Beyond the table's size: no branch.
static int gradient_branch(cudaStream_t s, cudaStream_t* branch, cudaEvent_t* join){
    constexpr int SLOTS = 16;
    static struct { int device; cudaStream_t origin, helper; cudaEvent_t fork, join; bool used; } table[SLOTS] = {};
    static std::mutex mutex;
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    std::lock_guard<std::mutex> lock(mutex);
    int slot = -1;
    for(int i = 0; i < SLOTS; i++){
        if(table[i].used && table[i].origin == s && table[i].device == dev){ slot = i; break; }
        if(!table[i].used && slot < 0) slot = i;
    }
    if(slot < 0) return B200RL_OK;                                      // table full: everything stays on s
    if(!table[slot].used){                                              // helper stream and events live on the current device, like s
        B200RL_CUDA_TRY(cudaStreamCreateWithFlags(&table[slot].helper, cudaStreamNonBlocking));
        B200RL_CUDA_TRY(cudaEventCreateWithFlags(&table[slot].fork, cudaEventDisableTiming));
        B200RL_CUDA_TRY(cudaEventCreateWithFlags(&table[slot].join, cudaEventDisableTiming));
        table[slot].origin = s; table[slot].device = dev; table[slot].used = true;
    }
    B200RL_CUDA_TRY(cudaEventRecord(table[slot].fork, s));
    B200RL_CUDA_TRY(cudaStreamWaitEvent(table[slot].helper, table[slot].fork, 0));
    *branch = table[slot].helper; *join = table[slot].join;
    return B200RL_OK;
}

static int dense_backward_impl(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                               float* dW, float* db, float* d_in, int ldi, int B, int I, int O, int act, void* scratch, size_t scratch_bytes, cudaStream_t s,
                               size_t plan_budget = SIZE_MAX){
    bool want_grads = dW != nullptr;
    // few outputs at a large batch: one pass over the layer's input (d_pre, bias and weight gradients, input gradient), when the scratch holds
    // its per-CTA sums; the tiled path otherwise
    if(skinny_backward_eligible(B, I, O) && (!want_grads || (scratch && scratch_bytes >= skinny_backward_scratch_bytes(I, O, SKINNY_CTAS)))){
        float* partial = want_grads ? reinterpret_cast<float*>(scratch) : nullptr;
        int rc = skinny_backward_launch(W, x, ldx, pre, ldpre, d_out, ldd, partial, d_in, ldi, B, I, O, act, SKINNY_CTAS, s);
        if(rc) return rc;
        if(want_grads){
            // records of O * I + O floats per CTA: one reduction when the bias gradient follows the weight gradient in memory (a flat arena)
            const int n = O * I, record = n + O;
            if(db == dW + n){
                reduce_strided_partials_kernel<<<(record + 31) / 32, dim3(32, 8), 0, s>>>(dW, partial, record, record, SKINNY_CTAS);
                B200RL_LAUNCH_CHECK("reduce_skinny");
            }
            else{
                reduce_strided_partials_kernel<<<(n + 31) / 32, dim3(32, 8), 0, s>>>(dW, partial, n, record, SKINNY_CTAS);
                B200RL_LAUNCH_CHECK("reduce_dW");
                reduce_strided_partials_kernel<<<(O + 31) / 32, dim3(32, 8), 0, s>>>(db, partial + n, O, record, SKINNY_CTAS);
                B200RL_LAUNCH_CHECK("reduce_bias");
            }
        }
        return B200RL_OK;
    }
    BackwardPlan p = plan_backward(B, I, O, plan_budget);
    if(want_grads && p.bytes > 0 && (scratch == nullptr || scratch_bytes < p.bytes)) return B200RL_ERR_INVALID_ARGUMENT;
    float* w_partial = reinterpret_cast<float*>(scratch);
    float* b_partial = w_partial + (p.splits > 1 ? (size_t)p.splits * O * I : 0);
    // backward_input only (no parameter gradients): d_pre is still needed, the column sums are not
    int segs = want_grads ? p.bias_segs : (B + 4095) / 4096;
    int rps = want_grads ? p.rows_per_seg : 4096;
    {
        const bool vec = (O % 4 == 0) && (ldpre % 4 == 0) && (ldd % 4 == 0) && ((reinterpret_cast<uintptr_t>(pre) | reinterpret_cast<uintptr_t>(d_out)) & 15u) == 0;
        if(vec){
            dim3 grid((O + 127) / 128, segs);
            B200RL_DISPATCH_ACT(act, (dpre_bias_vec_kernel<ACT><<<grid, 256, 0, s>>>(pre, ldpre, d_out, ldd, want_grads ? db : nullptr, b_partial, B, O, rps)));
        }
        else{
            dim3 grid((O + 31) / 32, segs), block(32, 8);
            B200RL_DISPATCH_ACT(act, (dpre_bias_kernel<ACT><<<grid, block, 0, s>>>(pre, ldpre, d_out, ldd, want_grads ? db : nullptr, b_partial, B, O, rps)));
        }
        B200RL_LAUNCH_CHECK("dpre_bias");
    }
    // Inside a stream capture the parameter-gradient chain (bias reduction, dW product, its reduction) and the input-gradient product
    // become parallel branches of the graph: both only read d_pre. Eager launches stay on one stream (the extra events would cost more
    // host time than the overlap returns at the sizes where it matters).
    cudaStream_t sg = s;
    cudaEvent_t join = nullptr;
    if(want_grads && d_in){
        cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
        B200RL_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
        if(cap == cudaStreamCaptureStatusActive){
            int rc = gradient_branch(s, &sg, &join);
            if(rc) return rc;
        }
    }
    if(want_grads && segs > 1){
        reduce_strided_partials_kernel<<<(O + 31) / 32, dim3(32, 8), 0, sg>>>(db, b_partial, O, O, segs);
        B200RL_LAUNCH_CHECK("reduce_bias");
    }
    if(want_grads){
        GemmArgs a{};
        a.A = d_out; a.lda = ldd; a.B = x; a.ldb = ldx; a.M = O; a.N = I; a.K = B; a.k_per_split = p.k_per_split;
        a.C = dW; a.ldc = I; a.partial = w_partial;
        int rc_tc = B200RL_ERR_UNSUPPORTED;
        if(use_tensor_cores(a)) rc_tc = launch_gemm_tc(a, EPI_ACCUMULATE, 0, false, false, p.splits, sg);
        else if(tc_eligible(I, O, B)){
            GemmArgs t = a;                        // dW^T[i][o] = sum_b x[b][i] * d_pre[b][o], stored transposed into dW / the partials
            t.A = x; t.lda = ldx; t.B = d_out; t.ldb = ldd; t.M = I; t.N = O; t.transpose_c = 1;
            rc_tc = launch_gemm_tc(t, EPI_ACCUMULATE, 0, false, false, p.splits, sg);
        }
        if(rc_tc != B200RL_OK && rc_tc != B200RL_ERR_UNSUPPORTED) return rc_tc;
        if(rc_tc == B200RL_ERR_UNSUPPORTED){
            B200RL_LAUNCH_SIMT_GEMM(false, false, EPI_ACCUMULATE, 0, a, p.splits, sg);
            B200RL_LAUNCH_CHECK("dense_dW");
        }
        if(p.splits > 1){
            long long n = (long long)O * I;
            if(p.splits >= 16 && n < (1ll << 30)){
                // many partial sums per element: eight lanes share an element's splits (a fixed order again: lane y takes y, y + 8, ...,
                // then the lanes ascending), so a thread's chain is splits / 8 loads long (74 splits of 256 x 256: 12.5 -> 8 us)
                reduce_strided_partials_kernel<<<(unsigned)((n + 31) / 32), dim3(32, 8), 0, sg>>>(dW, w_partial, (int)n, n, p.splits);
            }
            else{
                int blocks = (int)((n + 255) / 256); if(blocks > 4 * NUM_SMS) blocks = 4 * NUM_SMS;
                reduce_partials_kernel<<<blocks, 256, 0, sg>>>(dW, w_partial, n, p.splits);
            }
            B200RL_LAUNCH_CHECK("reduce_dW");
        }
    }
    if(join){ B200RL_CUDA_TRY(cudaEventRecord(join, sg)); }
    if(d_in){
        GemmArgs a{};
        a.A = d_out; a.lda = ldd; a.B = W; a.ldb = I; a.M = B; a.N = I; a.K = O; a.k_per_split = O;
        a.C = d_in; a.ldc = ldi;
        int rc_tc = B200RL_ERR_UNSUPPORTED;
        if(use_tensor_cores(a)){
            if(p.wt_bytes > 0 && scratch != nullptr && scratch_bytes >= p.bytes + p.wt_bytes){
                // operand image of W^T once per call (tf32 parts, tile layout), copied in by the kernel chunk by chunk
                float* image = reinterpret_cast<float*>(static_cast<char*>(scratch) + p.bytes);
                int rc = launch_weight_image(W, I, I, O, true, image, s);
                if(rc) return rc;
                GemmArgs g = a;
                g.B = image;
                rc_tc = launch_gemm_tc(g, EPI_STORE, 0, true, true, 1, s, true);
            }
            if(rc_tc == B200RL_ERR_UNSUPPORTED) rc_tc = launch_gemm_tc(a, EPI_STORE, 0, true, false, 1, s);
        }
        if(rc_tc != B200RL_OK && rc_tc != B200RL_ERR_UNSUPPORTED) return rc_tc;
        if(rc_tc == B200RL_ERR_UNSUPPORTED){
            B200RL_LAUNCH_SIMT_GEMM(true, false, EPI_STORE, 0, a, 1, s);
            B200RL_LAUNCH_CHECK("dense_d_in");
        }
    }
    if(join) B200RL_CUDA_TRY(cudaStreamWaitEvent(s, join, 0));
    return B200RL_OK;
}

// whole-network kernels for small batches (mlp_fused.cu)
bool mlp_fused_eligible(const b200rl_mlp_shape* sh, int batch);
size_t mlp_fused_backward_scratch_bytes(const b200rl_mlp_shape* sh, int batch);
int mlp_fused_forward(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out, float* y, int ldy, int batch, cudaStream_t s);
int mlp_fused_backward(const b200rl_mlp_shape* sh, const float* params, float* grads, const float* x, int ldx, const float* pre, const float* out, float* d_out,
                       float* d_input, int batch, void* scratch, size_t scratch_bytes, cudaStream_t s);

// whole-pass cooperative kernel for wide networks at small batches (mlp_coop.cu)
bool mlp_coop_eligible(const b200rl_mlp_shape* sh, int batch, bool forward);
int mlp_coop_forward(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out, float* y, int ldy,
                     float* tick, float* tock, int batch, cudaStream_t s);
int mlp_coop_backward(const b200rl_mlp_shape* sh, const float* params, float* grads, const float* x, int ldx, const float* pre, const float* out,
                      float* d_out, float* d_input, float* tick, float* tock, int batch, cudaStream_t s);

static bool valid_shape(const b200rl_mlp_shape* sh){
    if(!sh || sh->n_layers < 1 || sh->n_layers > B200RL_MAX_LAYERS || sh->input_dim < 1) return false;
    for(int l = 0; l < sh->n_layers; l++) if(sh->dims[l] < 1 || !valid_activation(sh->acts[l])) return false;
    return true;
}

}  // namespace b200rl

using namespace b200rl;

extern "C" {

int b200rl_dense_forward(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                         int batch, int input_dim, int output_dim, int activation, b200rl_stream_t stream){
    if(!W || !bias || !x || !y || batch < 0 || input_dim < 1 || output_dim < 1 || ldx < input_dim || ldy < output_dim || (pre && ldpre < output_dim) || !valid_activation(activation) || x == y)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    return dense_forward_impl(W, bias, x, ldx, pre, ldpre, y, ldy, batch, input_dim, output_dim, activation, (cudaStream_t)stream);
}

size_t b200rl_dense_forward_workspace_bytes(int batch, int input_dim, int output_dim){
    if(batch < 1 || input_dim < 1 || output_dim < 1) return 0;
    return forward_workspace_bytes(batch, input_dim, output_dim);
}
int b200rl_dense_forward_ws(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                            int batch, int input_dim, int output_dim, int activation, void* workspace, size_t workspace_bytes, b200rl_stream_t stream){
    if(!W || !bias || !x || !y || batch < 0 || input_dim < 1 || output_dim < 1 || ldx < input_dim || ldy < output_dim || (pre && ldpre < output_dim) || !valid_activation(activation) || x == y)
        return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    return dense_forward_impl(W, bias, x, ldx, pre, ldpre, y, ldy, batch, input_dim, output_dim, activation, (cudaStream_t)stream, workspace, workspace_bytes);
}

size_t b200rl_dense_backward_scratch_bytes(int batch, int input_dim, int output_dim){
    if(batch < 1 || input_dim < 1 || output_dim < 1) return 0;
    return backward_scratch_total(batch, input_dim, output_dim);
}

int b200rl_dense_backward(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                          float* d_W, float* d_bias, float* d_in, int ldi, int batch, int input_dim, int output_dim, int activation,
                          void* scratch, size_t scratch_bytes, b200rl_stream_t stream){
    if(!W || !pre || !d_out || batch < 0 || input_dim < 1 || output_dim < 1 || ldpre < output_dim || ldd < output_dim || !valid_activation(activation))
        return B200RL_ERR_INVALID_ARGUMENT;
    if((d_W == nullptr) != (d_bias == nullptr)) return B200RL_ERR_INVALID_ARGUMENT;
    if(d_W && (!x || ldx < input_dim)) return B200RL_ERR_INVALID_ARGUMENT;
    if(d_in && ldi < input_dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    return dense_backward_impl(W, x, ldx, pre, ldpre, d_out, ldd, d_W, d_bias, d_in, ldi, batch, input_dim, output_dim, activation, scratch, scratch_bytes, (cudaStream_t)stream);
}

// ---- backward without caller scratch and without allocation ----------------------------------------------------
// The partial sums go to this file-scope device array. In host code its name is only a handle, not a device address:
// the address is looked up once per device with cudaGetSymbolAddress (with that device current) and cached.
static __device__ __align__(256) unsigned char g_static_scratch[B200RL_STATIC_SCRATCH_BYTES];

static int static_scratch_address(void** out){
    static void* cached[MAX_DEVICES] = {};
    static std::mutex mutex;
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    std::lock_guard<std::mutex> lock(mutex);
    if(cached[dev] == nullptr){
        void* p = nullptr;
        B200RL_CUDA_TRY(cudaGetSymbolAddress(&p, g_static_scratch));
        cached[dev] = p;
    }
    *out = cached[dev];
    return B200RL_OK;
}

int b200rl_dense_backward_static_scratch(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                                         float* d_W, float* d_bias, float* d_in, int ldi, int batch, int input_dim, int output_dim,
                                         int activation, b200rl_stream_t stream){
    if(!W || !pre || !d_out || batch < 0 || input_dim < 1 || output_dim < 1 || ldpre < output_dim || ldd < output_dim || !valid_activation(activation))
        return B200RL_ERR_INVALID_ARGUMENT;
    if((d_W == nullptr) != (d_bias == nullptr)) return B200RL_ERR_INVALID_ARGUMENT;
    if(d_W && (!x || ldx < input_dim)) return B200RL_ERR_INVALID_ARGUMENT;
    if(d_in && ldi < input_dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    // The batch is split as far as the array allows (never refused for its batch size); what does not fit at all is a layer whose
    // weight matrix is so large that the array cannot hold two partial sums of its gradient.
    if(d_W && (size_t)input_dim * (size_t)output_dim > B200RL_STATIC_SCRATCH_MAX_WEIGHTS) return B200RL_ERR_SCRATCH_LIMIT;
    void* scratch = nullptr;
    int rc = static_scratch_address(&scratch);
    if(rc) return rc;
    return dense_backward_impl(W, x, ldx, pre, ldpre, d_out, ldd, d_W, d_bias, d_in, ldi, batch, input_dim, output_dim, activation,
                               scratch, B200RL_STATIC_SCRATCH_BYTES, (cudaStream_t)stream, (size_t)B200RL_STATIC_SCRATCH_BYTES);
}

size_t b200rl_mlp_num_params(const b200rl_mlp_shape* sh){
    if(!valid_shape(sh)) return 0;
    size_t n = 0; int in = sh->input_dim;
    for(int l = 0; l < sh->n_layers; l++){ n += (size_t)sh->dims[l] * in + sh->dims[l]; in = sh->dims[l]; }
    return n;
}

size_t b200rl_mlp_forward_workspace_bytes(const b200rl_mlp_shape* sh, int batch){
    if(!valid_shape(sh) || batch < 1) return 0;
    size_t m = 0; int I = sh->input_dim;
    for(int l = 0; l < sh->n_layers; l++){ const size_t b = forward_workspace_bytes(batch, I, sh->dims[l]); if(b > m) m = b; I = sh->dims[l]; }
    return m;
}

int b200rl_mlp_evaluate(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* y, int ldy,
                        float* tick, float* tock, int batch, b200rl_stream_t stream){
    return b200rl_mlp_evaluate_ws(sh, params, x, ldx, y, ldy, tick, tock, batch, nullptr, 0, stream);
}
int b200rl_mlp_evaluate_ws(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* y, int ldy,
                           float* tick, float* tock, int batch, void* workspace, size_t workspace_bytes, b200rl_stream_t stream){
    if(!valid_shape(sh) || !params || !x || !y || batch < 0 || ldx < sh->input_dim || ldy < sh->dims[sh->n_layers - 1]) return B200RL_ERR_INVALID_ARGUMENT;
    if(sh->n_layers > 1 && (!tick || (sh->n_layers > 2 && !tock))) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    if(mlp_fused_eligible(sh, batch)) return mlp_fused_forward(sh, params, x, ldx, nullptr, nullptr, y, ldy, batch, (cudaStream_t)stream);
    if(mlp_coop_eligible(sh, batch, true)) return mlp_coop_forward(sh, params, x, ldx, nullptr, nullptr, y, ldy, tick, tock, batch, (cudaStream_t)stream);
    const float* in = x; int ldin = ldx, I = sh->input_dim; const float* p = params;
    for(int l = 0; l < sh->n_layers; l++){
        int O = sh->dims[l]; bool last = l == sh->n_layers - 1;
        float* out = last ? y : ((l % 2 == 0) ? tick : tock);
        int ldo = last ? ldy : O;
        int rc = dense_forward_impl(p, p + (size_t)O * I, in, ldin, nullptr, 0, out, ldo, batch, I, O, sh->acts[l], (cudaStream_t)stream, workspace, workspace_bytes);
        if(rc) return rc;
        p += (size_t)O * I + O; in = out; ldin = ldo; I = O;
    }
    return B200RL_OK;
}

int b200rl_mlp_forward(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out,
                       int batch, b200rl_stream_t stream){
    return b200rl_mlp_forward_ws(sh, params, x, ldx, pre, out, batch, nullptr, 0, stream);
}
int b200rl_mlp_forward_ws(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out,
                          int batch, void* workspace, size_t workspace_bytes, b200rl_stream_t stream){
    if(!valid_shape(sh) || !params || !x || !pre || !out || batch < 0 || ldx < sh->input_dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    if(mlp_fused_eligible(sh, batch)) return mlp_fused_forward(sh, params, x, ldx, pre, out, nullptr, 0, batch, (cudaStream_t)stream);
    if(mlp_coop_eligible(sh, batch, true)) return mlp_coop_forward(sh, params, x, ldx, pre, out, nullptr, 0, nullptr, nullptr, batch, (cudaStream_t)stream);
    const float* in = x; int ldin = ldx, I = sh->input_dim; const float* p = params;
    for(int l = 0; l < sh->n_layers; l++){
        int O = sh->dims[l];
        int rc = dense_forward_impl(p, p + (size_t)O * I, in, ldin, pre, O, out, O, batch, I, O, sh->acts[l], (cudaStream_t)stream, workspace, workspace_bytes);
        if(rc) return rc;
        p += (size_t)O * I + O; in = out; ldin = O; I = O;
        pre += (size_t)batch * O; out += (size_t)batch * O;
    }
    return B200RL_OK;
}

size_t b200rl_mlp_backward_scratch_bytes(const b200rl_mlp_shape* sh, int batch){
    if(!valid_shape(sh) || batch < 1) return 0;
    size_t m = 0; int I = sh->input_dim;
    for(int l = 0; l < sh->n_layers; l++){ const size_t b = backward_scratch_total(batch, I, sh->dims[l]); if(b > m) m = b; I = sh->dims[l]; }
    const size_t fused = mlp_fused_backward_scratch_bytes(sh, batch);
    return fused > m ? fused : m;
}

int b200rl_mlp_backward(const b200rl_mlp_shape* sh, const float* params, float* grads, const float* x, int ldx, const float* pre,
                        const float* out, float* d_out, float* d_input, float* tick, float* tock, int batch,
                        void* scratch, size_t scratch_bytes, b200rl_stream_t stream){
    if(!valid_shape(sh) || !params || !x || !pre || !out || !d_out || batch < 0 || ldx < sh->input_dim) return B200RL_ERR_INVALID_ARGUMENT;
    if(!grads && !d_input) return B200RL_ERR_INVALID_ARGUMENT;          // grads == NULL: backward_input (nn_models/mlp/operations_generic.h:130-150)
    int L = sh->n_layers;
    if(L > 1 && (!tick || (L > 2 && !tock))) return B200RL_ERR_INVALID_ARGUMENT;
    if(batch == 0) return B200RL_OK;
    // small batches: the whole pass in two launches, when the caller's scratch has room for the gradients of all layers
    if(mlp_fused_eligible(sh, batch) && scratch && scratch_bytes >= mlp_fused_backward_scratch_bytes(sh, batch))
        return mlp_fused_backward(sh, params, grads, x, ldx, pre, out, d_out, d_input, batch, scratch, scratch_bytes, (cudaStream_t)stream);
    if(mlp_coop_eligible(sh, batch, false)) return mlp_coop_backward(sh, params, grads, x, ldx, pre, out, d_out, d_input, tick, tock, batch, (cudaStream_t)stream);
    size_t poff[B200RL_MAX_LAYERS], aoff[B200RL_MAX_LAYERS]; int Is[B200RL_MAX_LAYERS];
    { size_t po = 0, ao = 0; int I = sh->input_dim;
      for(int l = 0; l < L; l++){ poff[l] = po; aoff[l] = ao; Is[l] = I; po += (size_t)sh->dims[l] * I + sh->dims[l]; ao += (size_t)batch * sh->dims[l]; I = sh->dims[l]; } }
    float* d_cur = d_out; int ldd = sh->dims[L - 1];
    for(int l = L - 1; l >= 0; l--){
        int O = sh->dims[l], I = Is[l];
        const float* in = l == 0 ? x : out + aoff[l - 1];
        int ldin = l == 0 ? ldx : I;
        float* d_in = l == 0 ? d_input : ((l % 2 == 0) ? tick : tock);
        float* dW = grads ? grads + poff[l] : nullptr;
        int rc = dense_backward_impl(params + poff[l], in, ldin, pre + aoff[l], O, d_cur, ldd, dW, dW ? dW + (size_t)O * I : nullptr, d_in, I, batch, I, O, sh->acts[l],
                                     scratch, scratch_bytes, (cudaStream_t)stream);
        if(rc) return rc;
        d_cur = d_in; ldd = I;
    }
    return B200RL_OK;
}

}  // extern "C"
