// Backward pass of a dense layer with FEW outputs at a LARGE batch (the last layer of a critic or an actor: O <= 16 outputs, e.g.
// 256 -> 16 at 65,536 rows) in one pass over the layer's input:
//   d_pre = d_out * act'(pre)            [B, O]   (written back over d_out, like the general path)
//   d_b  += column sums of d_pre         [O]
//   d_W  += d_pre^T x                    [O, I]
//   d_in  = d_pre W                      [B, I]
// (nn/layers/dense/operations_generic.h:205-263). As three matrix products this shape is all overhead on the tiled kernels: the
// contraction of d_in is O <= 16 long and the weight gradient has O <= 16 rows, so a tile spends its time in staging rounds and in the
// epilogue. Here a thread owns up to two COLUMNS of the input (column c and c + 128), holds W[:, c] and its slice of the weight gradient
// in registers, and walks over the rows: per row it reads x[row][c] once (coalesced), takes the row of d_pre from shared memory (a
// broadcast), and does 2 x O multiply-adds per column. Every byte of x and d_in crosses HBM once; the algorithmic traffic
// (B x I x 8 bytes) is the roofline.
// Determinism: a CTA owns a fixed range of rows and sums them in ascending order (two row lanes, combined lane 0 + lane 1); the per-CTA
// partial sums are added by the fixed-order reduction kernels of dense.cu.
#include "common.cuh"

namespace b200rl {

namespace {
constexpr int SK_THREADS = 256, SK_COLS = 128, SK_LANES = 2, SK_BLOCK_ROWS = 32, SK_OT = 16, SK_INFLIGHT = 8;      // SK_INFLIGHT: rows a warp keeps in flight
}

// CPT: columns per thread (I <= 128 * CPT). WANT_GRADS: d_W / d_b partial sums. WANT_DIN: the input gradient.
// The CTA's rows are dealt to its two row lanes (rows r0 + lane, + 2, ...); the four warps of a row lane cover the columns. A warp walks
// over its lane's rows eight at a time and stages their d_pre rows into its OWN slice of shared memory (the four warps of a lane compute
// the same 8 x 16 values from d_out and pre, which stay unmodified during the main loop), so the main loop has no CTA-wide barrier and the
// warps drift apart: some wait on their loads while others compute. The write-back of d_pre over d_out and the bias sums follow in a
// second, short phase after a barrier.
template <int ACT, int CPT, bool WANT_GRADS, bool WANT_DIN>
__global__ void __launch_bounds__(SK_THREADS, 2) skinny_backward_kernel(const float* __restrict__ W, const float* __restrict__ x, long long ldx, const float* __restrict__ pre,
                                                                     long long ldpre, float* d_out, long long ldd, float* __restrict__ w_partial, float* __restrict__ b_partial,
                                                                     float* __restrict__ d_in, long long ldi, int B, int I, int O, int rows_per_cta, long long partial_stride){
    __shared__ __align__(16) float dp[SK_THREADS / 32][SK_INFLIGHT][SK_OT];     // per warp: d_pre of its eight rows in flight
    __shared__ float comb[WANT_GRADS ? SK_COLS * CPT * SK_OT : SK_THREADS];      // lane 1's weight-gradient slice for the lane combination; then the bias slots
    const int t = threadIdx.x, lane_row = t / SK_COLS, tc = t % SK_COLS, warp = t >> 5, lane = t & 31;
    const int r0 = blockIdx.x * rows_per_cta, r1 = min(B, r0 + rows_per_cta);
    float w[CPT][SK_OT], gw[CPT][SK_OT];
#pragma unroll
    for(int q = 0; q < CPT; q++){
        const int c = tc + SK_COLS * q;
#pragma unroll
        for(int j = 0; j < SK_OT; j++){
            w[q][j] = (c < I && j < O) ? __ldg(W + (size_t)j * I + c) : 0.0f;
            gw[q][j] = 0.0f;
        }
    }
    float (*my_dp)[SK_OT] = dp[warp];
#pragma unroll 1
    for(int base = r0 + lane_row; base < r1; base += SK_LANES * SK_INFLIGHT){
        float xv[SK_INFLIGHT][CPT];
#pragma unroll
        for(int u = 0; u < SK_INFLIGHT; u++){
            const int row = base + SK_LANES * u;
#pragma unroll
            for(int q = 0; q < CPT; q++){
                const int c = tc + SK_COLS * q;
                xv[u][q] = (WANT_GRADS && row < r1 && c < I) ? __ldg(x + (long long)row * ldx + c) : 0.0f;
            }
        }
        // 8 rows x 16 outputs = 128 values of d_pre, four per lane
        float st[4];
#pragma unroll
        for(int i = 0; i < 4; i++){
            const int e = lane + 32 * i, u = e / SK_OT, j = e % SK_OT, row = base + SK_LANES * u;
            float v = 0.0f;
            if(row < r1 && j < O){
                v = d_out[(long long)row * ldd + j];
                if constexpr(ACT != B200RL_ACT_IDENTITY) v *= d_activation<ACT>(__ldg(pre + (long long)row * ldpre + j));
            }
            st[i] = v;
        }
        __syncwarp();                                  // the previous iteration's reads of my_dp are done
#pragma unroll
        for(int i = 0; i < 4; i++){ const int e = lane + 32 * i; my_dp[e / SK_OT][e % SK_OT] = st[i]; }
        __syncwarp();
#pragma unroll
        for(int u = 0; u < SK_INFLIGHT; u++){
            const int row = base + SK_LANES * u;
            float d[SK_OT];
#pragma unroll
            for(int j4 = 0; j4 < SK_OT / 4; j4++){
                const float4 v = *reinterpret_cast<const float4*>(&my_dp[u][4 * j4]);
                d[4 * j4] = v.x; d[4 * j4 + 1] = v.y; d[4 * j4 + 2] = v.z; d[4 * j4 + 3] = v.w;
            }
#pragma unroll
            for(int q = 0; q < CPT; q++){
                if constexpr(WANT_GRADS){
#pragma unroll
                    for(int j = 0; j < SK_OT; j++) gw[q][j] = fmaf(d[j], xv[u][q], gw[q][j]);
                }
                if constexpr(WANT_DIN){
                    float acc = 0.0f;                                   // outputs ascending: the reference's order (operations_generic.h:247-254)
#pragma unroll
                    for(int j = 0; j < SK_OT; j++) acc = fmaf(d[j], w[q][j], acc);
                    const int c = tc + SK_COLS * q;
                    if(row < r1 && c < I) d_in[(long long)row * ldi + c] = acc;
                }
            }
        }
    }
    __syncthreads();                                   // every warp has read d_out for the last time
    // second phase: d_pre over d_out, and the bias sums: thread = (row slot t / 16, output t % 16), rows r0 + slot, + 16, ... ascending
    {
        const int slot = t / SK_OT, j = t % SK_OT;
        float gb = 0.0f;
        if(j < O){
            constexpr int STEP = SK_THREADS / SK_OT;
            for(int row = r0 + slot; row < r1; row += 4 * STEP){          // four independent loads in flight, summed in ascending row order
                float v[4];
#pragma unroll
                for(int u = 0; u < 4; u++){
                    const int rw = row + u * STEP;
                    v[u] = rw < r1 ? d_out[(long long)rw * ldd + j] : 0.0f;
                    if constexpr(ACT != B200RL_ACT_IDENTITY){ if(rw < r1) v[u] *= d_activation<ACT>(__ldg(pre + (long long)rw * ldpre + j)); }
                }
#pragma unroll
                for(int u = 0; u < 4; u++){
                    const int rw = row + u * STEP;
                    if constexpr(ACT != B200RL_ACT_IDENTITY){ if(rw < r1) d_out[(long long)rw * ldd + j] = v[u]; }
                    gb += v[u];
                }
            }
        }
        if constexpr(WANT_GRADS){
            // lane 0 + lane 1 of the weight gradient (fixed order), then the CTA's record: w_partial[cta * stride + j * I + c], b_partial[cta * stride + j]
            if(lane_row == 1){
#pragma unroll
                for(int q = 0; q < CPT; q++)
#pragma unroll
                    for(int jj = 0; jj < SK_OT; jj++) comb[(q * SK_OT + jj) * SK_COLS + tc] = gw[q][jj];
            }
            __syncthreads();
            if(lane_row == 0){
                float* dst = w_partial + (size_t)blockIdx.x * partial_stride;
#pragma unroll
                for(int q = 0; q < CPT; q++){
                    const int c = tc + SK_COLS * q;
#pragma unroll
                    for(int jj = 0; jj < SK_OT; jj++)
                        if(c < I && jj < O) dst[(size_t)jj * I + c] = gw[q][jj] + comb[(q * SK_OT + jj) * SK_COLS + tc];
                }
            }
            __syncthreads();
            comb[t] = gb;                              // [slot][j]
            __syncthreads();
            if(t < O){
                float sum = 0.0f;
                for(int sl = 0; sl < SK_THREADS / SK_OT; sl++) sum += comb[sl * SK_OT + t];      // slots ascending
                b_partial[(size_t)blockIdx.x * partial_stride + t] = sum;
            }
        }
    }
}

// Eligibility of the one-pass kernel: few outputs, an input row of at most 256 columns, a batch large enough that the tiled kernels'
// fixed costs dominate. The caller provides room for `ctas` partial sums of (O * I + O) floats.
bool skinny_backward_eligible(int B, int I, int O){ return O <= SK_OT && I <= 2 * SK_COLS && B >= 8192; }
size_t skinny_backward_scratch_bytes(int I, int O, int ctas){ return sizeof(float) * (size_t)ctas * ((size_t)O * I + O); }

template <int ACT, int CPT>
static void launch_skinny(bool grads, bool din, int ctas, cudaStream_t s, const float* W, const float* x, long long ldx, const float* pre, long long ldpre, float* d_out,
                          long long ldd, float* wp, float* bp, float* d_in, long long ldi, int B, int I, int O, int rows_per_cta, long long stride){
    if(grads && din) skinny_backward_kernel<ACT, CPT, true, true><<<ctas, SK_THREADS, 0, s>>>(W, x, ldx, pre, ldpre, d_out, ldd, wp, bp, d_in, ldi, B, I, O, rows_per_cta, stride);
    else if(grads)   skinny_backward_kernel<ACT, CPT, true, false><<<ctas, SK_THREADS, 0, s>>>(W, x, ldx, pre, ldpre, d_out, ldd, wp, bp, d_in, ldi, B, I, O, rows_per_cta, stride);
    else             skinny_backward_kernel<ACT, CPT, false, true><<<ctas, SK_THREADS, 0, s>>>(W, x, ldx, pre, ldpre, d_out, ldd, wp, bp, d_in, ldi, B, I, O, rows_per_cta, stride);
}

// partial (or null: input gradient only) receives one record of O * I + O floats per CTA -- the weight-gradient sums [O, I], then the bias
// sums [O] -- which the caller reduces in CTA order; ctas is chosen by the caller (a multiple of the SM count), rows are dealt out in
// contiguous ranges of a multiple of 32.
int skinny_backward_launch(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd, float* partial, float* d_in, int ldi,
                           int B, int I, int O, int act, int ctas, cudaStream_t s){
    float* w_partial = partial;
    float* b_partial = partial ? partial + (size_t)O * I : nullptr;
    const long long stride = (long long)O * I + O;
    const bool grads = w_partial != nullptr, din = d_in != nullptr;
    if(!grads && !din) return B200RL_ERR_INVALID_ARGUMENT;
    const int rows_per_cta = ((B + ctas - 1) / ctas + SK_BLOCK_ROWS - 1) / SK_BLOCK_ROWS * SK_BLOCK_ROWS;
    if(I <= SK_COLS){ B200RL_DISPATCH_ACT(act, (launch_skinny<ACT, 1>(grads, din, ctas, s, W, x, ldx, pre, ldpre, d_out, ldd, w_partial, b_partial, d_in, ldi, B, I, O, rows_per_cta, stride))); }
    else            { B200RL_DISPATCH_ACT(act, (launch_skinny<ACT, 2>(grads, din, ctas, s, W, x, ldx, pre, ldpre, d_out, ldd, w_partial, b_partial, d_in, ldi, B, I, O, rows_per_cta, stride))); }
    B200RL_LAUNCH_CHECK("skinny_backward");
    return B200RL_OK;
}


// ---------------------------------------------------------------------------------------------------------------
// Forward pass of the same shape (O <= 16 outputs, large batch): y = act(x W^T + b), optionally the pre-activations too
// (nn/layers/dense/operations_generic.h:103-160). The layer reads B x I inputs and writes B x O outputs, so it is bound by the read of x;
// on the tiled kernels a tile of 128 rows spends its time in one staging round per 32 columns. Here a warp takes four rows per pass: lane l
// owns columns 4l .. 4l+3 of every 128-column chunk (one 16-byte load per row and chunk, a warp reads whole rows), multiplies them with its
// slice of W (shared memory, padded to 16 outputs) into 4 x 16 partial sums, and the 64 sums are reduced over the 32 lanes by a halving
// exchange (32 + 16 + 8 + 4 + 2 shuffles instead of 64 x 5), after which lane l holds outputs 2 (l % 8), 2 (l % 8) + 1 of row l / 8.
// The summation order is a fixed tree (not the reference's ascending order): same bits on every run, within fp32 rounding of the reference.
// ---------------------------------------------------------------------------------------------------------------
namespace {
constexpr int SF_THREADS = 256, SF_ROWS = 4;
}

template <int ACT, int NCH, bool STORE_PRE>
__global__ void __launch_bounds__(SF_THREADS) skinny_forward_kernel(const float* __restrict__ W, const float* __restrict__ bias, const float* __restrict__ x, long long ldx,
                                                                    float* __restrict__ pre, long long ldpre, float* __restrict__ y, long long ldy, int B, int I, int O){
    extern __shared__ __align__(16) float ws[];                 // [16][128 * NCH], zero where j >= O or k >= I
    constexpr int KP = 128 * NCH;
    for(int idx = threadIdx.x; idx < SK_OT * KP; idx += SF_THREADS){
        const int j = idx / KP, k = idx % KP;
        ws[idx] = (j < O && k < I) ? __ldg(W + (size_t)j * I + k) : 0.0f;
    }
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int groups = (B + SF_ROWS - 1) / SF_ROWS;
    const int jo = 2 * (lane & 7);                               // this lane's two outputs after the reduction
    const float b0 = jo < O ? __ldg(bias + jo) : 0.0f, b1 = jo + 1 < O ? __ldg(bias + jo + 1) : 0.0f;
    auto load_rows = [&](int g, float4 (&dst)[SF_ROWS][NCH]){
#pragma unroll
        for(int r = 0; r < SF_ROWS; r++)
#pragma unroll
            for(int ch = 0; ch < NCH; ch++){
                const int k = 128 * ch + 4 * lane, row = g * SF_ROWS + r;
                dst[r][ch] = (row < B && k < I) ? __ldg(reinterpret_cast<const float4*>(x + (long long)row * ldx + k)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
    };
    const int g_step = gridDim.x * (SF_THREADS / 32);
    for(int g = blockIdx.x * (SF_THREADS / 32) + warp; g < groups; g += g_step){
        const int row0 = g * SF_ROWS;
        float4 xv[SF_ROWS][NCH];
        load_rows(g, xv);
        float v[SF_ROWS * SK_OT];
#pragma unroll
        for(int i = 0; i < SF_ROWS * SK_OT; i++) v[i] = 0.0f;
#pragma unroll
        for(int ch = 0; ch < NCH; ch++)
#pragma unroll
            for(int j = 0; j < SK_OT; j++){
                const float4 w4 = *reinterpret_cast<const float4*>(ws + j * KP + 128 * ch + 4 * lane);
#pragma unroll
                for(int r = 0; r < SF_ROWS; r++){
                    float a = v[r * SK_OT + j];
                    a = fmaf(xv[r][ch].x, w4.x, a); a = fmaf(xv[r][ch].y, w4.y, a); a = fmaf(xv[r][ch].z, w4.z, a); a = fmaf(xv[r][ch].w, w4.w, a);
                    v[r * SK_OT + j] = a;
                }
            }
        // halving exchange: after the step with offset 2^s a lane keeps the half of its values selected by bit s of its index
#pragma unroll
        for(int off = 16, n = 32; off >= 1; off >>= 1, n >>= 1){
            const bool upper = (lane & off) != 0;
#pragma unroll
            for(int i = 0; i < n; i++){
                const float a = v[i], b = v[i + n];
                const float send = upper ? a : b, keep = upper ? b : a;
                v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
            }
        }
        const int row = row0 + (lane >> 3);
        if(row < B){
            const float p0 = v[0] + b0, p1 = v[1] + b1;
            if(jo < O){
                if constexpr(STORE_PRE) pre[(long long)row * ldpre + jo] = p0;
                y[(long long)row * ldy + jo] = activation<ACT>(p0);
            }
            if(jo + 1 < O){
                if constexpr(STORE_PRE) pre[(long long)row * ldpre + jo + 1] = p1;
                y[(long long)row * ldy + jo + 1] = activation<ACT>(p1);
            }
        }
    }
}

bool skinny_forward_eligible(const float* x, int ldx, int B, int I, int O){
    return O <= SK_OT && I <= 256 && I % 4 == 0 && ldx % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && B >= 8192;
}

int skinny_forward_launch(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy, int B, int I, int O, int act, int ctas, cudaStream_t s){
    const int nch = I <= 128 ? 1 : 2;
    const size_t smem = sizeof(float) * SK_OT * 128 * nch;
    if(pre){
        if(nch == 1){ B200RL_DISPATCH_ACT(act, (skinny_forward_kernel<ACT, 1, true><<<ctas, SF_THREADS, smem, s>>>(W, bias, x, ldx, pre, ldpre, y, ldy, B, I, O))); }
        else        { B200RL_DISPATCH_ACT(act, (skinny_forward_kernel<ACT, 2, true><<<ctas, SF_THREADS, smem, s>>>(W, bias, x, ldx, pre, ldpre, y, ldy, B, I, O))); }
    }
    else{
        if(nch == 1){ B200RL_DISPATCH_ACT(act, (skinny_forward_kernel<ACT, 1, false><<<ctas, SF_THREADS, smem, s>>>(W, bias, x, ldx, pre, ldpre, y, ldy, B, I, O))); }
        else        { B200RL_DISPATCH_ACT(act, (skinny_forward_kernel<ACT, 2, false><<<ctas, SF_THREADS, smem, s>>>(W, bias, x, ldx, pre, ldpre, y, ldy, B, I, O))); }
    }
    B200RL_LAUNCH_CHECK("skinny_forward");
    return B200RL_OK;
}

}  // namespace b200rl
