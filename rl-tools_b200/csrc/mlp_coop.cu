// Whole-pass kernels for wide networks at small batches (e.g. 4 -> 256 -> 256 -> 1 at batch 256: the critic of the off-policy algorithms).
//
// At this size a layer's product is a few microseconds of work spread over 64 tiles, and a pass through per-layer kernels is a chain of
// dependent launches (~2.5 us each; five per layer in the backward pass: d_pre and the bias sums, the weight gradient, its reduction, the
// input gradient). The weights (256 KB per 256 x 256 layer) do not fit one CTA, so the pass cannot be a kernel of independent CTAs like the
// one for small networks; here ONE cooperative launch walks a list of phases with a grid-wide barrier between them, and inside a phase the
// CTAs share out the tiles of every product of that phase:
//   forward phase l : out_l = act(in_l W_l^T + b_l)                                   (nn/layers/dense/operations_generic.h:95-132)
//   backward phase l: dW_l += d_pre_l^T in_l, db_l += column sums of d_pre_l, and d_pre_(l-1) = (d_pre_l W_l) * act'(pre_(l-1)), the
//                     derivative folded into the epilogue of the input-gradient tiles (operations_generic.h:151-243)
// A tile is 32 x 32 outputs; the CTA brings both operands of up to 256 summed indices into shared memory with all of its loads in flight
// at once (one L2 round trip per tile instead of one per 16-wide k step), its eight warps take interleaved k and each lane a 4 x 8 patch,
// and the eight partial tiles are added in warp order (deterministic).
//
// The barrier counts arrivals in a device word and spins with a limit; a launch that runs into the limit sets a sticky status word and
// all of its CTAs return. The launch is cooperative, so all CTAs are resident together whatever else the device runs.
#include "common.cuh"
#include <cstdlib>
#include <mutex>
#include <vector>

namespace b200rl {

constexpr int CO_T = 32, CO_KC = 256, CO_PITCH = 36, CO_THREADS = 256, CO_WARPS = 8;
constexpr size_t CO_SMEM = sizeof(float) * 2 * CO_KC * CO_PITCH;          // both operand tiles; the eight partial tiles (32 KB) reuse the space
constexpr unsigned CO_SPIN_LIMIT = 1000000u;                              // polls of the barrier words (two L2 round trips each): about a second
// Barrier words per device, handed out round-robin per launch (a captured launch keeps the slot it got at capture time). Two launches may
// share a slot as long as they never run at the same time: launches on one stream never do, and the parallel branches of one captured graph
// get consecutive slots. What is not supported: two launches whose slots coincide after a wrap of the ring (4,096 launches apart) running
// concurrently on different streams.
constexpr int CO_SLOTS = 4096;

enum { CO_EPI_FORWARD = 0, CO_EPI_DX = 1, CO_EPI_DW = 2 };
struct CoopGemm {                    // C(m, n) = sum_k A(m, k) B(n, k); *_kcontig: the summed index is the contiguous one in memory
    const float* A; const float* B; float* C; float* C2; const float* bias; const float* aux;
    int lda, ldb, ldc, ldc2, ldaux, a_kcontig, b_kcontig, M, N, K, act, epi, accumulate, tiles_n, tiles;
};
enum { CO_PHASE_PRODUCTS = 0, CO_PHASE_DPRE = 1 };
struct CoopPhase {
    int type, n_gemms;
    CoopGemm g[2];
    const float* bias_src; float* bias_dst; int bias_ld, bias_rows, bias_cols, bias_items, bias_accumulate;      // db (+)= column sums
    float* d_out; const float* pre; int ew_ldd, ew_ldpre, ew_rows, ew_cols, ew_act;                              // d_pre of the last layer, in place
};
constexpr int CO_MAX_LAYERS = 4, CO_MAX_PHASES = CO_MAX_LAYERS + 1;
struct CoopArgs { int n_phases; unsigned* barrier; CoopPhase phase[CO_MAX_PHASES]; };
static_assert(sizeof(CoopArgs) <= 4000, "kernel arguments");

static __device__ unsigned g_coop_barriers[CO_SLOTS * 4];                 // per slot: arrivals, exits, status (sticky), unused

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p){
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
// false: the wait ran into its limit (or another CTA's did)
__device__ bool coop_barrier(unsigned* bar, unsigned target){
    __shared__ int ok_s;
    __syncthreads();
    if(threadIdx.x == 0){
        __threadfence();
        atomicAdd(bar, 1u);
        int ok = 1;
        unsigned spins = 0;
        while(ld_acquire_u32(bar) < target){
            if(++spins > CO_SPIN_LIMIT || ld_acquire_u32(bar + 2) != 0u){ atomicExch(bar + 2, 1u); ok = 0; break; }
        }
        ok_s = ok;
    }
    __syncthreads();
    return ok_s != 0;
}

// operand tile: S[k][r] = P(r0 + r, k0 + k) for r < 32, k < kc; zero where the row lies outside the operand. Plain loads throughout this
// file (no read-only path): most operands were written earlier in the same launch by other CTAs, and only the barrier's acquire orders those.
//
// 16-byte form (rows and pitch multiples of four floats): a thread's item u of a batch of eight is element group idx = base + u * 256.
//   summed index contiguous: a warp's request covers 8 rows x 64 bytes (8 cache lines; a lane per row would touch 32), the four values of a
//                            group go to four k rows of the tile (two-way bank conflicts at the pitch of 36)
//   row index contiguous   : 8 lanes x 16 bytes per k, stored as they come
struct CoopVec { const float* P; int ld, kcontig, r0, R, k0, kc, total; };
__device__ __forceinline__ bool coop_vec_ok(const float* P, int ld, int kcontig, int R, int kc){
    return (ld % 4 == 0) && ((reinterpret_cast<uintptr_t>(P) & 15u) == 0) && (kcontig ? kc % 4 == 0 : R % 4 == 0);
}
__device__ __forceinline__ void coop_vec_index(const CoopVec& o, int idx, int& r, int& k){
    if(o.kcontig){ r = (idx & 7) + ((idx >> 5) & 3) * 8; k = (((idx >> 3) & 3) + (idx >> 7) * 4) * 4; }
    else { r = (idx & 7) * 4; k = idx >> 3; }
}
__device__ __forceinline__ void coop_vec_fetch(const CoopVec& o, int base, float4 (&v)[8]){
#pragma unroll
    for(int u = 0; u < 8; u++){
        int r, k;
        coop_vec_index(o, base + u * CO_THREADS, r, k);
        const bool in = base + u * CO_THREADS < o.total && k < o.kc && o.r0 + r < o.R;
        const float* src = o.kcontig ? o.P + (size_t)(o.r0 + r) * o.ld + o.k0 + k : o.P + (size_t)(o.k0 + k) * o.ld + o.r0 + r;
        v[u] = in ? *reinterpret_cast<const float4*>(src) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}
__device__ __forceinline__ void coop_vec_store(const CoopVec& o, int base, float (*S)[CO_PITCH], const float4 (&v)[8]){
#pragma unroll
    for(int u = 0; u < 8; u++){
        int r, k;
        coop_vec_index(o, base + u * CO_THREADS, r, k);
        if(base + u * CO_THREADS >= o.total || k >= o.kc) continue;
        if(o.kcontig){ S[k][r] = v[u].x; S[k + 1][r] = v[u].y; S[k + 2][r] = v[u].z; S[k + 3][r] = v[u].w; }
        else *reinterpret_cast<float4*>(&S[k][r]) = v[u];
    }
}
__device__ __forceinline__ CoopVec coop_vec(const float* P, int ld, int kcontig, int r0, int R, int k0, int kc){
    CoopVec o{P, ld, kcontig, r0, R, k0, kc, 0};
    o.total = kcontig ? 32 * ((kc / 4 + 3) / 4 * 4) : 8 * kc;
    return o;
}
// 4-byte form for everything else (an odd input width, a single output column)
__device__ __forceinline__ void coop_load_scalar(float (*S)[CO_PITCH], const float* P, int ld, int kcontig, int r0, int R, int k0, int kc){
    const int total = 32 * kc;
    for(int base = threadIdx.x; base < total; base += CO_THREADS * 8){
        float v[8];
#pragma unroll
        for(int u = 0; u < 8; u++){
            const int idx = base + u * CO_THREADS, k = kcontig ? idx % kc : idx >> 5, r = kcontig ? idx / kc : idx & 31;
            v[u] = (idx < total && r0 + r < R) ? (kcontig ? P[(size_t)(r0 + r) * ld + k0 + k] : P[(size_t)(k0 + k) * ld + r0 + r]) : 0.0f;
        }
#pragma unroll
        for(int u = 0; u < 8; u++){
            const int idx = base + u * CO_THREADS, k = kcontig ? idx % kc : idx >> 5, r = kcontig ? idx / kc : idx & 31;
            if(idx < total) S[k][r] = v[u];
        }
    }
}
// both operands of a chunk: all loads of a thread are issued before the first store waits for one
__device__ __forceinline__ void coop_load_operands(float (*As)[CO_PITCH], float (*Bs)[CO_PITCH], const CoopGemm& g, int m0, int n0, int k0, int kc){
    const bool va = coop_vec_ok(g.A, g.lda, g.a_kcontig, g.M, kc), vb = coop_vec_ok(g.B, g.ldb, g.b_kcontig, g.N, kc);
    const CoopVec oa = coop_vec(g.A, g.lda, g.a_kcontig, m0, g.M, k0, kc), ob = coop_vec(g.B, g.ldb, g.b_kcontig, n0, g.N, k0, kc);
    if(va && vb){
        const int total = oa.total > ob.total ? oa.total : ob.total;
        for(int base = threadIdx.x; base < total; base += CO_THREADS * 8){
            float4 ra[8], rb[8];
            coop_vec_fetch(oa, base, ra);
            coop_vec_fetch(ob, base, rb);
            coop_vec_store(oa, base, As, ra);
            coop_vec_store(ob, base, Bs, rb);
        }
        return;
    }
    if(va){ for(int base = threadIdx.x; base < oa.total; base += CO_THREADS * 8){ float4 ra[8]; coop_vec_fetch(oa, base, ra); coop_vec_store(oa, base, As, ra); } }
    else coop_load_scalar(As, g.A, g.lda, g.a_kcontig, m0, g.M, k0, kc);
    if(vb){ for(int base = threadIdx.x; base < ob.total; base += CO_THREADS * 8){ float4 rb[8]; coop_vec_fetch(ob, base, rb); coop_vec_store(ob, base, Bs, rb); } }
    else coop_load_scalar(Bs, g.B, g.ldb, g.b_kcontig, n0, g.N, k0, kc);
}

__device__ void coop_gemm_tile(const CoopGemm& g, int tile, float* smem){
    float (*As)[CO_PITCH] = reinterpret_cast<float (*)[CO_PITCH]>(smem);
    float (*Bs)[CO_PITCH] = As + CO_KC;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, rg = lane >> 2, cg = lane & 3;
    const int m0 = (tile / g.tiles_n) * CO_T, n0 = (tile % g.tiles_n) * CO_T;
    float acc[4][8];
#pragma unroll
    for(int i = 0; i < 4; i++)
#pragma unroll
        for(int j = 0; j < 8; j++) acc[i][j] = 0.0f;
    for(int k0 = 0; k0 < g.K; k0 += CO_KC){
        const int kc = min(CO_KC, g.K - k0);
        __syncthreads();                                   // whoever read this shared memory last (previous item, previous chunk) is done
        coop_load_operands(As, Bs, g, m0, n0, k0, kc);
        __syncthreads();
#pragma unroll 4
        for(int k = warp; k < kc; k += CO_WARPS){
            const float4 a = *reinterpret_cast<const float4*>(&As[k][4 * rg]);
            const float4 b0 = *reinterpret_cast<const float4*>(&Bs[k][8 * cg]), b1 = *reinterpret_cast<const float4*>(&Bs[k][8 * cg + 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
            for(int i = 0; i < 4; i++)
#pragma unroll
                for(int j = 0; j < 8; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
    }
    __syncthreads();
    float* R = smem;                                       // [warp][32][32]
#pragma unroll
    for(int i = 0; i < 4; i++){
        float* row = R + (warp * CO_T + 4 * rg + i) * CO_T + 8 * cg;
        *reinterpret_cast<float4*>(row) = make_float4(acc[i][0], acc[i][1], acc[i][2], acc[i][3]);
        *reinterpret_cast<float4*>(row + 4) = make_float4(acc[i][4], acc[i][5], acc[i][6], acc[i][7]);
    }
    __syncthreads();
    const int r = tid >> 3, c4 = (tid & 7) * 4, m = m0 + r;
    float v[4] = {0.0f, 0.0f, 0.0f, 0.0f};
#pragma unroll
    for(int w = 0; w < CO_WARPS; w++){
        const float4 p = *reinterpret_cast<const float4*>(R + (w * CO_T + r) * CO_T + c4);
        v[0] += p.x; v[1] += p.y; v[2] += p.z; v[3] += p.w;
    }
    if(m >= g.M) return;
#pragma unroll
    for(int j = 0; j < 4; j++){
        const int n = n0 + c4 + j;
        if(n >= g.N) continue;
        float s = v[j];
        if(g.epi == CO_EPI_FORWARD){
            s += g.bias[n];
            if(g.C2) g.C2[(size_t)m * g.ldc2 + n] = s;
            g.C[(size_t)m * g.ldc + n] = activation_rt(s, g.act);
        }
        else if(g.epi == CO_EPI_DX){
            if(g.aux) s *= d_activation_rt(g.aux[(size_t)m * g.ldaux + n], g.act);      // plain load: written earlier in this launch by other CTAs
            g.C[(size_t)m * g.ldc + n] = s;
        }
        else{
            float* dst = g.C + (size_t)m * g.ldc + n;
            *dst = g.accumulate ? *dst + s : s;
        }
    }
}

// 32 columns of the bias gradient: eight row lanes per column, added in lane order
__device__ void coop_bias_item(const CoopPhase& p, int item, float* smem){
    const int tid = threadIdx.x, c = tid & 31, seg = tid >> 5, col = item * 32 + c;
    float s = 0.0f;
    if(col < p.bias_cols)
        for(int b = seg; b < p.bias_rows; b += CO_WARPS) s += p.bias_src[(size_t)b * p.bias_ld + col];
    __syncthreads();
    smem[seg * 32 + c] = s;
    __syncthreads();
    if(tid < 32 && col < p.bias_cols){
        float t = 0.0f;
#pragma unroll
        for(int w = 0; w < CO_WARPS; w++) t += smem[w * 32 + tid];
        p.bias_dst[col] = p.bias_accumulate ? p.bias_dst[col] + t : t;
    }
}

__global__ void __launch_bounds__(CO_THREADS, 1) mlp_coop_kernel(CoopArgs a){
    extern __shared__ __align__(16) float smem[];
    unsigned target = 0;
    for(int ph = 0; ph < a.n_phases; ph++){
        const CoopPhase& p = a.phase[ph];
        if(p.type == CO_PHASE_DPRE){
            const int total = p.ew_rows * p.ew_cols;
            for(int idx = blockIdx.x * CO_THREADS + threadIdx.x; idx < total; idx += gridDim.x * CO_THREADS){
                const int r = idx / p.ew_cols, c = idx % p.ew_cols;
                float* d = p.d_out + (size_t)r * p.ew_ldd + c;
                *d = *d * d_activation_rt(p.pre[(size_t)r * p.ew_ldpre + c], p.ew_act);
            }
        }
        else{
            const int t0 = p.g[0].tiles, t1 = p.n_gemms > 1 ? p.g[1].tiles : 0, items = t0 + t1 + p.bias_items;
            for(int item = blockIdx.x; item < items; item += gridDim.x){
                if(item < t0) coop_gemm_tile(p.g[0], item, smem);
                else if(item < t0 + t1) coop_gemm_tile(p.g[1], item - t0, smem);
                else coop_bias_item(p, item - t0 - t1, smem);
            }
        }
        if(ph + 1 < a.n_phases){
            target += gridDim.x;
            if(!coop_barrier(a.barrier, target)) return;
        }
    }
    // the last CTA out clears the slot for its next launch (every CTA has left the last barrier before it counts itself out)
    if(threadIdx.x == 0 && a.n_phases > 1){
        const unsigned old = atomicAdd(a.barrier + 1, 1u);
        if(old == gridDim.x - 1){ a.barrier[0] = 0u; a.barrier[1] = 0u; __threadfence(); }
    }
}

// ---------------------------------------------------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------------------------------------------------
bool mlp_fused_eligible(const b200rl_mlp_shape* sh, int batch);

// Which passes run here. Measured on the 4 -> 256 -> 256 -> 1 critic at batch 256 inside captured graphs: the backward pass 39 -> 22 us, the
// forward pass 19.4 -> 19 us (three launches against three phases: a tie), and the off-policy update as a whole is faster with the forward
// pass on the per-layer kernels. So the backward pass is the default; B200RL_COOPERATIVE_PASS=0 keeps every pass on the per-layer kernels,
// =2 also takes forward / evaluate here (both for measurements).
static int coop_mode(){
    static const int mode = [](){ const char* e = getenv("B200RL_COOPERATIVE_PASS"); return !e ? 1 : e[0] == '0' ? 0 : e[0] == '2' ? 2 : 1; }();
    return mode;
}
bool mlp_coop_eligible(const b200rl_mlp_shape* sh, int batch, bool forward){
    if(coop_mode() < (forward ? 2 : 1) || batch < 1 || batch > 512 || sh->n_layers > CO_MAX_LAYERS || sh->input_dim > 512 || mlp_fused_eligible(sh, batch)) return false;
    for(int l = 0; l < sh->n_layers; l++) if(sh->dims[l] > 512) return false;
    return true;
}

static int coop_slot(unsigned** out){
    static unsigned* base[MAX_DEVICES] = {};
    static unsigned next[MAX_DEVICES] = {};
    static std::mutex mutex;
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    std::lock_guard<std::mutex> lock(mutex);
    if(base[dev] == nullptr){
        void* p = nullptr;
        B200RL_CUDA_TRY(cudaGetSymbolAddress(&p, g_coop_barriers));
        base[dev] = static_cast<unsigned*>(p);
    }
    *out = base[dev] + 4 * (next[dev]++ % CO_SLOTS);
    return B200RL_OK;
}

static void set_tiles(CoopGemm& g){ g.tiles_n = (g.N + CO_T - 1) / CO_T; g.tiles = ((g.M + CO_T - 1) / CO_T) * g.tiles_n; }

static int coop_launch(CoopArgs& a, cudaStream_t s){
    int sms = 0;
    int rc = sm_count(&sms);
    if(rc) return rc;
    int most = 1;
    for(int ph = 0; ph < a.n_phases; ph++){
        const CoopPhase& p = a.phase[ph];
        const int items = p.type == CO_PHASE_DPRE ? (p.ew_rows * p.ew_cols + CO_THREADS - 1) / CO_THREADS
                                                  : p.g[0].tiles + (p.n_gemms > 1 ? p.g[1].tiles : 0) + p.bias_items;
        if(items > most) most = items;
    }
    const int grid = most < sms ? most : sms;
    rc = coop_slot(&a.barrier);
    if(rc) return rc;
    B200RL_CUDA_TRY(cudaFuncSetAttribute(mlp_coop_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)CO_SMEM));
    void* params[] = { &a };
    B200RL_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void*>(mlp_coop_kernel), dim3(grid), dim3(CO_THREADS), params, CO_SMEM, s));
    return B200RL_OK;
}

// pre / out: per-layer [batch, dims[l]] blocks one after the other (pre may be null: evaluate); the last layer's output goes to y when given
int mlp_coop_forward(const b200rl_mlp_shape* sh, const float* params, const float* x, int ldx, float* pre, float* out, float* y, int ldy,
                     float* tick, float* tock, int batch, cudaStream_t s){
    CoopArgs a{};
    const float* in = x; int ldin = ldx, I = sh->input_dim; const float* p = params;
    for(int l = 0; l < sh->n_layers; l++){
        const int O = sh->dims[l]; const bool last = l == sh->n_layers - 1;
        CoopPhase& ph = a.phase[a.n_phases++];
        ph.type = CO_PHASE_PRODUCTS; ph.n_gemms = 1;
        CoopGemm& g = ph.g[0];
        g.A = in; g.lda = ldin; g.a_kcontig = 1; g.B = p; g.ldb = I; g.b_kcontig = 1; g.M = batch; g.N = O; g.K = I;
        g.bias = p + (size_t)O * I; g.act = sh->acts[l]; g.epi = CO_EPI_FORWARD;
        if(out){ g.C = (last && y) ? y : out; g.ldc = (last && y) ? ldy : O; g.C2 = pre; g.ldc2 = O; }
        else   { g.C = last ? y : ((l % 2 == 0) ? tick : tock); g.ldc = last ? ldy : O; g.C2 = nullptr; }
        set_tiles(g);
        in = g.C; ldin = g.ldc; p += (size_t)O * I + O; I = O;
        if(out){ out += (size_t)batch * O; pre += (size_t)batch * O; }
    }
    return coop_launch(a, s);
}

int mlp_coop_backward(const b200rl_mlp_shape* sh, const float* params, float* grads, const float* x, int ldx, const float* pre, const float* out,
                      float* d_out, float* d_input, float* tick, float* tock, int batch, cudaStream_t s){
    const int L = sh->n_layers;
    size_t poff[CO_MAX_LAYERS], aoff[CO_MAX_LAYERS]; int Is[CO_MAX_LAYERS];
    { size_t po = 0, ao = 0; int I = sh->input_dim;
      for(int l = 0; l < L; l++){ poff[l] = po; aoff[l] = ao; Is[l] = I; po += (size_t)sh->dims[l] * I + sh->dims[l]; ao += (size_t)batch * sh->dims[l]; I = sh->dims[l]; } }
    CoopArgs a{};
    {
        CoopPhase& ph = a.phase[a.n_phases++];
        ph.type = CO_PHASE_DPRE; ph.d_out = d_out; ph.pre = pre + aoff[L - 1]; ph.ew_ldd = sh->dims[L - 1]; ph.ew_ldpre = sh->dims[L - 1];
        ph.ew_rows = batch; ph.ew_cols = sh->dims[L - 1]; ph.ew_act = sh->acts[L - 1];
    }
    const float* d_cur = d_out; int ldd = sh->dims[L - 1];
    for(int l = L - 1; l >= 0; l--){
        const int O = sh->dims[l], I = Is[l];
        const float* in = l == 0 ? x : out + aoff[l - 1];
        const int ldin = l == 0 ? ldx : I;
        float* d_in = l == 0 ? d_input : ((l % 2 == 0) ? tick : tock);
        if(!grads && !d_in) break;
        CoopPhase& ph = a.phase[a.n_phases++];
        ph.type = CO_PHASE_PRODUCTS; ph.n_gemms = 0;
        if(grads){
            CoopGemm& g = ph.g[ph.n_gemms++];
            g.A = d_cur; g.lda = ldd; g.a_kcontig = 0; g.B = in; g.ldb = ldin; g.b_kcontig = 0; g.M = O; g.N = I; g.K = batch;
            g.C = grads + poff[l]; g.ldc = I; g.epi = CO_EPI_DW; g.accumulate = 1;
            set_tiles(g);
            ph.bias_src = d_cur; ph.bias_ld = ldd; ph.bias_rows = batch; ph.bias_cols = O; ph.bias_dst = grads + poff[l] + (size_t)O * I;
            ph.bias_items = (O + 31) / 32; ph.bias_accumulate = 1;
        }
        if(d_in){
            CoopGemm& g = ph.g[ph.n_gemms++];
            g.A = d_cur; g.lda = ldd; g.a_kcontig = 1; g.B = params + poff[l]; g.ldb = I; g.b_kcontig = 0; g.M = batch; g.N = I; g.K = O;
            g.C = d_in; g.ldc = I; g.epi = CO_EPI_DX;
            if(l > 0){ g.aux = pre + aoff[l - 1]; g.ldaux = I; g.act = sh->acts[l - 1]; }
            set_tiles(g);
        }
        d_cur = d_in; ldd = I;
    }
    return coop_launch(a, s);
}

}  // namespace b200rl

// 0: no barrier of a whole-pass launch on the current device ever ran into its limit
extern "C" int b200rl_cooperative_pass_status(int* status){
    using namespace b200rl;
    if(!status) return B200RL_ERR_INVALID_ARGUMENT;
    void* p = nullptr;
    B200RL_CUDA_TRY(cudaGetSymbolAddress(&p, g_coop_barriers));
    std::vector<unsigned> host(CO_SLOTS * 4);
    B200RL_CUDA_TRY(cudaMemcpy(host.data(), p, host.size() * sizeof(unsigned), cudaMemcpyDeviceToHost));
    *status = 0;
    for(int i = 0; i < CO_SLOTS; i++) if(host[4 * i + 2] != 0u) *status = 1;
    return B200RL_OK;
}
