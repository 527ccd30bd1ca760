// Tensor-core Pendulum rollout for the 3 -> 64 -> 64 -> 1 actor (sm_100a, tcgen05 + TMEM).
//
// One persistent CTA per SM, 512 threads = 4 independent groups of 128 threads. A group owns a tile of up to 128
// environments for all T steps; thread r of the group owns environment r of the tile, which is row r of the MMA and
// lane r of tensor memory. The environments of a launch are spread evenly over all 4 x (#CTAs) groups (tiles of
// <= 128 environments, a multiple of 4), so every SM carries the same load and there is a single wave.
// Per step and group:
//   1. thread: reset-if-truncated, sincos, observation; first layer (K = 3) on CUDA cores with packed fp32x2 FMAs;
//      h1 is written RAW to tensor memory (A_hi: the tensor core reads the top 19 bits = the tf32 "hi" part) and the
//      remainder lo = h1 - tf32_trunc(h1) into a K-major, 128-byte-swizzled shared-memory tile (A_lo)
//   2. the group's leader issues 24 tcgen05.mma (M128 N64 K8, kind::tf32): A_lo*B_hi + A_hi*B_lo + A_hi*B_hi over
//      K = 64 ("3xTF32": the dropped lo*lo term is ~2^-22 relative, so the fp32 accumulator matches an fp32 GEMM to
//      ~1e-6), then tcgen05.commit -> the group's mbarrier
//   3. every thread waits (bounded), reads its accumulator row from TMEM (tcgen05.ld), applies bias + activation and
//      the 64 -> 1 output layer, then steps the environment in registers.
// While one group waits for the tensor core the other three run their CUDA-core phases. The second-layer weights
// (tf32 hi and lo parts, the B operand) stay resident in shared memory for the whole launch and are shared by the
// four groups. Tensor memory: 512 columns = 4 groups x (64 accumulator + 64 A_hi columns).
#include "common.cuh"
#include "pendulum.cuh"
#include "rollout.cuh"
#include "tcgen05.cuh"

namespace b200rl {

namespace {
constexpr int H = 64, TILE = 128, GROUPS = 4, THREADS = GROUPS * TILE;
constexpr uint32_t A_KBLOCK_BYTES = TILE * 128;        // 128 rows x 128 B (32 tf32 along K)
constexpr uint32_t B_KBLOCK_BYTES = H * 128;           // 64 rows x 128 B
constexpr uint32_t OFF_B_HI = 0, OFF_B_LO = 2 * B_KBLOCK_BYTES, OFF_A_LO = 4 * B_KBLOCK_BYTES;
constexpr uint32_t A_LO_BYTES = 2 * A_KBLOCK_BYTES;           // per group
constexpr uint32_t OFF_L1 = OFF_A_LO + GROUPS * A_LO_BYTES;   // per pair of hidden units: {w0a,w0b,w1a,w1b} {w2a,w2b,b1a,b1b}
constexpr uint32_t OFF_L3 = OFF_L1 + (H / 2) * 32;            // per pair: {b2a, b2b, w3a, w3b}
constexpr uint32_t OFF_B3 = OFF_L3 + (H / 2) * 16;
constexpr uint32_t OFF_MBAR = OFF_B3 + 16;
constexpr uint32_t OFF_ABORT = OFF_MBAR + 8 * GROUPS;
constexpr uint32_t OFF_SLOT = OFF_ABORT + 4 * GROUPS;
constexpr uint32_t SMEM_BYTES = OFF_SLOT + 16 + 1024;         // + slack to align the base to 1024 B
constexpr uint32_t TMEM_COLS = 512, TMEM_COLS_PER_GROUP = 128;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;        // ~1 s: far beyond any legitimate wait
constexpr uint32_t TF32_MASK = 0xFFFFE000u;
}

template <int ACT>
__device__ __forceinline__ float act_or_rt(float x, int rt){
    if constexpr(ACT >= 0) return activation<ACT>(x);
    else return activation_rt(x, rt);
}

template <int A1, int A2>
__global__ void __launch_bounds__(THREADS, 1) rollout_tc_kernel(RolloutArgs a, int n_tiles, int envs_per_tile){
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, g = tid >> 7, r = tid & 127, warp = tid >> 5;
    const float4* L1 = reinterpret_cast<const float4*>(base + OFF_L1);
    const float4* L3 = reinterpret_cast<const float4*>(base + OFF_L3);
    const float* B3 = reinterpret_cast<const float*>(base + OFF_B3);
    uint64_t* mbar = reinterpret_cast<uint64_t*>(base + OFF_MBAR) + g;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + OFF_ABORT) + g;
    uint32_t* slot = reinterpret_cast<uint32_t*>(base + OFF_SLOT);

    // ---- one-time staging of the actor: arena = W1[64,3] b1[64] W2[64,64] b2[64] W3[1,64] b3[1] ----
    const float* P = a.params;
    if(tid < H / 2){
        const int j = 2 * tid;
        float4* l1 = reinterpret_cast<float4*>(base + OFF_L1);
        l1[2 * tid]     = make_float4(__ldg(P + j * 3), __ldg(P + (j + 1) * 3), __ldg(P + j * 3 + 1), __ldg(P + (j + 1) * 3 + 1));
        l1[2 * tid + 1] = make_float4(__ldg(P + j * 3 + 2), __ldg(P + (j + 1) * 3 + 2), __ldg(P + 192 + j), __ldg(P + 192 + j + 1));
        reinterpret_cast<float4*>(base + OFF_L3)[tid] = make_float4(__ldg(P + 4352 + j), __ldg(P + 4352 + j + 1), __ldg(P + 4416 + j), __ldg(P + 4416 + j + 1));
    }
    if(tid == 0) *reinterpret_cast<float*>(base + OFF_B3) = __ldg(P + 4480);
    for(int idx = tid; idx < H * H; idx += THREADS){
        const int j = idx >> 6, k = idx & 63;                 // W2[j][k]: row j of the B operand, K index k
        const float w = __ldg(P + 256 + idx);
        const float hi = __uint_as_float(__float_as_uint(w) & TF32_MASK);
        const uint32_t off = (uint32_t)(k >> 5) * B_KBLOCK_BYTES + (uint32_t)j * 128 + ((((uint32_t)(k & 31) >> 2) ^ ((uint32_t)j & 7)) << 4) + ((uint32_t)k & 3) * 4;
        *reinterpret_cast<float*>(base + OFF_B_HI + off) = hi;
        *reinterpret_cast<float*>(base + OFF_B_LO + off) = w - hi;
    }
    if(r == 0){ tc::mbar_init(mbar, 1); *abort_flag = 0; }
    if(tid == 0) tc::fence_mbar_init();
    if(warp == 0){ tc::tmem_alloc(slot, TMEM_COLS); tc::tmem_relinquish(); }
    tc::fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = *slot;
    const uint32_t tmem_d = tmem_base + (uint32_t)g * TMEM_COLS_PER_GROUP;          // accumulator: 64 columns
    const uint32_t tmem_a = tmem_d + 64;                                            // A_hi: 64 columns
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;                    // this warp's lane quarter
    uint8_t* a_lo = base + OFF_A_LO + (uint32_t)g * A_LO_BYTES;
    const uint64_t desc_a_lo = tc::make_desc_kmajor_sw128(tc::smem_u32(a_lo));
    const uint64_t desc_b_hi = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_HI)), desc_b_lo = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_LO));
    constexpr uint32_t IDESC = tc::make_idesc_tf32(TILE, H);
    uint8_t* my_row_lo = a_lo + r * 128;
    const uint32_t swz = (uint32_t)r & 7;
    const int act1 = a.acts[0], act2 = a.acts[1], act3 = a.acts[2];
    const uint32_t bar_id = 1 + g;
    uint32_t phase = 0;
    bool failed = false;

    for(int tile = blockIdx.x * GROUPS + g; tile < n_tiles && !failed; tile += gridDim.x * GROUPS){
        const int local = tile * envs_per_tile + r;
        const bool valid = r < envs_per_tile && local < a.env_count;
        const int e = a.env_begin + (valid ? local : 0);
        float theta = 0.0f, theta_dot = 0.0f, er = 0.0f; int es = 0, resets = 0; bool trunc = false;
        if(valid){
            theta = a.states[2 * e]; theta_dot = a.states[2 * e + 1];
            es = a.episode_step[e]; trunc = a.truncated[e] != 0; er = a.episode_return[e];
            resets = a.reset_count ? a.reset_count[e] : 0;
        }
        for(int t = 0; t < a.n_steps; t++){
            if(trunc){
                if(a.reset_states != nullptr && resets < a.n_reset_rounds){
                    const float2 rs = *reinterpret_cast<const float2*>(a.reset_states + ((size_t)resets * a.n_envs + e) * 2);
                    theta = rs.x; theta_dot = rs.y;
                }
                else if(a.error_flag) *a.error_flag = 1;
                resets++; es = 0; er = 0.0f;
            }
            float sn, cs;
            sincosf(theta, &sn, &cs);
            const size_t row = (size_t)t * a.n_envs + e;
            if(valid){ a.obs[row * 3 + 0] = cs; a.obs[row * 3 + 1] = sn; a.obs[row * 3 + 2] = theta_dot; }

            // ---- layer 1 (CUDA cores, two hidden units per packed FMA); A_hi -> TMEM, A_lo -> swizzled smem ----
            const float2 cs2 = make_float2(cs, cs), sn2 = make_float2(sn, sn), td2 = make_float2(theta_dot, theta_dot);
#pragma unroll
            for(int hb = 0; hb < 2; hb++){               // K-block hb = hidden units 32 hb .. 32 hb + 31
                uint32_t hraw[32];
#pragma unroll
                for(int c = 0; c < 8; c++){              // 16-byte chunk c of the K-block: units 4c .. 4c+3
                    float lo[4];
#pragma unroll
                    for(int q = 0; q < 2; q++){
                        const int pp = hb * 16 + c * 2 + q;
                        const float4 w01 = L1[2 * pp], w2b = L1[2 * pp + 1];
                        float2 acc = make_float2(w2b.z, w2b.w);
                        acc = __ffma2_rn(make_float2(w01.x, w01.y), cs2, acc);
                        acc = __ffma2_rn(make_float2(w01.z, w01.w), sn2, acc);
                        acc = __ffma2_rn(make_float2(w2b.x, w2b.y), td2, acc);
                        const float h0 = act_or_rt<A1>(acc.x, act1), h1 = act_or_rt<A1>(acc.y, act1);
                        const uint32_t u0 = __float_as_uint(h0), u1 = __float_as_uint(h1);
                        hraw[c * 4 + q * 2] = u0; hraw[c * 4 + q * 2 + 1] = u1;
                        const float2 l = __fadd2_rn(make_float2(h0, h1),
                                                    make_float2(__uint_as_float((u0 & TF32_MASK) ^ 0x80000000u), __uint_as_float((u1 & TF32_MASK) ^ 0x80000000u)));
                        lo[q * 2] = l.x; lo[q * 2 + 1] = l.y;
                    }
                    *reinterpret_cast<float4*>(my_row_lo + hb * A_KBLOCK_BYTES + (((uint32_t)c ^ swz) << 4)) = make_float4(lo[0], lo[1], lo[2], lo[3]);
                }
                tc::tmem_st_32x32(tmem_a + lane_off + hb * 32, hraw);
            }
            tc::tmem_wait_st();
            tc::fence_proxy_async_smem();
            tc::fence_before_thread_sync();
            tc::named_barrier_sync(bar_id, TILE);
            if(*abort_flag){ failed = true; break; }

            // ---- layer 2 on the tensor core: D[128x64] = A_lo*B_hi + A_hi*B_lo + A_hi*B_hi ----
            if(r == 0){
                tc::fence_after_thread_sync();
#pragma unroll
                for(int kb = 0; kb < 2; kb++)
#pragma unroll
                    for(int ks = 0; ks < 4; ks++)
                        tc::mma_tf32_ss(tmem_d, desc_a_lo + (uint64_t)(kb * (A_KBLOCK_BYTES >> 4) + ks * 2), desc_b_hi + (uint64_t)(kb * (B_KBLOCK_BYTES >> 4) + ks * 2), IDESC, (kb | ks) ? 1u : 0u);
#pragma unroll
                for(int pass = 0; pass < 2; pass++){
                    const uint64_t db = pass == 0 ? desc_b_lo : desc_b_hi;
#pragma unroll
                    for(int kb = 0; kb < 2; kb++)
#pragma unroll
                        for(int ks = 0; ks < 4; ks++)
                            tc::mma_tf32_ts(tmem_d, tmem_a + (uint32_t)(kb * 32 + ks * 8), db + (uint64_t)(kb * (B_KBLOCK_BYTES >> 4) + ks * 2), IDESC, 1u);
                }
                tc::commit(mbar);
            }
            if(!tc::mbar_wait_bounded(mbar, phase, WAIT_LIMIT_CYCLES)){
                *abort_flag = 1;                              // seen by the whole group after its next barrier
                if(a.error_flag) *a.error_flag = 2;
            }
            phase ^= 1;
            tc::fence_after_thread_sync();

            // ---- epilogue: bias + activation of layer 2, output layer 64 -> 1 (two partial sums, packed) ----
            float2 out2 = make_float2(0.0f, 0.0f);
#pragma unroll
            for(int half = 0; half < 2; half++){
                uint32_t d[32];
                tc::tmem_ld_32x32(tmem_d + lane_off + half * 32, d);
                tc::tmem_wait_ld();
#pragma unroll
                for(int p = 0; p < 16; p++){
                    const float4 bw = L3[half * 16 + p];
                    const float2 pre = __fadd2_rn(make_float2(__uint_as_float(d[2 * p]), __uint_as_float(d[2 * p + 1])), make_float2(bw.x, bw.y));
                    out2 = __ffma2_rn(make_float2(bw.z, bw.w), make_float2(act_or_rt<A2>(pre.x, act2), act_or_rt<A2>(pre.y, act2)), out2);
                }
            }
            const float action = activation_rt(B3[0] + (out2.x + out2.y), act3);

            float nt, ntd;
            pendulum::step(theta, theta_dot, sn, action, nt, ntd);
            const float rwd = pendulum::reward(theta, theta_dot, action);
            if(valid){ a.act[row] = action; a.rew[row] = rwd; }
            es += 1; er = __fadd_rn(er, rwd);
            trunc = (es == a.step_limit);
            theta = nt; theta_dot = ntd;
        }
        if(valid && !failed){
            a.states[2 * e] = theta; a.states[2 * e + 1] = theta_dot;
            a.episode_step[e] = es; a.truncated[e] = trunc ? 1 : 0; a.episode_return[e] = er;
            if(a.reset_count) a.reset_count[e] = resets;
        }
    }
    if(failed) tc::mbar_wait_bounded(mbar, phase ^ 1, WAIT_LIMIT_CYCLES);   // give in-flight MMAs a bounded chance to drain
    tc::fence_before_thread_sync();
    __syncthreads();
    if(warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

template <int A1, int A2>
static int launch_tc(const RolloutArgs& a, cudaStream_t s){
    static bool configured = false;
    if(!configured){
        B200RL_CUDA_TRY(cudaFuncSetAttribute(rollout_tc_kernel<A1, A2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        configured = true;
    }
    // spread the environments evenly over every group of every SM: tiles of <= 128 environments (a multiple of 4)
    const int groups_total = NUM_SMS * GROUPS;
    int ept = ((a.env_count + groups_total - 1) / groups_total + 3) / 4 * 4;
    if(ept < 32) ept = 32;
    if(ept > TILE) ept = TILE;
    const int n_tiles = (a.env_count + ept - 1) / ept;
    int grid = (n_tiles + GROUPS - 1) / GROUPS;
    if(grid > NUM_SMS) grid = NUM_SMS;
    rollout_tc_kernel<A1, A2><<<grid, THREADS, SMEM_BYTES, s>>>(a, n_tiles, ept);
    B200RL_LAUNCH_CHECK("rollout_tc");
    return B200RL_OK;
}

int launch_rollout_tc(const RolloutArgs& a, cudaStream_t s){
    const int a1 = a.acts[0], a2 = a.acts[1];
    if(a1 == B200RL_ACT_RELU && a2 == B200RL_ACT_RELU) return launch_tc<B200RL_ACT_RELU, B200RL_ACT_RELU>(a, s);
    if(a1 == B200RL_ACT_TANH && a2 == B200RL_ACT_TANH) return launch_tc<B200RL_ACT_TANH, B200RL_ACT_TANH>(a, s);
    return launch_tc<-1, -1>(a, s);
}

}  // namespace b200rl
