// Tensor-core Pendulum rollout for the 3 -> 64 -> 64 -> 1 actor (sm_100a, tcgen05 + TMEM).
//
// One CTA (128 threads) owns a tile of 128 environments for all T steps; thread i owns environment i of the tile,
// which is also row i of the MMA and lane i of the TMEM accumulator. Per step:
//   1. thread: reset-if-truncated, sincos, observation -> HBM; first layer (K = 3) on CUDA cores;
//      h1 is split into tf32 hi/lo parts and written into the K-major, 128-byte-swizzled A tiles in shared memory
//   2. one thread issues 24 tcgen05.mma (M128 N64 K8, kind::tf32): lo*hi + hi*lo + hi*hi over K = 64
//      ("3xTF32": the dropped lo*lo term is ~2^-22 relative, so the fp32 accumulator matches an fp32 GEMM to ~1e-6)
//   3. tcgen05.commit -> mbarrier; every thread waits (bounded), reads its accumulator row from TMEM (tcgen05.ld),
//      applies bias + activation, the 64 -> 1 output layer, then steps the environment in registers.
// The second-layer weights (hi and lo parts) stay resident in shared memory as the B operand for the whole launch;
// two CTAs fit per SM (~99 KB shared memory, 64 TMEM columns each), so one CTA's CUDA-core phase overlaps the other's
// tensor-core phase.
#include "common.cuh"
#include "pendulum.cuh"
#include "rollout.cuh"
#include "tcgen05.cuh"

namespace b200rl {

namespace {
constexpr int H = 64, TILE = 128;
constexpr uint32_t A_KBLOCK_BYTES = TILE * 128;        // 128 rows x 128 B  (32 tf32 along K)
constexpr uint32_t B_KBLOCK_BYTES = H * 128;           // 64 rows x 128 B
constexpr uint32_t OFF_A_HI = 0, OFF_A_LO = 2 * A_KBLOCK_BYTES, OFF_B_HI = 4 * A_KBLOCK_BYTES, OFF_B_LO = OFF_B_HI + 2 * B_KBLOCK_BYTES;
constexpr uint32_t OFF_L1 = OFF_B_LO + 2 * B_KBLOCK_BYTES;     // float4 {w0, w1, w2, b1} per hidden unit
constexpr uint32_t OFF_L3 = OFF_L1 + H * 16;                   // float2 {b2, w3} per hidden unit
constexpr uint32_t OFF_B3 = OFF_L3 + H * 8;
constexpr uint32_t OFF_MBAR = OFF_B3 + 16;
constexpr uint32_t OFF_SLOT = OFF_MBAR + 8;
constexpr uint32_t SMEM_BYTES = OFF_SLOT + 8 + 1024;           // + slack to align the base to 1024 B
constexpr uint32_t TMEM_COLS = 64;
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;         // ~1 s: far beyond any legitimate wait
}

template <int ACT>
__device__ __forceinline__ float act_or_rt(float x, int rt){
    if constexpr(ACT >= 0) return activation<ACT>(x);
    else return activation_rt(x, rt);
}

template <int A1, int A2>
__global__ void __launch_bounds__(TILE, 2) rollout_tc_kernel(RolloutArgs a, int n_tiles){
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5;
    float4* L1 = reinterpret_cast<float4*>(base + OFF_L1);
    float2* L3 = reinterpret_cast<float2*>(base + OFF_L3);
    float* B3 = reinterpret_cast<float*>(base + OFF_B3);
    uint64_t* mbar = reinterpret_cast<uint64_t*>(base + OFF_MBAR);
    uint32_t* slot = reinterpret_cast<uint32_t*>(base + OFF_SLOT);

    // ---- one-time staging of the actor: arena = W1[64,3] b1[64] W2[64,64] b2[64] W3[1,64] b3[1] ----
    const float* P = a.params;
    if(tid < H){
        L1[tid] = make_float4(__ldg(P + tid * 3), __ldg(P + tid * 3 + 1), __ldg(P + tid * 3 + 2), __ldg(P + 192 + tid));
        L3[tid] = make_float2(__ldg(P + 4352 + tid), __ldg(P + 4416 + tid));
    }
    if(tid == 0) B3[0] = __ldg(P + 4480);
    for(int idx = tid; idx < H * H; idx += TILE){
        const int j = idx >> 6, k = idx & 63;                 // W2[j][k]: row j of the B operand, K index k
        float hi, lo;
        tc::split_tf32(__ldg(P + 256 + idx), hi, lo);
        const uint32_t off = (uint32_t)(k >> 5) * B_KBLOCK_BYTES + (uint32_t)j * 128 + ((((uint32_t)(k & 31) >> 2) ^ ((uint32_t)j & 7)) << 4) + ((uint32_t)k & 3) * 4;
        *reinterpret_cast<float*>(base + OFF_B_HI + off) = hi;
        *reinterpret_cast<float*>(base + OFF_B_LO + off) = lo;
    }
    if(tid == 0){ tc::mbar_init(mbar, 1); tc::fence_mbar_init(); }
    if(warp == 0){ tc::tmem_alloc(slot, TMEM_COLS); tc::tmem_relinquish(); }
    tc::fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = *slot;
    const uint32_t tmem_row = tmem_base + ((uint32_t)(warp * 32) << 16);
    const uint32_t a_hi_addr = tc::smem_u32(base + OFF_A_HI), a_lo_addr = tc::smem_u32(base + OFF_A_LO);
    const uint64_t desc_a_hi = tc::make_desc_kmajor_sw128(a_hi_addr), desc_a_lo = tc::make_desc_kmajor_sw128(a_lo_addr);
    const uint64_t desc_b_hi = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_HI)), desc_b_lo = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_LO));
    constexpr uint32_t IDESC = tc::make_idesc_tf32(TILE, H);
    uint8_t* my_row_hi = base + OFF_A_HI + tid * 128;
    uint8_t* my_row_lo = base + OFF_A_LO + tid * 128;
    const uint32_t swz = (uint32_t)tid & 7;
    const int act1 = a.acts[0], act2 = a.acts[1], act3 = a.acts[2];
    uint32_t phase = 0;
    bool failed = false;

    for(int tile = blockIdx.x; tile < n_tiles && !failed; tile += gridDim.x){
        const int local = tile * TILE + tid;
        const bool valid = local < a.env_count;
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

            // ---- layer 1 on CUDA cores, split, swizzled store: 16-byte chunk c of K-block kb holds h1[kb*32 + 4c .. +3] ----
#pragma unroll
            for(int c16 = 0; c16 < 16; c16++){
                float hi[4], lo[4];
#pragma unroll
                for(int q = 0; q < 4; q++){
                    const float4 w = L1[c16 * 4 + q];
                    float acc = w.w;
                    acc = fmaf(w.x, cs, acc); acc = fmaf(w.y, sn, acc); acc = fmaf(w.z, theta_dot, acc);
                    tc::split_tf32(act_or_rt<A1>(acc, act1), hi[q], lo[q]);
                }
                const uint32_t off = (uint32_t)(c16 >> 3) * A_KBLOCK_BYTES + ((((uint32_t)c16 & 7) ^ swz) << 4);
                *reinterpret_cast<float4*>(my_row_hi + off) = make_float4(hi[0], hi[1], hi[2], hi[3]);
                *reinterpret_cast<float4*>(my_row_lo + off) = make_float4(lo[0], lo[1], lo[2], lo[3]);
            }
            tc::fence_proxy_async_smem();
            tc::fence_before_thread_sync();
            __syncthreads();

            // ---- layer 2 on the tensor core: D[128x64] = A_lo*B_hi + A_hi*B_lo + A_hi*B_hi ----
            if(tid == 0){
                tc::fence_after_thread_sync();
                uint32_t accumulate = 0;
#pragma unroll
                for(int pass = 0; pass < 3; pass++){
                    const uint64_t da = pass == 0 ? desc_a_lo : desc_a_hi;
                    const uint64_t db = pass == 1 ? desc_b_lo : desc_b_hi;
#pragma unroll
                    for(int kb = 0; kb < 2; kb++){
#pragma unroll
                        for(int ks = 0; ks < 4; ks++){
                            tc::mma_tf32_ss(tmem_base, da + (uint64_t)(kb * (A_KBLOCK_BYTES >> 4) + ks * 2), db + (uint64_t)(kb * (B_KBLOCK_BYTES >> 4) + ks * 2), IDESC, accumulate);
                            accumulate = 1;
                        }
                    }
                }
                tc::commit(mbar);
            }
            const bool ok = tc::mbar_wait_bounded(mbar, phase, WAIT_LIMIT_CYCLES);
            phase ^= 1;
            if(__syncthreads_or(!ok)){          // uniform decision: leave the kernel instead of spinning
                failed = true;
                if(tid == 0 && a.error_flag) *a.error_flag = 2;
                break;
            }
            tc::fence_after_thread_sync();

            // ---- epilogue: bias + activation of layer 2, output layer 64 -> 1 ----
            uint32_t r0[32], r1[32];
            tc::tmem_ld_32x32(tmem_row, r0);
            tc::tmem_ld_32x32(tmem_row + 32, r1);
            tc::tmem_wait_ld();
            float out = B3[0];
#pragma unroll
            for(int j = 0; j < 32; j++){
                const float2 bw = L3[j];
                out = fmaf(bw.y, act_or_rt<A2>(__uint_as_float(r0[j]) + bw.x, act2), out);
            }
#pragma unroll
            for(int j = 0; j < 32; j++){
                const float2 bw = L3[32 + j];
                out = fmaf(bw.y, act_or_rt<A2>(__uint_as_float(r1[j]) + bw.x, act2), out);
            }
            const float action = activation_rt(out, act3);

            float nt, ntd;
            pendulum::step(theta, theta_dot, sn, action, nt, ntd);
            const float r = pendulum::reward(theta, theta_dot, action);
            if(valid){ a.act[row] = action; a.rew[row] = r; }
            es += 1; er = __fadd_rn(er, r);
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
    const int n_tiles = (a.env_count + TILE - 1) / TILE;
    const int grid = n_tiles < 2 * NUM_SMS ? n_tiles : 2 * NUM_SMS;      // persistent: two CTAs per SM
    rollout_tc_kernel<A1, A2><<<grid, TILE, SMEM_BYTES, s>>>(a, n_tiles);
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
