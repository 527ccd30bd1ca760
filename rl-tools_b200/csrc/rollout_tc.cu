// Tensor-core rollout for the OBS -> 64 -> 64 -> 1 actor (sm_100a, tcgen05 + TMEM). The environment is a compile-time policy (envs.cuh):
// the Pendulum (the headline workload; also the on-policy collect and the device-side random numbers) and the two Acrobot variants
// (trajectories from reset tables, with the terminated flag of every transition on request).
//
// One persistent CTA per SM, 512 threads = 4 independent groups of 128 threads. A group owns a tile of up to 128
// environments for all T steps; thread r of the group owns environment r of the tile, which is row r of the MMA and
// lane r of tensor memory. The environments of a launch are spread evenly over all 4 x (#CTAs) groups (tiles of
// <= 128 environments, a multiple of 4), so every SM carries the same load and there is a single wave.
//
// The second layer (the one dense contraction of the path) runs on the tensor core with fp32 accuracy through a split
// into fp16 parts: x = lead + rest with lead = fp16(x) (11 significant bits) and rest = fp16(x - lead), so lead + rest
// carries ~22 bits, and
//     h1 . W2  ~=  rest_h * lead_W  +  lead_h * rest_W  +  lead_h * lead_W          (fp32 accumulate, dropped term ~2^-24)
// Every part has K = 64 in ONE 128-byte row, an instruction covers K = 16, so a tile and step take 3 passes x 4
// tcgen05.mma (M128 N64 K16, kind::f16) plus one K step that adds the two parts of the bias through a constant "ones"
// tile: 13 MMAs. (The same accuracy through tf32 parts takes 25 MMAs of K = 8, and the 25 form ONE chain of dependent
// accumulations at ~110 cycles each, which sat on every group's critical path: 0.70 -> 0.62 ms per 65,536 x 200 rollout.)
// W2 and b2 are multiplied by a power of two that brings their largest magnitude into [2^13, 2^14), which keeps the
// remainder parts out of fp16's subnormal range; the accumulator is scaled back exactly in the epilogue. Layer-1
// activations are converted with saturation: hidden activations beyond +-65504 are outside this kernel's domain.
// Per step and group:
//   1. thread: reset-if-truncated, observation; first layer (K = OBS) on CUDA cores, weights as constant-bank FMA operands;
//      the leading parts of h1 go to tensor memory (two K elements per 32-bit column: 32 columns), the remainder parts into a
//      K-major, 128-byte-swizzled shared-memory tile
//   2. the group's leader issues the 13 MMAs and tcgen05.commit -> the group's mbarrier
//   3. every thread waits (bounded), reads its accumulator row from TMEM (tcgen05.ld), applies the activation and
//      the 64 -> 1 output layer, then steps the environment in registers.
// The groups work as two pairs {0,1} and {2,3} that take turns ISSUING to the tensor core: a pair's two MMA batches run together
// (one batch alone is bound by the latency of its chain of dependent MMAs) while the other pair is in its CUDA-core
// phases; the turn passes as soon as a pair has issued. (Measured against it: passing the turn only when the batches have
// completed, 0.900 against 0.864 ms; no turns at all, 0.73 against 0.63 ms.) The second-layer weights (both fp16 parts, the B
// operand) stay resident in shared memory for the whole launch and are shared by the four groups.
// Tensor memory: 4 groups x (64 accumulator + 32 operand columns) of the 512 allocated.
#include "common.cuh"
#include "envs.cuh"
#include "rollout.cuh"
#include "tcgen05.cuh"
#include <mutex>
#include <cuda_fp16.h>
#include <type_traits>


namespace b200rl {

namespace {
constexpr int H = 64, TILE = 128, GROUPS = 4, THREADS = GROUPS * TILE;
constexpr uint32_t A_PART_BYTES = TILE * 128;          // 128 rows x 128 B: the whole K = 64 as fp16
constexpr uint32_t B_PART_BYTES = H * 128;             // 64 rows x 128 B
constexpr uint32_t OFF_B_LEAD = 0, OFF_B_REST = B_PART_BYTES, OFF_A_REST = 2 * B_PART_BYTES;      // leading fp16 parts / fp16 parts of the remainders
constexpr uint32_t OFF_ONES = OFF_A_REST + GROUPS * A_PART_BYTES;  // [128 x 16] K=16 tile, columns 0 and 1 == 1: feeds the bias row through the MMA
constexpr uint32_t OFF_BIAS = OFF_ONES + 4096;                // [64 x 16] K=16 tile, column 0 == leading part of b2 (scaled), column 1 == its remainder part
constexpr uint32_t OFF_MBAR = OFF_BIAS + 2048;
constexpr uint32_t OFF_ABORT = OFF_MBAR + 8 * GROUPS;
constexpr uint32_t OFF_SLOT = OFF_ABORT + 4 * GROUPS;
constexpr uint32_t OFF_SCALE = OFF_SLOT + 8;                  // [0] scale of the second-layer operand (a power of two), [1] its inverse; [2..3] reduction scratch
constexpr uint32_t OFF_TURN = OFF_SCALE + 16 + 4 * 32;                   // 2 mbarriers: the tensor token alternating between the group pairs {0,1} and {2,3}
constexpr uint32_t OFF_STAGE = (OFF_TURN + 8 * 2 + 15) / 16 * 16;  // output staging for bulk stores: per group 3 buffers x (obs + act + rew rows of a tile)
__host__ __device__ constexpr uint32_t stage_buf_bytes(int obs_dim){ return TILE * 4 * obs_dim + TILE * 4 + TILE * 4; }
__host__ __device__ constexpr uint32_t smem_bytes(int obs_dim){ return OFF_STAGE + GROUPS * 3 * stage_buf_bytes(obs_dim) + 1024; }     // + slack to align the base to 1024 B
constexpr uint32_t TMEM_COLS = 512, TMEM_COLS_PER_GROUP = 128;          // per group 64 accumulator + 32 operand columns are used
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;        // ~1 s: far beyond any legitimate wait
constexpr int MAX_OBS = 6;
// offsets in the arena of the actor OBS -> 64 -> 64 -> 1, and in the constant bank (the same without W2)
struct Layout {
    int P_B1, P_W2, P_B2, P_W3, P_B3, C_B1, C_B2, C_W3, C_B3;
    __host__ __device__ constexpr Layout(int obs): P_B1(H * obs), P_W2(H * obs + H), P_B2(H * obs + H + H * H), P_W3(H * obs + 2 * H + H * H), P_B3(H * obs + 3 * H + H * H),
                               C_B1(H * obs), C_B2(H * obs + H), C_W3(H * obs + 2 * H), C_B3(H * obs + 3 * H) {}
};
constexpr int C_COUNT_MAX = H * MAX_OBS + 3 * H + 1;
}

// The small layers' weights (W1, b1, b2, W3, b3) are read by EVERY thread at EVERY step. As constant-bank operands
// of the FMA instructions they cost no load instruction and no shared-memory bandwidth (a warp-wide broadcast LDS.128
// occupies the 128 B/clk shared pipe for 4 cycles, which made the table look-ups the bottleneck of the CUDA-core
// phase). Filled by a device-to-device copy on the launch stream; launches are ordered by an event (see launch_tc).
__constant__ __align__(16) float c_actor[C_COUNT_MAX + 3];
// The first layer's weights once more, as pairs of neighbouring units: c_w1_pairs[(j / 2) * OBS + k] = (W1[j][k], W1[j + 1][k]), j even, so
// that two units advance with one packed multiply-add (the issue slots, not the arithmetic pipes, bound this kernel). Written by
// pack_w1_pairs_kernel on the launch stream.
__constant__ __align__(16) float2 c_w1_pairs[(H / 2) * MAX_OBS];
__global__ void pack_w1_pairs_kernel(const float* __restrict__ params, int obs_dim, float2* __restrict__ dst){
    for(int i = threadIdx.x; i < (H / 2) * obs_dim; i += blockDim.x){
        const int pair = i / obs_dim, k = i % obs_dim;
        dst[i] = make_float2(params[(2 * pair) * obs_dim + k], params[(2 * pair + 1) * obs_dim + k]);
    }
}

// x = lead + rest + O(2^-24 x): lead = fp16(x) (11 significant bits), rest = fp16(x - lead). Two values per register, the lower index in
// the low half. Conversions saturate at +-65504 instead of producing infinities.
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi){
    uint32_t r;
    asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}
__device__ __forceinline__ void split_f16_pair(float a, float b, uint32_t& lead, uint32_t& rest){
    lead = pack_f16x2_sat(a, b);
    const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&lead));
    const float2 d = __ffma2_rn(back, make_float2(-1.0f, -1.0f), make_float2(a, b));
    rest = pack_f16x2_sat(d.x, d.y);
}

// The same split of relu(a), relu(b) with the ReLU folded into the conversions (no separate maximum per unit): the leading part is
// converted with round-toward-zero and the conversion's own ReLU, so for x >= 0 the remainder x - lead is >= 0 and the second conversion's
// ReLU leaves it alone, while for x < 0 the leading part is 0, the remainder is x itself and the second ReLU zeroes it. Truncation makes the
// remainder up to twice as large as with round-to-nearest: lead + rest carries ~21 bits instead of ~22 (relative 2^-21 = 4.8e-7 worst case).
__device__ __forceinline__ void split_f16_pair_relu(float a, float b, uint32_t& lead, uint32_t& rest){
    asm("cvt.rz.relu.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(lead) : "f"(b), "f"(a));
    const float2 back = __half22float2(*reinterpret_cast<const __half2*>(&lead));
    const float2 d = __ffma2_rn(back, make_float2(-1.0f, -1.0f), make_float2(a, b));
    asm("cvt.rn.relu.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(rest) : "f"(d.y), "f"(d.x));
}

template <int ACT>
__device__ __forceinline__ float act_or_rt(float x, int rt){
    if constexpr(ACT >= 0) return activation<ACT>(x);
    else return activation_rt(x, rt);
}

// BULK: the trajectory rows of a tile and step are contiguous in HBM (obs 12 B, act 4 B, rew 4 B per environment), so the threads write them to
// a shared-memory staging buffer and the group's leader hands each buffer to the copy engine (cp.async.bulk shared -> global, one destination)
// one step later, at the barrier it already has before its MMA batch. Three buffers rotate: the buffer of step t is read by the copy issued
// after barrier t+1, the leader waits for that read before barrier t+2, and the buffer is written again in step t+3. Requires 16-byte aligned
// row starts (n_envs and the slab origin multiples of 4, aligned output pointers); the host selects the plain-store instantiation otherwise.
template <typename ENV, int A1, int A2, bool COLLECT, bool BULK>
__global__ void __launch_bounds__(THREADS, 1) rollout_tc_kernel(RolloutArgs a, int n_tiles, int envs_per_tile){
    static_assert(!(COLLECT && BULK), "dataset rows are strided: plain stores");
    constexpr bool IS_PENDULUM = std::is_same<ENV, PendulumEnv>::value;
    static_assert(!COLLECT || IS_PENDULUM, "the dataset columns are the Pendulum's");
    constexpr int S = ENV::STATE_DIM, O = ENV::OBS_DIM, RD = ENV::RESET_DIM;
    static_assert(O <= MAX_OBS, "constant bank");
    constexpr Layout L(O);
    constexpr int P_W2 = L.P_W2, P_B2 = L.P_B2, C_W1 = 0, C_B1 = L.C_B1, C_W3 = L.C_W3, C_B3 = L.C_B3;
    constexpr uint32_t STAGE_BUF_BYTES = stage_buf_bytes(O), STAGE_GROUP_BYTES = 3 * STAGE_BUF_BYTES;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment by OFFSET from the __shared__ array, so the compiler keeps the shared address space (LDS/STS, not generic)
    uint8_t* base = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, g = tid >> 7, r = tid & 127, warp = tid >> 5;
    uint64_t* mbar = reinterpret_cast<uint64_t*>(base + OFF_MBAR) + g;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base + OFF_ABORT) + g;
    uint32_t* slot = reinterpret_cast<uint32_t*>(base + OFF_SLOT);
    uint64_t* turn = reinterpret_cast<uint64_t*>(base + OFF_TURN);

    // ---- one-time staging of the second layer (B operand); arena = W1[64,3] b1[64] W2[64,64] b2[64] W3[1,64] b3[1] ----
    // W2 and b2 are multiplied by a power of two that brings the largest magnitude into [2^13, 2^14): the remainder parts then stay clear
    // of fp16's subnormal range; the accumulator is scaled back (exactly) in the epilogue.
    const float* P = a.params;
    float* scale_slot = reinterpret_cast<float*>(base + OFF_SCALE);
    {
        float m = 0.0f;
        for(int idx = tid; idx < H * H + H; idx += THREADS) m = fmaxf(m, fabsf(__ldg(P + P_W2 + idx)));       // W2 and b2 are adjacent in the arena
#pragma unroll
        for(int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        if((tid & 31) == 0) scale_slot[4 + warp] = m;
        __syncthreads();
        if(tid == 0){
            float mm = 0.0f;
            for(int w = 0; w < THREADS / 32; w++) mm = fmaxf(mm, scale_slot[4 + w]);
            // exponent of the largest magnitude -> scale = 2^(13 - exponent); degenerate inputs (all zero, inf, nan) take scale 1
            const int ex = (int)((__float_as_uint(mm) >> 23) & 0xFF) - 127;
            const bool ok = mm > 0.0f && ex > -100 && ex < 100;
            scale_slot[0] = ok ? __uint_as_float((uint32_t)(127 + 13 - ex) << 23) : 1.0f;
            scale_slot[1] = ok ? __uint_as_float((uint32_t)(127 - 13 + ex) << 23) : 1.0f;
        }
        __syncthreads();
    }
    const float w_scale = scale_slot[0], w_unscale = scale_slot[1];
    for(int idx = tid; idx < H * H / 2; idx += THREADS){
        const int j = idx >> 5, k = (idx & 31) * 2;           // W2[j][k], W2[j][k+1]: row j of the B operand, K index k
        uint32_t lead, rest;
        split_f16_pair(__ldg(P + P_W2 + j * H + k) * w_scale, __ldg(P + P_W2 + j * H + k + 1) * w_scale, lead, rest);
        const uint32_t off = (uint32_t)j * 128 + ((((uint32_t)k >> 3) ^ ((uint32_t)j & 7)) << 4) + ((uint32_t)k & 7) * 2;
        *reinterpret_cast<uint32_t*>(base + OFF_B_LEAD + off) = lead;
        *reinterpret_cast<uint32_t*>(base + OFF_B_REST + off) = rest;
    }
    // bias of layer 2 as one extra K step: D += ones[128 x 16] * bias[64 x 16]^T with columns 0 and 1 populated (leading and remainder part)
    for(int idx = tid; idx < TILE * 16; idx += THREADS)
        *reinterpret_cast<__half*>(base + OFF_ONES + tc::noswizzle_k16_offset(idx >> 4, idx & 15)) = __float2half((idx & 15) < 2 ? 1.0f : 0.0f);
    for(int idx = tid; idx < H * 16; idx += THREADS){
        const int j = idx >> 4, k = idx & 15;
        uint32_t lead, rest;
        split_f16_pair(__ldg(P + P_B2 + j) * w_scale, 0.0f, lead, rest);
        const uint16_t v = k == 0 ? (uint16_t)(lead & 0xFFFF) : (k == 1 ? (uint16_t)(rest & 0xFFFF) : (uint16_t)0);
        *reinterpret_cast<uint16_t*>(base + OFF_BIAS + tc::noswizzle_k16_offset(j, k)) = v;
    }
    if(r == 0){ tc::mbar_init(mbar, 1); *abort_flag = 0; }
    if(tid < 2) tc::mbar_init(turn + tid, 2);                 // each completes when BOTH leaders of the other pair have issued
    if(tid == 0) tc::fence_mbar_init();
    if(warp == 0){ tc::tmem_alloc(slot, TMEM_COLS); tc::tmem_relinquish(); }
    tc::fence_proxy_async_smem();
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    if(tid == 0){ tc::mbar_arrive(turn); tc::mbar_arrive(turn); }          // pair {0,1} holds the token first
    const uint32_t tmem_base = *slot;
    const uint32_t tmem_d = tmem_base + (uint32_t)g * TMEM_COLS_PER_GROUP;          // accumulator: 64 columns
    const uint32_t tmem_a = tmem_d + 64;                                            // leading fp16 part of A, two K elements per column: 32 columns
    const uint32_t lane_off = (uint32_t)((warp & 3) * 32) << 16;                    // this warp's lane quarter
    uint8_t* a_rest = base + OFF_A_REST + (uint32_t)g * A_PART_BYTES;
    const uint64_t desc_a_rest = tc::make_desc_kmajor_sw128(tc::smem_u32(a_rest));
    const uint64_t desc_b_lead = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_LEAD)), desc_b_rest = tc::make_desc_kmajor_sw128(tc::smem_u32(base + OFF_B_REST));
    const uint64_t desc_ones = tc::make_desc_kmajor_noswizzle_k8(tc::smem_u32(base + OFF_ONES));
    const uint64_t desc_bias = tc::make_desc_kmajor_noswizzle_k8(tc::smem_u32(base + OFF_BIAS));
    constexpr uint32_t IDESC = tc::make_idesc_f16(TILE, H);
    uint8_t* my_row_rest = a_rest + r * 128;              // this thread's row of the remainder-part tile
    const uint32_t swz = (uint32_t)r & 7;
    const int act1 = a.acts[0], act2 = a.acts[1], act3 = a.acts[2];
    const uint32_t bar_id = 1 + g;
    uint32_t phase = 0, turn_phase = 0;
    bool failed = false;
    uint64_t* my_turn = turn + (g >> 1);
    uint64_t* next_turn = turn + ((g >> 1) ^ 1);
    GaussianHead head{};
    const size_t ld = COLLECT ? (size_t)a.ld_dataset : 0;
    if constexpr(COLLECT) head.init(a.log_std);
    uint8_t* stage_base = base + OFF_STAGE + (uint32_t)g * STAGE_GROUP_BYTES;

    const int rounds = (n_tiles + (int)gridDim.x * GROUPS - 1) / ((int)gridDim.x * GROUPS);
    for(int round = 0; round < rounds && !failed; round++){
        const int tile = (round * (int)gridDim.x + (int)blockIdx.x) * GROUPS + g;
        if(tile >= n_tiles){
            // no environments for this group in this round: it still hands the tensor token on, once per step
            if(r == 0){
                for(int t = 0; t < a.n_steps; t++){
                    if(!tc::mbar_wait_bounded(my_turn, turn_phase, WAIT_LIMIT_CYCLES)){ failed = true; break; }
                    turn_phase ^= 1;
                    tc::mbar_arrive(next_turn);
                }
            }
            continue;
        }
        const int local = tile * envs_per_tile + r;
        const bool valid = r < envs_per_tile && local < a.env_count;
        const int e = a.env_begin + (valid ? local : 0);
        float state[S], er = 0.0f; int es = 0, resets = 0; bool trunc = false;
#pragma unroll
        for(int k = 0; k < S; k++) state[k] = 0.0f;
        if(valid){
#pragma unroll
            for(int k = 0; k < S; k++) state[k] = a.states[(size_t)S * e + k];
            es = a.episode_step[e]; trunc = a.truncated[e] != 0; er = a.episode_return[e];
            resets = a.reset_count ? a.reset_count[e] : 0;
            if constexpr(COLLECT) a.dataset[(size_t)e * ld + COL_RESET] = trunc ? 1.0f : 0.0f;      // collect, operations_generic.h:115-117
        }
        const int tile_first = a.env_begin + tile * envs_per_tile;
        const int tile_count = min(envs_per_tile, a.env_count - tile * envs_per_tile);
        // leader only: hands the staged rows of step `ts` to the copy engine
        auto bulk_flush = [&](int ts){
            uint8_t* buf = stage_base + (uint32_t)(ts % 3) * STAGE_BUF_BYTES;
            const size_t row0 = (size_t)ts * a.n_envs + tile_first;
            tc::bulk_store(a.obs + row0 * O, buf, (uint32_t)tile_count * 4 * O);
            tc::bulk_store(a.act + row0, buf + TILE * 4 * O, (uint32_t)tile_count * 4);
            tc::bulk_store(a.rew + row0, buf + TILE * 4 * (O + 1), (uint32_t)tile_count * 4);
            tc::bulk_commit();
        };
        for(int t = 0; t < a.n_steps; t++){
            float* st_obs = reinterpret_cast<float*>(stage_base + (uint32_t)(t % 3) * STAGE_BUF_BYTES);
            float* st_act = st_obs + TILE * O;
            float* st_rew = st_act + TILE;
            StepDraws draws{};             // the trajectory-only kernels need the draws at a reset only: nothing per step on their hot path
            if constexpr(IS_PENDULUM){ if(a.device_rng && (COLLECT || trunc)) draws = step_draws(a.rng_seed, a.rng_step0 + (unsigned long long)t, (uint32_t)e); }
            if(trunc && valid){
                bool drawn = false;
                if constexpr(IS_PENDULUM){
                    if(a.device_rng){    // theta ~ U(-pi, pi), theta_dot ~ U(-1, 1) (rl/environments/pendulum/operations_generic.h:57-61)
                        state[0] = fmaf(draws.u_theta, 2.0f * pendulum::PI_F, -pendulum::PI_F); state[1] = fmaf(draws.u_theta_dot, 2.0f, -1.0f);
                        drawn = true;
                    }
                }
                if(!drawn){
                    if(a.reset_states != nullptr && resets < a.n_reset_rounds){
                        const float* rs = a.reset_states + ((size_t)resets * a.n_envs + e) * RD;      // scalar loads: the table may be a view at any 4-byte offset
                        float u[RD];
#pragma unroll
                        for(int k = 0; k < RD; k++) u[k] = __ldg(rs + k);
                        ENV::reset(state, u);
                    }
                    else if(a.error_flag) *a.error_flag = 1;
                }
                resets++; es = 0; er = 0.0f;
            }
            float o[O];
            ENV::observe(state, o);
            const size_t row = (size_t)t * a.n_envs + e;
            float* drow = COLLECT ? a.dataset + row * ld : nullptr;
            if(valid){
#pragma unroll
                for(int k = 0; k < O; k++){
                    if constexpr(COLLECT) drow[COL_OBS + k] = o[k];
                    else if constexpr(BULK) st_obs[r * O + k] = o[k];
                    else a.obs[row * O + k] = o[k];
                }
            }

            // ---- layer 1 (CUDA cores, weights as constant-bank operands); leading fp16 parts -> TMEM, remainder parts -> swizzled smem tile ----
            uint32_t lead_all[32];
            float2 o2[O];
#pragma unroll
            for(int k = 0; k < O; k++) o2[k] = make_float2(o[k], o[k]);
#pragma unroll
            for(int c = 0; c < 8; c++){                  // 16-byte chunk c of the row: units 8c .. 8c+7
                uint32_t rest[4];
#pragma unroll
                for(int q = 0; q < 4; q++){
                    float h[2];
                    {
                        const int pair = c * 4 + q;                                          // units 2 pair, 2 pair + 1
                        float2 acc = *reinterpret_cast<const float2*>(&c_actor[C_B1 + 2 * pair]);            // bias first, inputs ascending: the reference's order
#pragma unroll
                        for(int k = 0; k < O; k++) acc = __ffma2_rn(c_w1_pairs[pair * O + k], o2[k], acc);
                        if constexpr(A1 == B200RL_ACT_RELU){ h[0] = acc.x; h[1] = acc.y; }       // the ReLU rides on the conversions below
                        else { h[0] = act_or_rt<A1>(acc.x, act1); h[1] = act_or_rt<A1>(acc.y, act1); }
                    }
                    if constexpr(A1 == B200RL_ACT_RELU) split_f16_pair_relu(h[0], h[1], lead_all[c * 4 + q], rest[q]);
                    else split_f16_pair(h[0], h[1], lead_all[c * 4 + q], rest[q]);
                }
                *reinterpret_cast<uint4*>(my_row_rest + (((uint32_t)c ^ swz) << 4)) = make_uint4(rest[0], rest[1], rest[2], rest[3]);
            }
            tc::tmem_st_32x32(tmem_a + lane_off, lead_all);
            tc::tmem_wait_st();
            tc::fence_proxy_async_smem();
            tc::fence_before_thread_sync();
            if constexpr(BULK){ if(r == 0) tc::bulk_wait_read<0>(); }      // the copy of step t-2 has read its buffer (re-used from step t+1 on)
            tc::named_barrier_sync(bar_id, TILE);
            if(*abort_flag){ failed = true; break; }

            // ---- layer 2 on the tensor core. The issuing turn alternates between the group pairs {0,1} and {2,3}: one pair's MMA batches
            // run while the other pair is in its CUDA-core phases; two batches in flight hide the accumulator dependency between MMAs ----
            if(r == 0){
                if(!tc::mbar_wait_bounded(my_turn, turn_phase, WAIT_LIMIT_CYCLES)){ *abort_flag = 1; if(a.error_flag) *a.error_flag = 2; }
                turn_phase ^= 1;
                tc::fence_after_thread_sync();
                // remainder * leading (A from shared memory), leading * remainder and leading * leading (A from tensor memory, 8 columns
                // per K = 16 step): the small terms first; then the bias step
#pragma unroll
                for(int ks = 0; ks < 4; ks++) tc::mma_f16_ss(tmem_d, desc_a_rest + (uint64_t)(ks * 2), desc_b_lead + (uint64_t)(ks * 2), IDESC, ks ? 1u : 0u);
#pragma unroll
                for(int pass = 0; pass < 2; pass++){
                    const uint64_t db = pass == 0 ? desc_b_rest : desc_b_lead;
#pragma unroll
                    for(int ks = 0; ks < 4; ks++) tc::mma_f16_ts(tmem_d, tmem_a + (uint32_t)(ks * 8), db + (uint64_t)(ks * 2), IDESC, 1u);
                }
                tc::mma_f16_ss(tmem_d, desc_ones, desc_bias, IDESC, 1u);
                tc::commit(mbar);
                tc::mbar_arrive(next_turn);
                if constexpr(BULK){ if(t > 0) bulk_flush(t - 1); }          // every thread of the group finished step t-1 before this step's barrier
            }
            __syncwarp();                                     // the leader's lanes rejoin before the warp-wide TMEM loads
            if(!tc::mbar_wait_bounded(mbar, phase, WAIT_LIMIT_CYCLES)){
                *abort_flag = 1;                              // seen by the whole group after its next barrier
                if(a.error_flag) *a.error_flag = 2;
            }
            phase ^= 1;
            tc::fence_after_thread_sync();

            // ---- epilogue: activation of layer 2 (bias came through the MMA), output layer 64 -> 1 (four partial sums) ----
            float2 oa = make_float2(0.0f, 0.0f), ob = make_float2(0.0f, 0.0f);      // partial sums of units j = 0, 1 (mod 4) and j = 2, 3 (mod 4)
#pragma unroll
            for(int half = 0; half < 2; half++){
                uint32_t d[32];
                tc::tmem_ld_32x32(tmem_d + lane_off + half * 32, d);
                tc::tmem_wait_ld();
#pragma unroll
                for(int p = 0; p < 8; p++){
                    const int j = half * 32 + p * 4;
                    // ReLU commutes with the positive scale: it is taken out once after the sum; other activations scale each unit back first
                    constexpr bool HOMOGENEOUS = A2 == B200RL_ACT_RELU || A2 == B200RL_ACT_IDENTITY;
                    const float back = HOMOGENEOUS ? 1.0f : w_unscale;
                    const float2 ha = make_float2(act_or_rt<A2>(__uint_as_float(d[p * 4 + 0]) * back, act2), act_or_rt<A2>(__uint_as_float(d[p * 4 + 1]) * back, act2));
                    const float2 hb = make_float2(act_or_rt<A2>(__uint_as_float(d[p * 4 + 2]) * back, act2), act_or_rt<A2>(__uint_as_float(d[p * 4 + 3]) * back, act2));
                    oa = __ffma2_rn(*reinterpret_cast<const float2*>(&c_actor[C_W3 + j]), ha, oa);
                    ob = __ffma2_rn(*reinterpret_cast<const float2*>(&c_actor[C_W3 + j + 2]), hb, ob);
                }
            }
            const float osum = (oa.x + oa.y) + (ob.x + ob.y);
            float action = activation_rt(c_actor[C_B3] + ((A2 == B200RL_ACT_RELU || A2 == B200RL_ACT_IDENTITY) ? osum * w_unscale : osum), act3);
            if constexpr(COLLECT){
                const float mean = action;
                action = head.sample(mean, a.device_rng ? draws.normal : (valid ? __ldg(a.noise + row) : 0.0f));
                if(valid){ drow[COL_ACTION_MEAN] = mean; drow[COL_ACTION] = action; drow[COL_LOG_PROB] = head.log_prob(mean, action, a.neg_half_log_2pi); }
            }

            float next[S];
            const float rwd = ENV::transition_obs(state, o, action, next);
            es += 1; er = __fadd_rn(er, rwd);
            if constexpr(COLLECT){
                trunc = a.step_limit > 0 && es >= a.step_limit;             // operations_generic_per_env.h:72
                if(valid){
                    const float flag = trunc ? 1.0f : 0.0f;
                    drow[COL_REWARD] = rwd; drow[COL_TERMINATED] = 0.0f; drow[COL_TRUNCATED] = flag;
                    drow[(size_t)a.n_envs * ld + COL_RESET] = flag;         // all_reset[pos + N]
                }
            }
            else{
                if(valid){
                    if constexpr(BULK){ st_act[r] = action; st_rew[r] = rwd; }
                    else{ a.act[row] = action; a.rew[row] = rwd; }
                }
                bool term = false;
                if constexpr(ENV::TERMINATES){
                    term = ENV::terminated(next);
                    if(valid && a.terminated) a.terminated[row] = term ? 1 : 0;
                }
                else if(a.terminated){ if(valid) a.terminated[row] = 0; }
                trunc = term || (es == a.step_limit);                         // operations_generic_per_env.h:93-97
            }
#pragma unroll
            for(int k = 0; k < S; k++) state[k] = next[k];
        }
        if constexpr(BULK){
            // last step of the tile: make the staged rows visible to the copy engine, flush, and wait until every buffer has been read
            tc::fence_proxy_async_smem();
            tc::named_barrier_sync(bar_id, TILE);
            if(r == 0 && !failed && a.n_steps > 0){ bulk_flush(a.n_steps - 1); tc::bulk_wait_read<0>(); }
            tc::named_barrier_sync(bar_id, TILE);
        }
        if constexpr(COLLECT){
            if(valid && !failed){                  // final observation, operations_generic.h:136-143
                float o[O];
                ENV::observe(state, o);
                float* drow = a.dataset + ((size_t)a.n_steps * a.n_envs + e) * ld;
#pragma unroll
                for(int k = 0; k < O; k++) drow[COL_OBS + k] = o[k];
            }
        }
        if(valid && !failed){
#pragma unroll
            for(int k = 0; k < S; k++) a.states[(size_t)S * e + k] = state[k];
            a.episode_step[e] = es; a.truncated[e] = trunc ? 1 : 0; a.episode_return[e] = er;
            if(a.reset_count) a.reset_count[e] = resets;
        }
    }
    if(failed) tc::mbar_wait_bounded(mbar, phase ^ 1, WAIT_LIMIT_CYCLES);   // give in-flight MMAs a bounded chance to drain
    tc::fence_before_thread_sync();
    __syncthreads();
    if(warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

// All launches on a device share the constant bank holding the small layers, so each launch (copies + kernel) is ordered after the
// previous one on that device with an event: a launch on another stream waits for the kernel that still reads the old constants.
// The kernel fills every SM, so this ordering costs no concurrency. The event, like the kernel's shared-memory attribute, belongs
// to a device: both are kept per device ordinal.
namespace {
struct TcDeviceState { cudaEvent_t order = nullptr; bool configured[3][16] = {}; float2* w1_pairs = nullptr; };
TcDeviceState g_tc_state[MAX_DEVICES];
std::mutex g_tc_mutex;
}

static int upload_small_layers(TcDeviceState& st, const float* params, int obs_dim, cudaStream_t s, cudaEvent_t* order_event){
    const Layout L(obs_dim);
    if(!st.order) B200RL_CUDA_TRY(cudaEventCreateWithFlags(&st.order, cudaEventDisableTiming));
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    B200RL_CUDA_TRY(cudaStreamIsCapturing(s, &cap));
    *order_event = cap == cudaStreamCaptureStatusNone ? st.order : nullptr;
    if(*order_event) B200RL_CUDA_TRY(cudaStreamWaitEvent(s, st.order, 0));
    B200RL_CUDA_TRY(cudaMemcpyToSymbolAsync(c_actor, params, sizeof(float) * (size_t)L.P_W2, 0, cudaMemcpyDeviceToDevice, s));                           // W1, b1
    B200RL_CUDA_TRY(cudaMemcpyToSymbolAsync(c_actor, params + L.P_B2, sizeof(float) * (2 * H + 1), sizeof(float) * (size_t)L.C_B2, cudaMemcpyDeviceToDevice, s));   // b2, W3, b3
    if(!st.w1_pairs){                                            // the symbol's address on this device
        void* p = nullptr;
        B200RL_CUDA_TRY(cudaGetSymbolAddress(&p, c_w1_pairs));
        st.w1_pairs = static_cast<float2*>(p);
    }
    pack_w1_pairs_kernel<<<1, 128, 0, s>>>(params, obs_dim, st.w1_pairs);
    B200RL_LAUNCH_CHECK("pack_w1_pairs");
    return B200RL_OK;
}

template <typename ENV> struct EnvIndex { static constexpr int value = std::is_same<ENV, PendulumEnv>::value ? 0 : std::is_same<ENV, AcrobotSwingupEnv>::value ? 1 : 2; };

template <typename ENV, int A1, int A2, bool COLLECT, bool BULK>
static int launch_tc_variant(const RolloutArgs& a, cudaStream_t s, int variant){
    constexpr uint32_t SMEM_BYTES = smem_bytes(ENV::OBS_DIM);
    int dev = 0, sms = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    rc = sm_count(&sms);
    if(rc) return rc;
    std::lock_guard<std::mutex> lock(g_tc_mutex);
    TcDeviceState& st = g_tc_state[dev];
    if(!st.configured[EnvIndex<ENV>::value][variant]){
        B200RL_CUDA_TRY(cudaFuncSetAttribute(rollout_tc_kernel<ENV, A1, A2, COLLECT, BULK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        st.configured[EnvIndex<ENV>::value][variant] = true;
    }
    cudaEvent_t order_event = nullptr;
    rc = upload_small_layers(st, a.params, ENV::OBS_DIM, s, &order_event);
    if(rc) return rc;
    // spread the environments evenly over every group of every SM: tiles of <= 128 environments (a multiple of 4)
    const int groups_total = sms * GROUPS;
    int ept = ((a.env_count + groups_total - 1) / groups_total + 3) / 4 * 4;
    if(ept < 32) ept = 32;
    if(ept > TILE) ept = TILE;
    const int n_tiles = (a.env_count + ept - 1) / ept;
    int grid = (n_tiles + GROUPS - 1) / GROUPS;
    if(grid > sms) grid = sms;
    rollout_tc_kernel<ENV, A1, A2, COLLECT, BULK><<<grid, THREADS, SMEM_BYTES, s>>>(a, n_tiles, ept);
    B200RL_LAUNCH_CHECK("rollout_tc");
    if(order_event) B200RL_CUDA_TRY(cudaEventRecord(order_event, s));
    return B200RL_OK;
}

// Bulk stores need 16-byte aligned row starts in all three outputs; per-thread stores otherwise (and always for the strided dataset rows)
template <typename ENV, int A1, int A2, bool COLLECT>
static int launch_tc(const RolloutArgs& a, cudaStream_t s, int variant){
    if constexpr(COLLECT) return launch_tc_variant<ENV, A1, A2, true, false>(a, s, variant);
    else{
        const bool aligned = ((reinterpret_cast<uintptr_t>(a.obs) | reinterpret_cast<uintptr_t>(a.act) | reinterpret_cast<uintptr_t>(a.rew)) & 15u) == 0 &&
                             a.n_envs % 4 == 0 && a.env_begin % 4 == 0 && a.env_count % 4 == 0;
        return aligned ? launch_tc_variant<ENV, A1, A2, false, true>(a, s, variant) : launch_tc_variant<ENV, A1, A2, false, false>(a, s, variant + 1);
    }
}

int launch_rollout_tc(const RolloutArgs& a, cudaStream_t s){
    const int a1 = a.acts[0], a2 = a.acts[1];
    if(a.dataset){
        if(a1 == B200RL_ACT_RELU && a2 == B200RL_ACT_RELU) return launch_tc<PendulumEnv, B200RL_ACT_RELU, B200RL_ACT_RELU, true>(a, s, 0);
        return launch_tc<PendulumEnv, -1, -1, true>(a, s, 1);
    }
    if(a1 == B200RL_ACT_RELU && a2 == B200RL_ACT_RELU) return launch_tc<PendulumEnv, B200RL_ACT_RELU, B200RL_ACT_RELU, false>(a, s, 2);
    if(a1 == B200RL_ACT_TANH && a2 == B200RL_ACT_TANH) return launch_tc<PendulumEnv, B200RL_ACT_TANH, B200RL_ACT_TANH, false>(a, s, 4);
    return launch_tc<PendulumEnv, -1, -1, false>(a, s, 6);
}

// the other environments: trajectories only (no dataset rows, reset tables only), ReLU specialisation or run-time activations
template <typename ENV>
static int launch_env_tc(const RolloutArgs& a, cudaStream_t s){
    if(a.dataset || a.device_rng) return B200RL_ERR_UNSUPPORTED;
    if(a.acts[0] == B200RL_ACT_RELU && a.acts[1] == B200RL_ACT_RELU) return launch_tc<ENV, B200RL_ACT_RELU, B200RL_ACT_RELU, false>(a, s, 2);
    return launch_tc<ENV, -1, -1, false>(a, s, 6);
}
int launch_env_rollout_tc(int env, const RolloutArgs& a, cudaStream_t s){
    if(env == B200RL_ENV_PENDULUM) return launch_rollout_tc(a, s);
    if(env == B200RL_ENV_ACROBOT_SWINGUP) return launch_env_tc<AcrobotSwingupEnv>(a, s);
    if(env == B200RL_ENV_ACROBOT) return launch_env_tc<AcrobotEnv>(a, s);
    return B200RL_ERR_INVALID_ARGUMENT;
}

}  // namespace b200rl
