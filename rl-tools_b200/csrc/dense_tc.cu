// Tensor-core contraction for the dense layer (sm_100a, tcgen05 + TMEM), fp32 in / fp32 out through the 3xTF32 split:
//   C[m][n] = sum_k A(m,k) * B(n,k)   with   A*B ~= A_lo*B_hi + A_hi*B_lo + A_hi*B_hi   (tf32 parts, fp32 accumulate)
// The operands are plain fp32 matrices in HBM (activations, weights, gradients) in either orientation; the split into
// hi/lo parts cannot be done by a TMA copy, so the 256 threads of the CTA stage each 32-wide k chunk themselves:
// coalesced global loads -> hi/lo split in registers -> K-major, 128-byte-swizzled shared-memory tiles (a transposing
// store when k is not the contiguous index in memory). Two stages: while the tensor core works on chunk c (12
// tcgen05.mma M128 x N x K8 per chunk into a fresh 128 x N TMEM accumulator, committed to the chunk's mbarrier) the threads
// prefetch and stage chunk c+1 and add chunk c-1 from TMEM to their fp32 register accumulators.
// The MMAs are issued by a warp of their own: issuing an M128 x N256 x K8 MMA blocks the thread for about as long as the MMA
// runs (~105 cycles each, measured), so an issuing thread that also stages operands makes every other warp wait for it at the
// next barrier. The CTA therefore has three warpgroups: two stage + accumulate (256 threads, registers raised to 240 with
// setmaxnreg) and one that holds the issuing warp (registers lowered to 24; its other three warps exit). Measured and not
// kept: letting those three warps stage the B operand -- 96 threads cannot keep enough 16-byte loads in flight (Little's law:
// ~17 KB in flight against the ~48 KB the 256 staging threads sustain) and the 65,536 x 256 x 256 forward fell from 114 to 171 us.
// One CTA per SM, persistent over (row tile, column tile, k split) work items; N <= 256 per tile; tiles of <= 64 columns use a
// variant with a quarter of the accumulator registers that prefetches two k chunks ahead.
// Operands whose rows (not k) are contiguous in memory are loaded as 4 x 4 blocks with 16-byte loads and transposed in registers.
// Epilogue: transposition through shared memory with 16-byte accesses so that every global store instruction writes four full
// 128-byte lines, then bias + pre-activation store + activation (forward), plain store (input gradient) or accumulate / split-k
// partial store, optionally transposed (weight gradient).
#include "common.cuh"
#include "dense.cuh"
#include "tcgen05.cuh"
#include <atomic>
#include <type_traits>

namespace b200rl {

namespace {
constexpr int TC_THREADS = 256, TC_LAUNCH_THREADS = 384, TC_M = 128, TC_KC = 32, TC_NMAX = 256;      // 256 staging threads + the issuing warpgroup
constexpr uint32_t A_TILE_BYTES = TC_M * 128;                       // one k chunk of A: 128 rows x 32 tf32
constexpr uint32_t TMEM_COLS = 512;                                  // two 256-column accumulators (one per k chunk in flight)
constexpr long long WAIT_LIMIT_CYCLES = 2000000000LL;
}

// x = hi + lo with BOTH parts rounded to nearest tf32: the tensor core truncates whatever it is given, so rounding here
// keeps the representation error at ~2^-23 |x| (a truncated remainder would leave ~2^-20). This kernel is tensor-bound,
// the two conversions per element are free.
__device__ __forceinline__ void split_rn(float x, float& hi, float& lo){
    // round to nearest (ties away) in integer arithmetic: add half a tf32 ulp to the bit pattern, clear the low 13 bits --
    // two full-rate ALU operations instead of a conversion-pipe instruction
    hi = __uint_as_float((__float_as_uint(x) + 0x1000u) & 0xFFFFE000u);
    const float r = x - hi;
    lo = __uint_as_float((__float_as_uint(r) + 0x1000u) & 0xFFFFE000u);
}

// set to 1 by a kernel whose bounded wait expired (read back through b200rl_device_error_state)
__device__ int g_dense_tc_error = 0;

// Staging of one operand chunk (`rows` x 32 elements, element (r, k) = KCONTIG ? P[r*ld + k] : P[k*ld + r]) is split in
// two halves so that the global-load latency overlaps the tensor-core work on the previous chunk:
//   prefetch_operand : all loads of the chunk are issued back to back into registers (16 bytes per thread and iteration)
//   store_operand    : tf32 hi/lo split and 16-byte stores into the two K-major SW128 tiles (a transposing store when k
//                      is not the contiguous index in memory); rows >= row_limit and k >= k_end are zero.
template <bool KCONTIG, int ITERS>
__device__ __forceinline__ void prefetch_operand(float4 (&reg)[ITERS], const float* __restrict__ P, long long ld, int row0, int row_limit, int rows,
                                                 int k0, int k_end, bool vec_ok, int tid){
#pragma unroll
    for(int it = 0; it < ITERS; it++){
        const int idx = tid + it * TC_THREADS;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if(idx < rows * 8){
            const int r = KCONTIG ? (idx >> 3) : (idx % rows), c = KCONTIG ? (idx & 7) : (idx / rows);
            const int gr = row0 + r, gk = k0 + c * 4;
            if(gr < row_limit){
                if constexpr(KCONTIG){
                    const float* src = P + (long long)gr * ld + gk;
                    if(vec_ok && gk + 3 < k_end) v = __ldg(reinterpret_cast<const float4*>(src));
                    else{
                        if(gk + 0 < k_end) v.x = __ldg(src + 0);
                        if(gk + 1 < k_end) v.y = __ldg(src + 1);
                        if(gk + 2 < k_end) v.z = __ldg(src + 2);
                        if(gk + 3 < k_end) v.w = __ldg(src + 3);
                    }
                }
                else{
                    // consecutive threads read consecutive rows for a fixed k: coalesced
                    const float* src = P + (long long)gk * ld + gr;
                    if(gk + 0 < k_end) v.x = __ldg(src);
                    if(gk + 1 < k_end) v.y = __ldg(src + ld);
                    if(gk + 2 < k_end) v.z = __ldg(src + 2 * ld);
                    if(gk + 3 < k_end) v.w = __ldg(src + 3 * ld);
                }
            }
        }
        reg[it] = v;
    }
}
// Rows contiguous in memory (k is the strided index), 16-byte aligned: a thread takes a 4-row x 4-k block with four 16-byte loads
// ALONG THE ROWS (one per k) instead of sixteen scalar loads; store_operand_blocks transposes the block in registers. Block g of the
// chunk = (k piece c = g % 8, row quad r4 = g / 8): c is the fast index so that the later 16-byte shared-memory stores of a warp cover
// every swizzled piece of four rows (no bank conflicts).
template <int ITERS>
__device__ __forceinline__ void prefetch_operand_blocks(float4 (&reg)[ITERS], const float* __restrict__ P, long long ld, int row0, int row_limit, int rows,
                                                        int k0, int k_end, int tid){
    static_assert(ITERS % 4 == 0);
#pragma unroll
    for(int j = 0; j < ITERS / 4; j++){
        const int g = tid + j * TC_THREADS, c = g & 7, r4 = g >> 3;
        const int gr = row0 + r4 * 4;
#pragma unroll
        for(int kk = 0; kk < 4; kk++){
            const int gk = k0 + c * 4 + kk;
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            if(r4 * 4 < rows && gk < k_end){
                const float* src = P + (long long)gk * ld + gr;
                if(gr + 3 < row_limit) v = __ldg(reinterpret_cast<const float4*>(src));
                else{
                    if(gr + 0 < row_limit) v.x = __ldg(src + 0);
                    if(gr + 1 < row_limit) v.y = __ldg(src + 1);
                    if(gr + 2 < row_limit) v.z = __ldg(src + 2);
                }
            }
            reg[j * 4 + kk] = v;
        }
    }
}
template <int ITERS>
__device__ __forceinline__ void store_operand_blocks(const float4 (&reg)[ITERS], uint8_t* hi_tile, uint8_t* lo_tile, int rows, int tid){
#pragma unroll
    for(int j = 0; j < ITERS / 4; j++){
        const int g = tid + j * TC_THREADS, c = g & 7, r4 = g >> 3;
        if(r4 * 4 < rows){
            const float col[4][4] = {{reg[j * 4 + 0].x, reg[j * 4 + 1].x, reg[j * 4 + 2].x, reg[j * 4 + 3].x},
                                     {reg[j * 4 + 0].y, reg[j * 4 + 1].y, reg[j * 4 + 2].y, reg[j * 4 + 3].y},
                                     {reg[j * 4 + 0].z, reg[j * 4 + 1].z, reg[j * 4 + 2].z, reg[j * 4 + 3].z},
                                     {reg[j * 4 + 0].w, reg[j * 4 + 1].w, reg[j * 4 + 2].w, reg[j * 4 + 3].w}};
#pragma unroll
            for(int rr = 0; rr < 4; rr++){
                const int r = r4 * 4 + rr;
                float4 h, l;
                split_rn(col[rr][0], h.x, l.x); split_rn(col[rr][1], h.y, l.y); split_rn(col[rr][2], h.z, l.z); split_rn(col[rr][3], h.w, l.w);
                const uint32_t off = (uint32_t)r * 128 + ((uint32_t)(c ^ (r & 7)) << 4);
                *reinterpret_cast<float4*>(hi_tile + off) = h;
                *reinterpret_cast<float4*>(lo_tile + off) = l;
            }
        }
    }
}
// dispatch between the two forms (blocks = rows contiguous, aligned, enough registers for whole 4 x 4 blocks)
template <bool KCONTIG, int ITERS>
__device__ __forceinline__ void fetch_chunk(float4 (&reg)[ITERS], const float* __restrict__ P, long long ld, int row0, int row_limit, int rows,
                                            int k0, int k_end, bool vec_ok, int tid){
    if constexpr(!KCONTIG && ITERS % 4 == 0){
        if(vec_ok){ prefetch_operand_blocks<ITERS>(reg, P, ld, row0, row_limit, rows, k0, k_end, tid); return; }
    }
    prefetch_operand<KCONTIG, ITERS>(reg, P, ld, row0, row_limit, rows, k0, k_end, vec_ok, tid);
}
template <bool KCONTIG, int ITERS>
__device__ __forceinline__ void stage_chunk(const float4 (&reg)[ITERS], uint8_t* hi_tile, uint8_t* lo_tile, int rows, bool vec_ok, int tid);

template <bool KCONTIG, int ITERS>
__device__ __forceinline__ void store_operand(const float4 (&reg)[ITERS], uint8_t* hi_tile, uint8_t* lo_tile, int rows, int tid){
#pragma unroll
    for(int it = 0; it < ITERS; it++){
        const int idx = tid + it * TC_THREADS;
        if(idx < rows * 8){
            const int r = KCONTIG ? (idx >> 3) : (idx % rows), c = KCONTIG ? (idx & 7) : (idx / rows);
            float4 h, l;
            split_rn(reg[it].x, h.x, l.x); split_rn(reg[it].y, h.y, l.y); split_rn(reg[it].z, h.z, l.z); split_rn(reg[it].w, h.w, l.w);
            const uint32_t off = (uint32_t)r * 128 + ((uint32_t)(c ^ (r & 7)) << 4);
            *reinterpret_cast<float4*>(hi_tile + off) = h;
            *reinterpret_cast<float4*>(lo_tile + off) = l;
        }
    }
}

template <bool KCONTIG, int ITERS>
__device__ __forceinline__ void stage_chunk(const float4 (&reg)[ITERS], uint8_t* hi_tile, uint8_t* lo_tile, int rows, bool vec_ok, int tid){
    if constexpr(!KCONTIG && ITERS % 4 == 0){
        if(vec_ok){ store_operand_blocks<ITERS>(reg, hi_tile, lo_tile, rows, tid); return; }
    }
    store_operand<KCONTIG, ITERS>(reg, hi_tile, lo_tile, rows, tid);
}

// Per k chunk the tensor core starts a FRESH accumulator (alternating between two 256-column TMEM buffers) and the
// threads add the finished chunk to fp32 registers with round-to-nearest adds. The tensor core's own accumulation
// truncates, so a long chain of dependent MMAs into one accumulator drifts (measured: mean error 1.2e-6 at K = 256 with
// 96 chained MMAs); with 12 MMAs per chain and the cross-chunk sum in registers the result is as accurate as an fp32
// FMA loop.
// NB = 32-column accumulator blocks per thread: 4 for tiles up to 256 columns, 1 for tiles up to 64 columns. The narrow variant has
// registers to spare and prefetches TWO k chunks ahead: with a short MMA per chunk its loop is otherwise one global-load latency per
// chunk long (the 256 -> 16 and 64 -> 256 layers of the training workload spent a third of the step there).
// B_IMG: a.B is a weight image (launch_weight_image): thread 0 brings each chunk's B tiles in with one bulk copy, issued one chunk
// ahead as soon as the stage's previous MMAs have completed; the stage's "full" barrier then waits for the copy's bytes as well as for
// the staging threads' arrival, and the staging threads handle the A operand only.
template <bool A_KCONTIG, bool B_KCONTIG, int EPI, int ACT, int NB, bool B_IMG>
__global__ void __launch_bounds__(TC_LAUNCH_THREADS, 1) gemm_tc_kernel(GemmArgs a, int n_pad, int m_tiles, int n_tiles, int splits, int a_vec, int b_vec, int c_vec){
    static_assert(!B_IMG || (A_KCONTIG && EPI != EPI_ACCUMULATE), "weight images serve the forward and input-gradient products");
    extern __shared__ uint8_t smem_raw[];
    uint8_t* base = smem_raw + ((1024u - (tc::smem_u32(smem_raw) & 1023u)) & 1023u);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t b_tile_bytes = (uint32_t)n_pad * 128;
    const uint32_t stage_bytes = 2 * A_TILE_BYTES + 2 * b_tile_bytes;
    uint8_t* ctrl = base + 2 * stage_bytes;
    uint64_t* chunk_bar = reinterpret_cast<uint64_t*>(ctrl);          // [2]: the MMAs of the chunk using stage / TMEM buffer s have completed
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl + 16);      // [2]: stage s holds the operands of the next chunk
    uint32_t* slot = reinterpret_cast<uint32_t*>(ctrl + 32);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(ctrl + 36);

    if(tid == 0){
        tc::mbar_init(chunk_bar, 1); tc::mbar_init(chunk_bar + 1, 1); tc::mbar_init(full_bar, 1); tc::mbar_init(full_bar + 1, 1);
        tc::fence_mbar_init(); *abort_flag = 0;
    }
    if(warp == 0){ tc::tmem_alloc(slot, TMEM_COLS); tc::tmem_relinquish(); }
    tc::fence_before_thread_sync();
    __syncthreads();
    tc::fence_after_thread_sync();
    const uint32_t tmem_base = *slot;
    const uint32_t idesc = tc::make_idesc_tf32(TC_M, n_pad);
    const int total = m_tiles * n_tiles * splits;

    if(tid >= TC_THREADS){
        // ---- issuing warpgroup: one thread walks the same (work item, chunk) sequence as the staging threads ----
        tc::setmaxnreg_dec<24>();
        if(tid != TC_THREADS) return;
        uint32_t u = 0;
        for(int item = blockIdx.x; item < total; item += gridDim.x){
            const int z = item / (m_tiles * n_tiles);
            const int k_begin = z * a.k_per_split, k_end = min(a.K, k_begin + a.k_per_split);
            const int n_chunks = (k_end - k_begin + TC_KC - 1) / TC_KC;
            for(int c = 0; c < n_chunks; c++, u++){
                const uint32_t s = u & 1;
                if(!tc::mbar_wait_bounded(full_bar + s, (u >> 1) & 1, WAIT_LIMIT_CYCLES) || *abort_flag){ *abort_flag = 1; g_dense_tc_error = 1; return; }
                tc::fence_after_thread_sync();
                uint8_t* stage = base + s * stage_bytes;
                const uint64_t da_hi = tc::make_desc_kmajor_sw128(tc::smem_u32(stage)), da_lo = tc::make_desc_kmajor_sw128(tc::smem_u32(stage + A_TILE_BYTES));
                const uint64_t db_hi = tc::make_desc_kmajor_sw128(tc::smem_u32(stage + 2 * A_TILE_BYTES));
                const uint64_t db_lo = tc::make_desc_kmajor_sw128(tc::smem_u32(stage + 2 * A_TILE_BYTES + b_tile_bytes));
                const uint32_t d = tmem_base + s * 256;
#pragma unroll
                for(int pass = 0; pass < 3; pass++){                 // the small correction terms first, then hi * hi
                    const uint64_t da = pass == 0 ? da_lo : da_hi, db = pass == 1 ? db_lo : db_hi;
#pragma unroll
                    for(int ks = 0; ks < 4; ks++) tc::mma_tf32_ss(d, da + (uint64_t)(ks * 2), db + (uint64_t)(ks * 2), idesc, (pass | ks) ? 1u : 0u);
                }
                tc::commit(chunk_bar + s);
            }
        }
        return;
    }
    tc::setmaxnreg_inc<240>();
    const int q = warp & 3, col_half = warp >> 2;                     // this warp: TMEM lanes 32 q .. +31, 32-column blocks col_half, col_half + 2, ...
    const uint32_t lane_off = (uint32_t)(q * 32) << 16;
    const int n_blocks = (n_pad + 31) / 32;
    uint32_t u = 0;                                                   // running chunk counter: stage and TMEM buffer u & 1
    bool aborted = false;

    // adds the finished chunk (buffer `buf`, barrier phase `parity`) to the register accumulators
    constexpr int SETS = NB == 1 ? 2 : 1;                             // register sets = prefetch distance in chunks
    constexpr int B_ITERS = NB == 1 ? 2 : 8;                          // 16-byte pieces of a B chunk per thread (64 or 256 rows)
    auto accumulate = [&](float (&acc)[NB][32], uint32_t buf, uint32_t parity){
        if(!tc::mbar_wait_bounded(chunk_bar + buf, parity, WAIT_LIMIT_CYCLES)) *abort_flag = 1;
        tc::fence_after_thread_sync();
#pragma unroll
        for(int bi = 0; bi < NB; bi++){
            const int cb = col_half + 2 * bi;
            if(cb < n_blocks){
                uint32_t v[32];
                tc::tmem_ld_32x32(tmem_base + buf * 256 + lane_off + (uint32_t)(cb * 32), v);
                tc::tmem_wait_ld();
#pragma unroll
                for(int j = 0; j < 32; j++) acc[bi][j] += __uint_as_float(v[j]);
            }
        }
    };

    for(int item = blockIdx.x; item < total && !aborted; item += gridDim.x){
        const int z = item / (m_tiles * n_tiles), mn = item % (m_tiles * n_tiles);
        const int m0 = (mn / n_tiles) * TC_M, n0 = (mn % n_tiles) * n_pad;
        const int k_begin = z * a.k_per_split, k_end = min(a.K, k_begin + a.k_per_split);
        const int n_chunks = (k_end - k_begin + TC_KC - 1) / TC_KC;
        const int b_rows = min(n_pad, ((a.N - n0) + 15) / 16 * 16);           // rows of the B tile that can hold data
        float acc[NB][32];
#pragma unroll
        for(int bi = 0; bi < NB; bi++)
#pragma unroll
            for(int j = 0; j < 32; j++) acc[bi][j] = 0.0f;
        float4 ra[SETS][4], rb[B_IMG ? 1 : SETS][B_IMG ? 1 : B_ITERS];
        // image chunk (n tile, k chunk) -> the B area of a stage (hi tile, lo tile: contiguous in both)
        const int k_chunks_total = (a.K + TC_KC - 1) / TC_KC;
        auto load_b_image = [&](int chunk, uint32_t stage_index){
            const size_t index = (size_t)(mn % n_tiles) * k_chunks_total + (size_t)(k_begin / TC_KC + chunk);
            tc::mbar_expect_tx(full_bar + stage_index, 2 * b_tile_bytes);
            tc::bulk_load(base + stage_index * stage_bytes + 2 * A_TILE_BYTES, reinterpret_cast<const uint8_t*>(a.B) + index * 2 * b_tile_bytes, 2 * b_tile_bytes, full_bar + stage_index);
        };
        if constexpr(B_IMG){ if(tid == 0 && n_chunks > 0) load_b_image(0, u & 1); }       // both stages are free at the start of a work item
#pragma unroll
        for(int p = 0; p < SETS; p++){
            if(p < n_chunks){
                fetch_chunk<A_KCONTIG, 4>(ra[p], a.A, a.lda, m0, a.M, TC_M, k_begin + p * TC_KC, k_end, a_vec != 0, tid);
                if constexpr(!B_IMG) fetch_chunk<B_KCONTIG, B_ITERS>(rb[p], a.B, a.ldb, n0, a.N, b_rows, k_begin + p * TC_KC, k_end, b_vec != 0, tid);
            }
        }
        // one k chunk; SET selects the register set at compile time. Returns false when the kernel is aborting.
        auto chunk_body = [&](auto SET, int c) -> bool {
            constexpr int P = decltype(SET)::value;
            const uint32_t s = u & 1;
            uint8_t* stage = base + s * stage_bytes;
            // stage s and TMEM buffer s are free: the chunk that used them last (u - 2) was waited for in the previous iteration
            stage_chunk<A_KCONTIG, 4>(ra[P], stage, stage + A_TILE_BYTES, TC_M, a_vec != 0, tid);
            if constexpr(!B_IMG) stage_chunk<B_KCONTIG, B_ITERS>(rb[P], stage + 2 * A_TILE_BYTES, stage + 2 * A_TILE_BYTES + b_tile_bytes, b_rows, b_vec != 0, tid);
            if(!B_IMG && b_rows < n_pad && c < 2){
                // rows of the padded tile that never receive data: zero them once per stage and work item
                for(int idx = tid; idx < (n_pad - b_rows) * 8; idx += TC_THREADS){
                    const uint32_t off = (uint32_t)(b_rows + (idx >> 3)) * 128 + ((uint32_t)(idx & 7) << 4);
                    *reinterpret_cast<float4*>(stage + 2 * A_TILE_BYTES + off) = make_float4(0.f, 0.f, 0.f, 0.f);
                    *reinterpret_cast<float4*>(stage + 2 * A_TILE_BYTES + b_tile_bytes + off) = make_float4(0.f, 0.f, 0.f, 0.f);
                }
            }
            tc::fence_proxy_async_smem();
            tc::fence_before_thread_sync();
            tc::named_barrier_sync(1, TC_THREADS);
            if(*abort_flag) return false;
            if(tid == 0) tc::mbar_arrive(full_bar + s);              // the issuing warp takes over from here
            if(c + SETS < n_chunks){
                const int k0 = k_begin + (c + SETS) * TC_KC;
                fetch_chunk<A_KCONTIG, 4>(ra[P], a.A, a.lda, m0, a.M, TC_M, k0, k_end, a_vec != 0, tid);
                if constexpr(!B_IMG) fetch_chunk<B_KCONTIG, B_ITERS>(rb[P], a.B, a.ldb, n0, a.N, b_rows, k0, k_end, b_vec != 0, tid);
            }
            if(c > 0) accumulate(acc, s ^ 1, ((u - 1) >> 1) & 1);
            // the other stage is free now (chunk c-1, its last user, has completed; the first chunk of an item finds it free anyway):
            // bring in the weights of chunk c+1 while chunk c runs on the tensor core
            if constexpr(B_IMG){ if(tid == 0 && c + 1 < n_chunks){ tc::fence_after_thread_sync(); load_b_image(c + 1, s ^ 1); } }
            u++;
            return true;
        };
        for(int c = 0; c < n_chunks && !aborted; c += SETS){
            if(!chunk_body(std::integral_constant<int, 0>{}, c)){ aborted = true; break; }
            if constexpr(SETS == 2){
                if(c + 1 < n_chunks && !chunk_body(std::integral_constant<int, 1>{}, c + 1)){ aborted = true; break; }
            }
        }
        if(aborted) break;
        accumulate(acc, (u - 1) & 1, ((u - 1) >> 1) & 1);
        // a wait that ran out leaves half-finished sums in the accumulators: nothing of this work item may reach global memory
        // (an accumulating epilogue would corrupt the gradient). The barrier makes the decision the same for every thread.
        tc::named_barrier_sync(1, TC_THREADS);
        if(*abort_flag){ aborted = true; break; }

        // ---- epilogue, vector form (forward / plain store with 16-byte aligned rows): the warp transposes each 32 x 32 block through a
        // private shared-memory patch with 16-byte accesses on both sides (row pitch 36 floats: conflict-free for both the row-wise
        // writes and the 8-lanes-per-row reads), so that every global store instruction writes four full 128-byte lines.
        // (The scalar form below issues 32 four-byte-per-lane stores per block and output: ~16 k cycles per 128 x 256 tile. Measured
        // and not kept: storing straight from the accumulator registers, 16 bytes per lane and one row per lane -- every instruction then
        // touches 32 half-filled sectors and the 256 -> 256 forward went from 114 to 167 us.) ----
        bool direct = false;
        if constexpr(EPI != EPI_ACCUMULATE) direct = (c_vec & 1) && (EPI != EPI_FORWARD || a.pre == nullptr || (c_vec & 2));
        if(direct){
            float* vpatch = reinterpret_cast<float*>(base) + warp * (32 * 36);
            const int g = lane & 7, rsub = lane >> 3;
#pragma unroll
            for(int bi = 0; bi < NB; bi++){
                const int cb = col_half + 2 * bi;
                if(cb >= n_blocks) continue;
#pragma unroll
                for(int j4 = 0; j4 < 8; j4++)
                    *reinterpret_cast<float4*>(vpatch + lane * 36 + 4 * j4) = make_float4(acc[bi][4 * j4], acc[bi][4 * j4 + 1], acc[bi][4 * j4 + 2], acc[bi][4 * j4 + 3]);
                __syncwarp();
                const int n = n0 + cb * 32 + 4 * g;
                const bool n_ok = cb * 32 + 4 * g < n_pad && n < a.N, full = n + 3 < a.N;
                float bias4[4] = {0.f, 0.f, 0.f, 0.f};
                if constexpr(EPI == EPI_FORWARD){
                    if(n_ok){
                        if(full && (c_vec & 4)){ const float4 b4 = __ldg(reinterpret_cast<const float4*>(a.bias + n)); bias4[0] = b4.x; bias4[1] = b4.y; bias4[2] = b4.z; bias4[3] = b4.w; }
                        else{
#pragma unroll
                            for(int e = 0; e < 4; e++) if(n + e < a.N) bias4[e] = __ldg(a.bias + n + e);
                        }
                    }
                }
#pragma unroll
                for(int it = 0; it < 8; it++){
                    const int r = 4 * it + rsub, m = m0 + q * 32 + r;
                    if(m < a.M && n_ok){
                        const float4 v = *reinterpret_cast<const float4*>(vpatch + r * 36 + 4 * g);
                        float x[4] = {v.x, v.y, v.z, v.w};
                        float* crow = a.C + (long long)m * a.ldc + n;
                        if constexpr(EPI == EPI_FORWARD){
#pragma unroll
                            for(int e = 0; e < 4; e++) x[e] += bias4[e];
                            if(a.pre){
                                float* prow = a.pre + (long long)m * a.ldpre + n;
                                if(full) *reinterpret_cast<float4*>(prow) = make_float4(x[0], x[1], x[2], x[3]);
                                else{
#pragma unroll
                                    for(int e = 0; e < 4; e++) if(n + e < a.N) prow[e] = x[e];
                                }
                            }
#pragma unroll
                            for(int e = 0; e < 4; e++) x[e] = activation<ACT>(x[e]);
                        }
                        if(full) *reinterpret_cast<float4*>(crow) = make_float4(x[0], x[1], x[2], x[3]);
                        else{
#pragma unroll
                            for(int e = 0; e < 4; e++) if(n + e < a.N) crow[e] = x[e];
                        }
                    }
                }
                __syncwarp();
            }
        }
        // ---- epilogue, transposing form: through a warp-private 32 x 33 patch (stage 0 is free: every MMA has completed), so
        // that each global store instruction writes one full 128-byte row segment ----
        float* patch = reinterpret_cast<float*>(base) + warp * (32 * 33);
#pragma unroll
        for(int bi = 0; bi < NB; bi++){
            const int cb = col_half + 2 * bi;
            if(cb >= n_blocks || direct) continue;
#pragma unroll
            for(int j = 0; j < 32; j++) patch[lane * 33 + j] = acc[bi][j];
            __syncwarp();
            const int n = n0 + cb * 32 + lane;
            const bool n_ok = cb * 32 + lane < n_pad && n < a.N;
            float bias = 0.0f;
            if constexpr(EPI == EPI_FORWARD){ if(n_ok) bias = __ldg(a.bias + n); }
            for(int r = 0; r < 32; r++){
                const int m = m0 + q * 32 + r;
                if(m >= a.M || !n_ok) continue;
                float x = patch[r * 33 + lane];
                if constexpr(EPI == EPI_FORWARD){
                    x += bias;
                    if(a.pre) a.pre[(long long)m * a.ldpre + n] = x;
                    a.C[(long long)m * a.ldc + n] = activation<ACT>(x);
                }
                else if constexpr(EPI == EPI_STORE){
                    a.C[(long long)m * a.ldc + n] = x;
                }
                else{
                    if(a.transpose_c){
                        if(splits == 1) a.C[(long long)n * a.ldc + m] += x;
                        else a.partial[((long long)z * a.N + n) * a.M + m] = x;
                    }
                    else{
                        if(splits == 1) a.C[(long long)m * a.ldc + n] += x;
                        else a.partial[((long long)z * a.M + m) * a.N + n] = x;
                    }
                }
            }
            __syncwarp();
        }
        tc::fence_before_thread_sync();
        tc::named_barrier_sync(1, TC_THREADS);         // the patch area (stage 0) is overwritten by the next work item
        if(*abort_flag){ aborted = true; break; }
    }
    if(aborted && tid == 0) g_dense_tc_error = 1;
    tc::fence_before_thread_sync();
    tc::named_barrier_sync(1, TC_THREADS);
    if(warp == 0) tc::tmem_dealloc(tmem_base, TMEM_COLS);
}

template <bool A_KC, bool B_KC, int EPI, int ACT, int NB, bool B_IMG = false>
static int launch_variant(const GemmArgs& a, int splits, int n_pad, cudaStream_t s){
    const int n_tiles = (a.N + n_pad - 1) / n_pad, m_tiles = (a.M + TC_M - 1) / TC_M;
    const uint32_t smem = 2 * (2 * A_TILE_BYTES + 2 * (uint32_t)n_pad * 128) + 64 + 1024;
    // the attribute belongs to the (function, device) pair: one flag per device ordinal
    static std::atomic<bool> configured[MAX_DEVICES];
    int dev = 0, sms = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    if(!configured[dev].load(std::memory_order_acquire)){
        B200RL_CUDA_TRY(cudaFuncSetAttribute(gemm_tc_kernel<A_KC, B_KC, EPI, ACT, NB, B_IMG>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(2 * (2 * A_TILE_BYTES + 2 * TC_NMAX * 128) + 64 + 1024)));
        configured[dev].store(true, std::memory_order_release);
    }
    rc = sm_count(&sms);
    if(rc) return rc;
    const long long total = (long long)m_tiles * n_tiles * splits;
    const int grid = (int)(total < sms ? total : sms);
    auto aligned = [](const float* p, long long ld){ return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && (ld & 3) == 0; };
    // k-contiguous operands: 16-byte loads along k need an aligned base, pitch and k range; row-contiguous operands: 16-byte loads along
    // the rows need an aligned base and pitch (tile origins are multiples of 16 rows)
    const int a_vec = aligned(a.A, a.lda) && (!A_KC || a.k_per_split % 4 == 0), b_vec = aligned(a.B, a.ldb) && (!B_KC || a.k_per_split % 4 == 0);
    const int c_vec = (aligned(a.C, a.ldc) ? 1 : 0) | ((a.pre == nullptr || aligned(a.pre, a.ldpre)) ? 2 : 0) |
                      ((a.bias != nullptr && (reinterpret_cast<uintptr_t>(a.bias) & 15u) == 0) ? 4 : 0);
    gemm_tc_kernel<A_KC, B_KC, EPI, ACT, NB, B_IMG><<<grid, TC_LAUNCH_THREADS, smem, s>>>(a, n_pad, m_tiles, n_tiles, splits, a_vec, b_vec, c_vec);
    B200RL_LAUNCH_CHECK("gemm_tc");
    return B200RL_OK;
}
static int tile_columns(int N){
    int n_pad = (N + 15) / 16 * 16;
    return n_pad > TC_NMAX ? TC_NMAX : n_pad;
}
template <bool A_KC, bool B_KC, int EPI, int ACT, bool B_IMG = false>
static int launch_one(const GemmArgs& a, int splits, cudaStream_t s){
    const int n_pad = tile_columns(a.N);
    if(n_pad <= 64) return launch_variant<A_KC, B_KC, EPI, ACT, 1, B_IMG>(a, splits, n_pad, s);
    return launch_variant<A_KC, B_KC, EPI, ACT, 4, B_IMG>(a, splits, n_pad, s);
}

// ---- weight image: one thread per 16-byte piece (4 k values of one row) of the image ----
__global__ void __launch_bounds__(256) weight_image_kernel(const float* __restrict__ W, long long ld, int N, int K, int transposed, int n_pad, int n_tiles, int k_chunks,
                                                           uint8_t* __restrict__ image){
    const long long piece = blockIdx.x * (long long)blockDim.x + threadIdx.x, pieces = (long long)n_tiles * k_chunks * n_pad * 8;
    if(piece >= pieces) return;
    const int c = (int)(piece & 7), row = (int)((piece >> 3) % n_pad);
    const long long tile = (piece >> 3) / n_pad;                         // n tile * k_chunks + k chunk
    const int chunk = (int)(tile % k_chunks), n = (int)(tile / k_chunks) * n_pad + row, k0 = chunk * TC_KC + c * 4;
    float4 h = make_float4(0.f, 0.f, 0.f, 0.f), l = h;
    if(n < N){
        float v[4];
#pragma unroll
        for(int e = 0; e < 4; e++){
            const int k = k0 + e;
            v[e] = k < K ? (transposed ? __ldg(W + (long long)k * ld + n) : __ldg(W + (long long)n * ld + k)) : 0.0f;
        }
        split_rn(v[0], h.x, l.x); split_rn(v[1], h.y, l.y); split_rn(v[2], h.z, l.z); split_rn(v[3], h.w, l.w);
    }
    const size_t tile_bytes = (size_t)n_pad * 128, off = (size_t)row * 128 + ((size_t)(c ^ (row & 7)) << 4);
    *reinterpret_cast<float4*>(image + (size_t)tile * 2 * tile_bytes + off) = h;
    *reinterpret_cast<float4*>(image + (size_t)tile * 2 * tile_bytes + tile_bytes + off) = l;
}
size_t weight_image_bytes(int N, int K){
    const int n_pad = tile_columns(N);
    return (size_t)((N + n_pad - 1) / n_pad) * (size_t)((K + TC_KC - 1) / TC_KC) * 2 * (size_t)n_pad * 128;
}
int launch_weight_image(const float* W, long long ld, int N, int K, bool transposed, float* image, cudaStream_t s){
    if((reinterpret_cast<uintptr_t>(image) & 15u) != 0) return B200RL_ERR_INVALID_ARGUMENT;
    const int n_pad = tile_columns(N), n_tiles = (N + n_pad - 1) / n_pad, k_chunks = (K + TC_KC - 1) / TC_KC;
    const long long pieces = (long long)n_tiles * k_chunks * n_pad * 8;
    weight_image_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, s>>>(W, ld, N, K, transposed ? 1 : 0, n_pad, n_tiles, k_chunks, reinterpret_cast<uint8_t*>(image));
    B200RL_LAUNCH_CHECK("weight_image");
    return B200RL_OK;
}

int launch_gemm_tc(const GemmArgs& a, int epilogue, int activation, bool a_kcontig, bool b_kcontig, int splits, cudaStream_t s, bool b_image){
    if(a.M < 1 || a.N < 1 || a.K < 1) return B200RL_ERR_UNSUPPORTED;
    if(b_image){
        if(!a_kcontig || splits != 1 || a.k_per_split < a.K) return B200RL_ERR_UNSUPPORTED;
        if(epilogue == EPI_FORWARD){ B200RL_DISPATCH_ACT(activation, return (launch_one<true, true, EPI_FORWARD, ACT, true>(a, 1, s))); }
        if(epilogue == EPI_STORE) return launch_one<true, true, EPI_STORE, 0, true>(a, 1, s);
        return B200RL_ERR_UNSUPPORTED;
    }
    if(epilogue == EPI_FORWARD && a_kcontig && b_kcontig){
        B200RL_DISPATCH_ACT(activation, return (launch_one<true, true, EPI_FORWARD, ACT>(a, 1, s)));
    }
    if(epilogue == EPI_STORE && a_kcontig && !b_kcontig) return launch_one<true, false, EPI_STORE, 0>(a, 1, s);
    if(epilogue == EPI_STORE && a_kcontig && b_kcontig) return launch_one<true, true, EPI_STORE, 0>(a, 1, s);
    if(epilogue == EPI_ACCUMULATE && !a_kcontig && !b_kcontig) return launch_one<false, false, EPI_ACCUMULATE, 0>(a, splits, s);
    return B200RL_ERR_UNSUPPORTED;
}

}  // namespace b200rl

extern "C" int b200rl_device_error_state(int* state_host){
    if(!state_host) return B200RL_ERR_INVALID_ARGUMENT;
    B200RL_CUDA_TRY(cudaMemcpyFromSymbol(state_host, b200rl::g_dense_tc_error, sizeof(int)));
    return B200RL_OK;
}
extern "C" int b200rl_device_error_clear(void){
    const int zero = 0;
    B200RL_CUDA_TRY(cudaMemcpyToSymbol(b200rl::g_dense_tc_error, &zero, sizeof(int)));
    return B200RL_OK;
}
