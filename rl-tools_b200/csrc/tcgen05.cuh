// Thin inline-PTX wrappers for the Blackwell (sm_100a) tensor-core path: TMEM allocation, tcgen05.mma with
// shared-memory operand descriptors, tcgen05.commit -> mbarrier, tcgen05.ld, proxy fences, bounded mbarrier waits,
// and bulk (TMA) shared->global stores. Everything here is single-CTA (cta_group::1): every copy has exactly one destination.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200rl { namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void* p){ return (uint32_t)__cvta_generic_to_shared(p); }

// ---- TMEM allocation (one full warp executes these) -----------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns){   // columns: power of two, 32..512
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" :: "r"(smem_u32(smem_slot)), "r"(columns) : "memory");
}
__device__ __forceinline__ void tmem_relinquish(){
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t tmem_addr, uint32_t columns){
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" :: "r"(tmem_addr), "r"(columns) : "memory");
}

// ---- fences --------------------------------------------------------------------------------------------------
__device__ __forceinline__ void fence_before_thread_sync(){ asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_thread_sync(){ asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// makes this thread's generic-proxy shared-memory writes visible to the async proxy (tensor core / bulk copies)
__device__ __forceinline__ void fence_proxy_async_smem(){ asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- mbarrier -------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count){
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar){
    asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" :: "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void fence_mbar_init(){ asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity){
    uint32_t done;
    // the last operand is a suspend-time hint: the thread sleeps in hardware until the phase completes (or the hint
    // expires) instead of burning issue slots that the other groups of the CTA need
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(done) : "r"(smem_u32(bar)), "r"(parity), "r"(0x989680u) : "memory");
    return done != 0;
}
// Waits for the phase with the given parity, giving up after ~limit_cycles SM clocks. Returns false on time-out so
// the caller can raise an error flag and leave instead of spinning forever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, long long limit_cycles){
    if(mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while(!mbar_try_wait(bar, parity)){
        if(clock64() - t0 > limit_cycles) return false;
    }
    return true;
}

// transaction count of the barrier's current phase += bytes (the phase then also waits for that many bytes of bulk copies)
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes){
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" :: "r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// bulk (TMA) load global -> this CTA's shared memory, one destination; completion is signalled on the mbarrier as `bytes` transaction
// bytes. Both addresses 16-byte aligned, size a multiple of 16 bytes.
__device__ __forceinline__ void bulk_load(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar){
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 :: "r"(smem_u32(smem)), "l"(gmem), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

// ---- operand descriptors -------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major operand stored with the 128-byte swizzle: rows of 128 bytes
// (32 tf32 values along K), 8-row groups 1024 bytes apart, 16-byte chunk index XORed with (row mod 8); the tile
// base must be 1024-byte aligned. Advancing along K inside the 128-byte row adds the byte offset to the start
// address field (units of 16 bytes).
__device__ __forceinline__ uint64_t make_desc_kmajor_sw128(uint32_t smem_addr){
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);          // start address
    d |= (uint64_t)1 << 16;                               // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                     // stride byte offset: 8 rows x 128 B
    d |= (uint64_t)1 << 46;                               // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                               // layout type: SWIZZLE_128B
    return d;
}
// Descriptor for a K-major operand WITHOUT swizzle whose K extent is one instruction (8 tf32 = 32 bytes per row): "core
// matrices" of 8 rows x 16 bytes are stored contiguously (row i at +16 i); the second 16-byte K chunk of the same 8 rows
// follows at +128 bytes (leading byte offset), the next 8 rows at +256 bytes (stride byte offset). A 128-row tile is 4 KB.
__device__ __forceinline__ uint64_t make_desc_kmajor_noswizzle_k8(uint32_t smem_addr){
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr >> 4) & 0x3FFF);
    d |= (uint64_t)(128 >> 4) << 16;                      // leading byte offset: next K chunk
    d |= (uint64_t)(256 >> 4) << 32;                      // stride byte offset: next 8 rows
    d |= (uint64_t)1 << 46;                               // descriptor version (Blackwell)
    return d;                                             // layout type 0: no swizzle
}
// byte offset of element (row, k) inside such a tile
__host__ __device__ constexpr uint32_t noswizzle_k8_offset(uint32_t row, uint32_t k){
    return (row >> 3) * 256u + (k >> 2) * 128u + (row & 7u) * 16u + (k & 3u) * 4u;
}
// Instruction descriptor for kind::tf32, fp32 accumulate, both operands K-major, shape M x N (K = 8 per instruction)
__host__ __device__ constexpr uint32_t make_idesc_tf32(int M, int N){
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// The same for kind::f16 with fp16 operands (K = 16 per instruction, 32 bytes per row like the tf32 K = 8 step), fp32 accumulate
__host__ __device__ constexpr uint32_t make_idesc_f16(int M, int N){
    return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}
// byte offset of element (row, k) of a K = 16 fp16 tile without swizzle (the layout of make_desc_kmajor_noswizzle_k8 with 2-byte elements)
__host__ __device__ constexpr uint32_t noswizzle_k16_offset(uint32_t row, uint32_t k){
    return (row >> 3) * 256u + (k >> 3) * 128u + (row & 7u) * 16u + (k & 7u) * 2u;
}
__device__ __forceinline__ void mma_f16_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate){
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
// fp16 A operand from tensor memory: lane = row, two consecutive K elements per 32-bit column
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate){
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 :: "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; issued by ONE thread
__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate){
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 :: "r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
// same with the A operand read from tensor memory (lane = row, one 32-bit column per K element)
__device__ __forceinline__ void mma_tf32_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate){
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
                 :: "r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u) : "memory");
}
// mbarrier arrives (count 1) once every tcgen05 operation issued so far by this thread has completed
__device__ __forceinline__ void commit(uint64_t* bar){
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" :: "r"(smem_u32(bar)) : "memory");
}

// ---- TMEM -> registers: 32 lanes x 32 consecutive columns; a warp reads its own lane quarter (warp_id % 4) ------
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]){
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
                   "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
                   "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
                 : "r"(taddr) : "memory");
}
// registers -> TMEM, same shape: thread i of the warp writes 32 consecutive columns of lane (warp quarter base + i)
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]){
    asm volatile("tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
                 "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
                 :: "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                    "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
                    "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
                    "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31]) : "memory");
}
__device__ __forceinline__ void tmem_wait_st(){ asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld(){ asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- register reallocation between warpgroups (all four warps of a warpgroup execute the same instruction) ------------------
template <int N> __device__ __forceinline__ void setmaxnreg_inc(){ asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" :: "n"(N)); }
template <int N> __device__ __forceinline__ void setmaxnreg_dec(){ asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" :: "n"(N)); }

// ---- named barrier for a sub-group of the CTA (id 1..15; id 0 is __syncthreads) ---------------------------------------
__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads){
    asm volatile("bar.sync %0, %1;" :: "r"(id), "r"(threads) : "memory");
}

// ---- bulk (TMA) store shared -> global: both addresses 16-byte aligned, size a multiple of 16 bytes --------------
__device__ __forceinline__ void bulk_store(void* gmem, const void* smem, uint32_t bytes){
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" :: "l"(gmem), "r"(smem_u32(smem)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit(){ asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read(){ asm volatile("cp.async.bulk.wait_group.read %0;" :: "n"(N) : "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_all(){ asm volatile("cp.async.bulk.wait_group %0;" :: "n"(N) : "memory"); }

// ---- 3xTF32 split: x = hi + lo with hi = round-to-nearest tf32(x), lo = x - hi (exact in fp32) ---------------------
__device__ __forceinline__ void split_tf32(float x, float& hi, float& lo){
    uint32_t h;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    lo = x - hi;
}

}}  // namespace b200rl::tc
