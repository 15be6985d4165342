// Building blocks shared by the tcgen05 / TMEM matmul kernels (sm_100a only): inline-PTX
// wrappers for mbarriers, TMA loads, tcgen05 MMA / commit / TMEM loads, bounded waits, the
// persistent work-item cursor, the warp-wide block-descriptor window and the host-side tensor
// map encoder.  Everything lives in an anonymous namespace: each kernel file gets its own copy.
#pragma once
#include <cstdio>
#include <mutex>

#include "bsa_common.cuh"

namespace bsa {
namespace {

constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s
constexpr int kTile = 64;                       // edge of a 16-bit operand tile in elements
constexpr int kTileBytes = kTile * kTile * 2;   // 8 KB

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (for a role that polls several barriers and serves whichever is ready).
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the wait was given up (time-out here, or an abort raised by
// another role of this CTA through `abort_flag`, a word in shared memory).
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, int* abort_flag, uint32_t* status) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*(volatile int*)abort_flag) return false;
        if (global_ns() - t0 > kWaitLimitNs) {
            *(volatile int*)abort_flag = 1;
            atomicExch(status, (uint32_t)BSA_ERR_DEVICE_TIMEOUT);
            return false;
        }
    }
}
// After an abort a producer's copies may still be in flight, and they must not land in shared memory
// that the SM has already handed to the next CTA.  An mbarrier cannot tell a stage that is being
// filled from an idle one (one of its two parity tests passes at any time), so the producer waits a
// fixed time that is long against a copy's latency (a few microseconds) before it leaves.
constexpr unsigned long long kCopyDrainNs = 200000ull;      // 0.2 ms
__device__ __forceinline__ void let_copies_land() {
    const unsigned long long t0 = global_ns();
    while (global_ns() - t0 < kCopyDrainNs) {}
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, int* abort_flag, uint32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, status);
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16).
__device__ __forceinline__ void bulk_load_1d(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// True in exactly one lane of a converged warp.  Code around an `if (elect_one())` stays
// warp-uniform, so the descriptors of the tcgen05 instructions inside it are computed once per
// warp in uniform registers instead of being moved there per instruction.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.u32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}

__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];"
                 ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void tc_mma_f16(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_32x32b_x64(uint32_t taddr, uint32_t (&r)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, "
        "%32, %33, %34, %35, %36, %37, %38, %39, %40, %41, %42, %43, %44, %45, %46, %47, "
        "%48, %49, %50, %51, %52, %53, %54, %55, %56, %57, %58, %59, %60, %61, %62, %63}, [%64];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31]),
          "=r"(r[32]), "=r"(r[33]), "=r"(r[34]), "=r"(r[35]), "=r"(r[36]), "=r"(r[37]), "=r"(r[38]), "=r"(r[39]),
          "=r"(r[40]), "=r"(r[41]), "=r"(r[42]), "=r"(r[43]), "=r"(r[44]), "=r"(r[45]), "=r"(r[46]), "=r"(r[47]),
          "=r"(r[48]), "=r"(r[49]), "=r"(r[50]), "=r"(r[51]), "=r"(r[52]), "=r"(r[53]), "=r"(r[54]), "=r"(r[55]),
          "=r"(r[56]), "=r"(r[57]), "=r"(r[58]), "=r"(r[59]), "=r"(r[60]), "=r"(r[61]), "=r"(r[62]), "=r"(r[63])
        : "r"(taddr) : "memory");
}
// 16 TMEM lanes x 64 columns spread over all 32 threads: thread t gets, for each 8-column
// unit u, r[4u + 0,1] = (lane t/4, columns 8u + 2(t%4) + 0,1) and r[4u + 2,3] = the same columns
// of lane t/4 + 8 (the layout of an m16n8 accumulator fragment).
__device__ __forceinline__ void tc_ld_16x256b_x8(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void st_global_v8(void* ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// ---- helpers of the fused attention kernels
__device__ __forceinline__ float attn_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Three-input maximum / minimum and two-wide fp32 arithmetic (one instruction for two lanes of a
// 64-bit register pair): they halve the instruction count of the softmax element loops.
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ float fmin3(float a, float b, float c) {
    float d;
    asm("min.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_pack(float lo, float hi) {
    uint64_t d;
    asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(lo), "f"(hi));
    return d;
}
__device__ __forceinline__ void f2_unpack(uint64_t v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ uint64_t f2_fma(uint64_t a, uint64_t b, uint64_t c) {
    uint64_t d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ uint64_t f2_add(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ uint64_t f2_mul(uint64_t a, uint64_t b) {
    uint64_t d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
// Four 8 x 8 matrices of 16-bit elements from the m8n8 fragment layout (lane t holds elements
// 2 (t % 4) + {0, 1} of row t / 4 of each matrix) to shared memory; lanes 8 i .. 8 i + 7 give the row
// addresses of matrix i.
__device__ __forceinline__ void stmatrix_x4(uint32_t addr, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                 ::"r"(addr), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
}

// 16 TMEM lanes x 16 columns, same thread mapping as the .x8 load of the common header:
// r[4u + 0,1] = (lane t/4, columns 8u + 2(t%4) + 0,1), r[4u + 2,3] = the same columns of lane t/4 + 8.
__device__ __forceinline__ void tc_ld_16x256b_x2(uint32_t taddr, uint32_t (&r)[8]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x2.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_ld_16x256b_x4(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.16x256b.x4.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tc_st_16x256b_x2(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.16x256b.x2.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}
// 16 TMEM lanes x 32 columns of 32-bit words: r[2u] goes to (lane t / 4, column 4u + t % 4), r[2u + 1] to the
// same column of lane t / 4 + 8.  With two 16-bit values per word this is the layout of a 16 x 64 K-major A
// operand in tensor memory when r[2u], r[2u + 1] hold the packed elements 8u + 2 (t % 4) + {0, 1} of the two rows.
__device__ __forceinline__ void tc_st_16x128b_x8(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
                   "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
                 : "memory");
}
__device__ __forceinline__ void tc_st_16x128b_x4(uint32_t taddr, const uint32_t (&r)[8]) {
    asm volatile("tcgen05.st.sync.aligned.16x128b.x4.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]) : "memory");
}
// D (+)= A B with the A operand in tensor memory (M rows on the lanes, two 16-bit K elements per column)
__device__ __forceinline__ void tc_mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t desc_b, uint32_t idesc,
                                              uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(tmem_d), "r"(tmem_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
    if (BF16) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t*>(&h);
    }
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// Iterates the work items of one CTA (item = blockIdx.x + n * gridDim.x) and keeps the group
// offset-table words of the next two items in flight, so that by the time an item becomes
// current its words have arrived and no role stalls on a dependent global load per item.
// Positions advance incrementally (the host passes gridDim.x split by the items per batch
// entry): an integer division by a run-time value costs a lone thread hundreds of cycles.
struct Cursor {
    int item, stride, items, chunks, per_z, stride_z, stride_rem;
    int groups, zstep, rot;             // groups per batch entry; stride_z mod groups; 1: rotate the groups (below)
    int table_shift;                    // group g reads table[g >> table_shift] (1: two virtual groups per real one)
    const int32_t* table;
    int item_no;                        // how many items this CTA has finished
    int z, g, chunk, first, count;      // current item: batch entry, group, slice, block range
    int z1, r1, m1, a1, b1;             // next item: batch entry, index inside it, z mod groups, table[g], table[g + 1]
    int z2, r2, m2, a2, b2;             // the item after that

    // Group of position `rem` of batch entry z (zm = z mod groups if the walk is rotated, else 0).  Rotated, batch
    // entry z starts its groups at group z mod groups instead of group 0: layouts keep their long groups at fixed
    // places (the global rows and columns of a BigBird or local + global layout), and with every batch entry
    // starting at group 0 those land on the few walkers whose number is congruent to their position modulo
    // gcd(groups, walkers) -- 74 of 592 pipelines of the fused forward took all 128-block rows of benchmark
    // configuration 5 (2.2 times the mean load); rotated they spread over all walkers (1.03).  The fused kernels
    // rotate; the matmul engines do not (their dsd by rows ran 11 % slower rotated on that configuration).
    __device__ __forceinline__ int group_of(int rem, int zm, int& lin) const {
        lin = chunks == 1 ? rem : rem / chunks;
        int gg = lin + zm;
        if (gg >= groups) gg -= groups;
        return gg;
    }
    __device__ __forceinline__ void load_words(bool in_range, int rem, int zm, int& a, int& b) const {
        a = 0; b = 0;
        if (in_range) {
            int lin;
            const int gg = group_of(rem, zm, lin) >> table_shift;
            a = table[gg]; b = table[gg + 1];
        }
    }
    __device__ __forceinline__ void step_pos(int& zz, int& rem, int& zm) const {
        zz += stride_z;
        zm += zstep;
        rem += stride_rem;
        if (rem >= per_z) { rem -= per_z; ++zz; zm += rot; }
        if (zm >= groups) zm -= groups;             // zm < groups + zstep + 1 <= 2 * groups before this
    }
    __device__ __forceinline__ void set_current(int zz, int rem, int zm, int a, int b) {
        int lin;
        z = zz;
        g = group_of(rem, zm, lin);
        chunk = rem - lin * chunks;
        first = a;
        count = b - a;
    }
    // The walker is number `first_item` of `walkers` (the CTA and the grid, or a pipeline of a CTA and the
    // number of pipelines in the grid); p.stride_z / p.stride_rem are `walkers` split by the items per batch entry.
    template <class Params>
    __device__ __forceinline__ void init(const Params& p, int shift = 0, bool rotate = false) { init_as(p, (int)blockIdx.x, (int)gridDim.x, shift, rotate); }
    template <class Params>
    __device__ __forceinline__ void init_as(const Params& p, int first_item, int walkers, int shift = 0, bool rotate = false) {
        table_shift = shift;
        rot = rotate ? 1 : 0;
        item = first_item; stride = walkers; items = p.items;
        chunks = p.chunks; per_z = p.groups * p.chunks; table = p.table;
        stride_z = p.stride_z; stride_rem = p.stride_rem;
        groups = p.groups; zstep = rotate ? p.stride_z % p.groups : 0;      // (two divisions per walker and launch)
        item_no = 0;
        z = g = chunk = first = count = 0;
        int z0 = item / per_z, r0 = item - z0 * per_z, m0 = rotate ? z0 % groups : 0, a0, b0;
        load_words(item < items, r0, m0, a0, b0);
        z1 = z0; r1 = r0; m1 = m0; step_pos(z1, r1, m1);
        load_words(item + stride < items, r1, m1, a1, b1);
        z2 = z1; r2 = r1; m2 = m1; step_pos(z2, r2, m2);
        load_words(item + 2 * stride < items, r2, m2, a2, b2);
        if (item < items) set_current(z0, r0, m0, a0, b0);
    }
    __device__ __forceinline__ bool valid() const { return item < items; }
    __device__ __forceinline__ bool has_next() const { return item + stride < items; }
    __device__ __forceinline__ int next_first() const { return a1; }
    __device__ __forceinline__ int next_count() const { return b1 - a1; }
    __device__ __forceinline__ int next_z() const { return z1; }
    __device__ __forceinline__ int next_group() const { int lin; return group_of(r1, m1, lin); }
    __device__ __forceinline__ void advance() {
        item += stride;
        ++item_no;
        const int zc = z1, rc = r1, mc = m1, ac = a1, bc = b1;
        z1 = z2; r1 = r2; m1 = m2; a1 = a2; b1 = b2;
        step_pos(z2, r2, m2);
        load_words(item + 2 * stride < items, r2, m2, a2, b2);
        if (item < items) set_current(zc, rc, mc, ac, bc);
    }
};

// A warp-wide window of 32 block descriptors of the current group: lane l holds descriptor
// base + l and the following 32 are already being loaded.  get() must be called by all 32
// lanes with the same index, in non-decreasing order; indices may be skipped.
struct DescWindow {
    BlockDesc mine, ahead;
    int base;
    __device__ __forceinline__ void begin(const BlockDesc* blocks, int first, int count, const BlockDesc& first_chunk,
                                          int lane) {
        mine = first_chunk;
        base = 0;
        ahead = BlockDesc{0, 0};
        if (32 + lane < count) ahead = blocks[first + 32 + lane];
    }
    // Moves the window on until it holds descriptor i (and the 31 after its base); lane l then finds
    // descriptor base + l in `mine`.
    __device__ __forceinline__ void seek(const BlockDesc* blocks, int first, int count, int i, int lane) {
        while (i >= base + 32) {
            mine = ahead;
            base += 32;
            if (base + 32 + lane < count) ahead = blocks[first + base + 32 + lane];
        }
    }
    __device__ __forceinline__ BlockDesc get(const BlockDesc* blocks, int first, int count, int i, int lane) {
        seek(blocks, first, count, i, lane);
        BlockDesc d;
        d.idx = __shfl_sync(0xffffffffu, mine.idx, i - base);
        d.packed = __shfl_sync(0xffffffffu, mine.packed, i - base);
        return d;
    }
};

__device__ __forceinline__ BlockDesc load_first_chunk(const BlockDesc* blocks, int first, int count, int lane) {
    BlockDesc d{0, 0};
    if (lane < count) d = blocks[first + lane];
    return d;
}

// Hands a fully read TMEM accumulator buffer back to the MMA warps (one arrival per warp).
__device__ __forceinline__ void release_accumulator(uint64_t* acc_empty, int lane) {
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(acc_empty);
}

// Shared-memory matrix descriptor of a 16-bit operand made of 64x64 tiles, each stored as 64
// rows of 128 bytes with the 128-byte swizzle.  For a K-major operand a row is one M/N index
// and the 8-row groups (1024 B apart, the stride byte offset) run along M/N, so tiles placed
// back to back continue the operand to 128, 192, 256 rows.  For an MN-major operand a row is
// one K index, the 8-row groups run along K, and the leading byte offset (8192 B) is the
// distance between tiles holding consecutive 64-wide ranges of M/N.
// Bits: start address >> 4 in [0,14), LBO >> 4 in [16,30), SBO >> 4 in [32,46), descriptor
// version 1 in [46,48), layout type SWIZZLE_128B = 2 in [61,64).
__device__ __forceinline__ uint64_t make_tile_desc(uint32_t smem_addr, bool mn_major) {
    uint64_t d = (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
    d |= (uint64_t)(mn_major ? (kTileBytes >> 4) : 1) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// 4x4 transpose of 32-bit words among the four threads of a quad (lanes 4i .. 4i+3): on entry
// thread q holds m[u] = element (u, q); on return it holds m[j] = element (q, j).
__device__ __forceinline__ void quad_transpose(uint32_t (&m)[4], int q) {
    const bool b0 = (q & 1) != 0, b1 = (q & 2) != 0;
    uint32_t s0 = b0 ? m[0] : m[1], s1 = b0 ? m[2] : m[3];
    s0 = __shfl_xor_sync(0xffffffffu, s0, 1);
    s1 = __shfl_xor_sync(0xffffffffu, s1, 1);
    if (b0) { m[0] = s0; m[2] = s1; } else { m[1] = s0; m[3] = s1; }
    s0 = b1 ? m[0] : m[2];
    s1 = b1 ? m[1] : m[3];
    s0 = __shfl_xor_sync(0xffffffffu, s0, 2);
    s1 = __shfl_xor_sync(0xffffffffu, s1, 2);
    if (b1) { m[0] = s0; m[1] = s1; } else { m[2] = s0; m[3] = s1; }
}

// ------------------------------------------------------------------ host side
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* sym = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(sym);
    });
    return fn;
}

// Host work that need not be repeated per call.  Encoding a tensor map goes through the driver, and a
// launch-bound caller (a few microseconds of kernel work per call) issues the same maps over and over:
// a map depends only on the base address, the shape and the element type, so the last maps are kept
// (a small direct-mapped table under a mutex; a hit copies 128 bytes).  One table per kernel file.
struct MapKey {
    const void* base;
    int64_t batches, rows, cols;
    int dtype, variant;                 // variant: box height / operand majorness, whatever else the encoder depends on
    bool operator==(const MapKey& o) const {
        return base == o.base && batches == o.batches && rows == o.rows && cols == o.cols && dtype == o.dtype &&
               variant == o.variant;
    }
};
template <class Encode>
bool cached_map(CUtensorMap* map, const MapKey& key, Encode encode) {
    constexpr int kSlots = 64;
    struct Slot { MapKey key; CUtensorMap map; bool used; };
    static Slot slots[kSlots] = {};
    static std::mutex mutex;
    const uintptr_t h = reinterpret_cast<uintptr_t>(key.base) >> 8;
    const int slot = (int)((h ^ (h >> 7) ^ (uintptr_t)(key.rows * 31 + key.cols * 7 + key.variant)) % kSlots);
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (slots[slot].used && slots[slot].key == key) { *map = slots[slot].map; return true; }
    }
    // The driver call needs the device's primary context bound to the calling thread: cudaSetDevice on
    // the current device does that (a thread that has only launched kernels so far may not have it).
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaSetDevice(dev) != cudaSuccess) { cudaGetLastError(); return false; }
    if (!encode(map)) return false;
    std::lock_guard<std::mutex> lock(mutex);
    slots[slot].key = key; slots[slot].map = *map; slots[slot].used = true;
    return true;
}

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel and device instead of once per call.  The
// attribute is a maximum: it is only ever raised (a kernel launched with different sizes, e.g. per head
// dimension, must not have it lowered by the smaller configuration).
inline bool ensure_dynamic_smem(const void* kernel, int bytes) {
    constexpr int kEntries = 64;
    struct Entry { const void* kernel; int dev, bytes; };
    static Entry done[kEntries] = {};
    static int count = 0;
    static std::mutex mutex;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return false; }
    std::lock_guard<std::mutex> lock(mutex);
    Entry* entry = nullptr;
    for (int i = 0; i < count; ++i)
        if (done[i].kernel == kernel && done[i].dev == dev) { entry = &done[i]; break; }
    if (entry && entry->bytes >= bytes) return true;
    if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    if (entry) entry->bytes = bytes;
    else if (count < kEntries) done[count++] = Entry{kernel, dev, bytes};
    return true;
}

// 3-D tensor map over a row-major [batches, rows, cols] 16-bit tensor with a 64x64x1 box and the
// 128-byte swizzle.  Out-of-range parts of a box read as zero and are not written.
bool encode_map(CUtensorMap* map, int dtype, const void* base, int64_t batches, int64_t rows, int64_t cols,
                int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * (cuuint64_t)cols * 2};
    const cuuint32_t box[3] = {kTile, (cuuint32_t)box_rows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUtensorMapDataType type = dtype == BSA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                             : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult res = fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS)
        std::fprintf(stderr, "bsa: cuTensorMapEncodeTiled failed with CUresult %d (base %p, dims %lld x %lld x %lld)\n",
                     (int)res, base, (long long)batches, (long long)rows, (long long)cols);
    return res == CUDA_SUCCESS;
}

bool make_map(CUtensorMap* map, int dtype, const void* base, int64_t batches, int64_t rows, int64_t cols,
              int box_rows = kTile) {
    return cached_map(map, MapKey{base, batches, rows, cols, dtype, box_rows},
                      [&](CUtensorMap* m) { return encode_map(m, dtype, base, batches, rows, cols, box_rows); });
}

// Number of SMs of the current device (asked once per device).
int sm_count() {
    static int cached[64] = {};
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64 && cached[dev] > 0) return cached[dev];
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (dev >= 0 && dev < 64) cached[dev] = sms;
    return sms;
}

}  // namespace
}  // namespace bsa
