// tcgen05 / TMEM engine of the block-sparse matmul (sm_100a only).
//
// Replaces the CUDA-core kernels sparse_smm_{sdd,dsd,dds}_32x32x32_kernel
// (reference sparse/native/sparse_smm_gpu.cu:22-267) and the unfinished
// half-precision sparse_hmm_sdd_32x32x32_kernel (sparse_hmm_gpu.cu:26-142,
// fp16 accumulation) for 16-bit inputs with block 64: fp16 / bf16 operands,
// fp32 accumulation in tensor memory.
//
// Structure.  Everything is expressed in 64x64 16-bit tiles (8 KB, rows of
// 128 bytes, 128-byte swizzle), the one shape that is both a TMA box of a
// dense operand, a whole sparse block, and a legal UMMA operand in either
// major-ness (so trans_a / trans_b only flip descriptor bits and swap two TMA
// coordinates).  A persistent CTA per SM walks work items; an item is one
// group of the layout (a block row or block column) of one batch entry:
//   sdd  item = block row r.  Its blocks are taken two at a time; a pair is
//        one accumulation: A = rows r of op(A), B0|B1 = rows c0, c1 of op(B)^T
//        (adjacent in shared memory, one N = 128 operand), K-steps over the
//        dense inner size.  Output: the pair's two blocks.
//   dsd  item = group m (and a 128-wide slice of N).  One accumulation over
//        the group's blocks: A = the sparse block, B0|B1 = the k-block rows of
//        op(B).  Output: C[m*64.., slice].
//   dds  item = group n (and a 64-tall slice of M).  One accumulation over the
//        group's blocks: A = op(A)[slice, k-block], B = the sparse block.
//        Output: C[slice, n*64..].
// Warp roles (10 warps):
//   warp 0      TMA producer of the A tiles (lane 0 issues; arms the stage barrier)
//   warp 1      TMA producer of the B tiles
//   warps 2-5   tcgen05.mma issuers.  A single thread issues one MMA per ~150
//               cycles whatever its shape, which is slower than these small
//               MMAs execute, so the K = 64 of a stage is split over 4 (N = 64)
//               or 2 (N = 128) issuers.  Each issuer owns a private partial
//               accumulator in TMEM, so no ordering between issuers is needed.
//   warps 6-9   epilogue: tcgen05.ld of the partials, sum, convert, swizzled
//               shared tile, TMA store (up to 6 stores in flight).
// Shared-memory stages and the two TMEM accumulator buffers are handed over
// with mbarriers.  Group offsets and block descriptors are prefetched one to
// two items ahead so no role waits on a dependent global load per step.
// Every mbarrier wait is bounded: on a time-out the CTA records
// BSA_ERR_DEVICE_TIMEOUT in the workspace word, stops issuing work, drains
// what it has in flight, frees its TMEM and returns.
#include <cstdio>
#include <mutex>

#include "bsa_common.cuh"

namespace bsa {
namespace {

constexpr int kTile = 64;                       // tile edge in elements
constexpr int kTileBytes = kTile * kTile * 2;   // 8 KB
constexpr int kMaxStages = 9;
constexpr int kStageBytesTotal = 18 * kTileBytes;   // 144 KB of operand stages (9 x 2 or 6 x 3 tiles)
constexpr int kOutBufs = 6;                     // epilogue staging tiles (TMA stores in flight)
constexpr int kAccCols = 256;                   // TMEM columns per accumulator buffer (all partials)
constexpr int kTmemCols = 2 * kAccCols;
constexpr int kMmaWarps = 4;
constexpr int kFirstMmaWarp = 2;
constexpr int kFirstEpilogueWarp = kFirstMmaWarp + kMmaWarps;
constexpr int kThreads = (kFirstEpilogueWarp + 4) * 32;
constexpr int kEpilogueThreads = 128;
constexpr unsigned long long kWaitLimitNs = 2000000000ull;   // 2 s

// Optional role timing (compile with -DBSA_TC_TIMING): CTA 0 adds the cycles each role spent in
// its waits to 64-bit counters at byte offset 64 of the workspace.
#ifdef BSA_TC_TIMING
#define TC_TIME_DECL(name) long long name = 0
#define TC_TIMED(name, stmt) { const long long tic_ = clock64(); stmt; name += clock64() - tic_; }
#define TC_TIME_OUT(slot, name) if (blockIdx.x == 0) atomicAdd(reinterpret_cast<unsigned long long*>(p.status) + 8 + (slot), (unsigned long long)(name))
#else
#define TC_TIME_DECL(name)
#define TC_TIMED(name, stmt) { stmt; }
#define TC_TIME_OUT(slot, name)
#endif

struct __align__(8) Barriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[2];
    uint64_t acc_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
};
constexpr int kSmemBytes = 1024 /* alignment slack */ + kStageBytesTotal + kOutBufs * kTileBytes + (int)sizeof(Barriers);

struct TcParams {
    const BlockDesc* blocks;
    const int32_t* table;
    uint32_t* status;        // workspace word
    int nnz, groups, batches;
    int size_m, size_n, size_k;
    int mode, trans_a, trans_b;
    int chunks;              // dsd: 128-wide slices of N; dds: 64-tall slices of M; sdd: 1
    int items;
    int slots;               // operand tiles per stage: 2 (A + B) or 3 (A + B0 + B1)
    int stages;              // pipeline depth
    int issuers;             // MMA issuing warps in use: 4 (N = 64) or 2 (N up to 128)
    uint32_t idesc64, idesc128;   // instruction descriptors for N = 64 and N = 128
};

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
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait.  Returns false if the wait was given up (time-out here, or an
// abort raised by another role of this CTA).
__device__ __noinline__ bool mbar_wait_slow(uint64_t* bar, uint32_t parity, Barriers* bars, uint32_t* status) {
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 256; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*(volatile int*)&bars->abort_flag) return false;
        if (global_ns() - t0 > kWaitLimitNs) {
            *(volatile int*)&bars->abort_flag = 1;
            atomicExch(status, (uint32_t)BSA_ERR_DEVICE_TIMEOUT);
            return false;
        }
    }
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, Barriers* bars, uint32_t* status) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, bars, status);
}

__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(dst)), "l"(map), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, const void* src, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                 ::"l"(map), "r"(smem_u32(src)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
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
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// AND-vote over the 128 epilogue threads (named barrier 2), so that giving up on a wait is a
// decision all of them take together and none is left alone at a later named barrier.
__device__ __forceinline__ bool epilogue_all(bool v) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.and.pred p, 2, %2, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(r) : "r"((uint32_t)v), "n"(kEpilogueThreads) : "memory");
    return r != 0;
}

// Shared-memory matrix descriptor of a 16-bit operand made of 64x64 tiles, each stored as 64
// rows of 128 bytes with the 128-byte swizzle.  For a K-major operand a row is one M/N index
// and the 8-row groups (1024 B apart, the stride byte offset) run along M/N, so a second tile
// placed right behind the first continues the operand to 128 rows.  For an MN-major operand a
// row is one K index, the 8-row groups run along K, and the leading byte offset (8192 B) is
// the distance to the tile holding M/N indices 64-127.
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

// Iterates the work items of one CTA (item = blockIdx.x + n * gridDim.x) and keeps the group
// offset-table words of the next two items in flight, so that by the time an item becomes
// current its words have arrived and no role stalls on a dependent global load per item.
struct Cursor {
    int item, stride, items, chunks, per_z;
    const int32_t* table;
    int z, g, chunk, first, count;      // current item: batch entry, group, slice, block range
    int n1_a, n1_b, n2_a, n2_b;         // table[g], table[g + 1] of the next item and the one after

    __device__ __forceinline__ void load_words(int it, int& a, int& b) const {
        a = 0; b = 0;
        if (it < items) { const int gg = (it % per_z) / chunks; a = table[gg]; b = table[gg + 1]; }
    }
    __device__ __forceinline__ void set_current(int a, int b) {
        z = item / per_z;
        const int rem = item - z * per_z;
        g = rem / chunks;
        chunk = rem - g * chunks;
        first = a;
        count = b - a;
    }
    __device__ __forceinline__ void init(const TcParams& p) {
        item = (int)blockIdx.x; stride = (int)gridDim.x; items = p.items;
        chunks = p.chunks; per_z = p.groups * p.chunks; table = p.table;
        z = g = chunk = first = count = 0;
        int a, b;
        load_words(item, a, b);
        load_words(item + stride, n1_a, n1_b);
        load_words(item + 2 * stride, n2_a, n2_b);
        if (item < items) set_current(a, b);
    }
    __device__ __forceinline__ bool valid() const { return item < items; }
    __device__ __forceinline__ bool has_next() const { return item + stride < items; }
    __device__ __forceinline__ int next_first() const { return n1_a; }
    __device__ __forceinline__ int next_count() const { return n1_b - n1_a; }
    __device__ __forceinline__ void advance() {
        item += stride;
        const int a = n1_a, b = n1_b;
        n1_a = n2_a; n1_b = n2_b;
        load_words(item + 2 * stride, n2_a, n2_b);
        if (item < items) set_current(a, b);
    }
};

// A warp-wide window of 32 block descriptors of the current group: lane l holds descriptor
// base + l, the following 32 are already being loaded.  get() must be called by all 32 lanes
// with the same, non-decreasing index.
struct DescWindow {
    BlockDesc mine, ahead;
    __device__ __forceinline__ void begin(const BlockDesc& first_chunk) { mine = first_chunk; ahead = BlockDesc{0, 0}; }
    __device__ __forceinline__ BlockDesc get(const BlockDesc* blocks, int first, int count, int i, int lane) {
        if ((i & 31) == 0) {
            if (i > 0) mine = ahead;
            if (i + 32 + lane < count) ahead = blocks[first + i + 32 + lane];
        }
        BlockDesc d;
        d.idx = __shfl_sync(0xffffffffu, mine.idx, i & 31);
        d.packed = __shfl_sync(0xffffffffu, mine.packed, i & 31);
        return d;
    }
};

__device__ __forceinline__ BlockDesc load_first_chunk(const BlockDesc* blocks, int first, int count, int lane) {
    BlockDesc d{0, 0};
    if (lane < count) d = blocks[first + lane];
    return d;
}

// Number of accumulations (each ends in an epilogue) and K-steps per accumulation of an item.
__device__ __forceinline__ void item_shape(const TcParams& p, int count, int& flushes, int& ksteps) {
    if (p.mode == BSA_MODE_SDD) {
        flushes = (count + 1) >> 1;
        ksteps = (p.size_k + kTile - 1) / kTile;
    } else {
        flushes = 1;
        ksteps = count;
    }
}

// Number of B tiles (64 output columns each) of one accumulation; there is always one A tile.
__device__ __forceinline__ int b_tiles(const TcParams& p, int count, int chunk, int flush) {
    if (p.mode == BSA_MODE_SDD) return min(2, count - 2 * flush);
    if (p.mode == BSA_MODE_DSD) return min(2, (p.size_n - chunk * 2 * kTile + kTile - 1) / kTile);
    return 1;
}

__global__ void __launch_bounds__(kThreads, 1)
tc_matmul_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;                                   // p.stages * p.slots tiles
    uint8_t* out_base = smem + kStageBytesTotal;                  // kOutBufs tiles
    Barriers* bars = reinterpret_cast<Barriers*>(out_base + kOutBufs * kTileBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stage_bytes = p.slots * kTileBytes;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], p.issuers); }
        for (int s = 0; s < 2; ++s) { mbar_init(&bars->acc_full[s], p.issuers); mbar_init(&bars->acc_empty[s], 4); }
        mbar_init(&bars->drain, p.issuers);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (warp == kFirstMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"((uint32_t)kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;

    const bool a_mn_major = p.trans_a != 0;      // op(A) tile arrives with M contiguous
    const bool b_mn_major = p.trans_b == 0;      // op(B) tile arrives with N contiguous

    if (warp < 2) {
        // ------------------------------------------------------------ TMA producers
        // Warp 0 loads the A tile of every stage and arms its barrier with the byte count of
        // the whole stage; warp 1 loads the B tile(s).  All 32 lanes walk the items together
        // (descriptor windows are warp-wide); lane 0 waits and issues.
        const bool load_a = warp == 0;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        TC_TIME_DECL(t_wait); TC_TIME_DECL(t_issue); TC_TIME_DECL(t_all);
#ifdef BSA_TC_TIMING
        const long long t_begin = clock64();
#endif
        Cursor cur;
        cur.init(p);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            int flushes, ksteps;
            item_shape(p, cur.count, flushes, ksteps);
            DescWindow win;
            win.begin(pre);
            for (int f = 0; ok && f < flushes; ++f) {
                const int nb = b_tiles(p, cur.count, cur.chunk, f);
                BlockDesc d0{0, 0}, d1{0, 0};
                if (p.mode == BSA_MODE_SDD) {
                    d0 = win.get(p.blocks, cur.first, cur.count, 2 * f, lane);
                    d1 = win.get(p.blocks, cur.first, cur.count, 2 * f + 1, lane);
                }
                for (int k = 0; ok && k < ksteps; ++k) {
                    BlockDesc d{0, 0};
                    if (p.mode != BSA_MODE_SDD) d = win.get(p.blocks, cur.first, cur.count, k, lane);
                    if (lane == 0) {
                        TC_TIMED(t_wait, ok = mbar_wait(&bars->empty[stage], phase ^ 1, bars, p.status));
#ifdef BSA_TC_TIMING
                        const long long tic_issue = clock64();
#endif
                        if (ok) {
                            uint8_t* slot = stage_base + stage * stage_bytes;
                            uint64_t* full = &bars->full[stage];
                            if (load_a) mbar_expect_tx(full, (uint32_t)((1 + nb) * kTileBytes));
                            if (p.mode == BSA_MODE_SDD) {
                                const int k0 = k * kTile, m0 = cur.g * kTile;
                                if (load_a) {
                                    if (a_mn_major) tma_load_3d(slot, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot, &map_a, full, k0, m0, cur.z);
                                } else {
                                    for (int j = 0; j < nb; ++j) {
                                        const int n0 = (j == 0 ? d0.col() : d1.col()) * kTile;
                                        if (b_mn_major) tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, n0, k0, cur.z);
                                        else            tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, k0, n0, cur.z);
                                    }
                                }
                            } else if (p.mode == BSA_MODE_DSD) {
                                const int k0 = (p.trans_a ? d.row() : d.col()) * kTile;
                                if (load_a) {
                                    tma_load_3d(slot, &map_a, full, 0, d.idx * kTile, cur.z);
                                } else {
                                    for (int j = 0; j < nb; ++j) {
                                        const int n0 = (cur.chunk * 2 + j) * kTile;
                                        if (b_mn_major) tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, n0, k0, cur.z);
                                        else            tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, k0, n0, cur.z);
                                    }
                                }
                            } else {
                                const int k0 = (p.trans_b ? d.col() : d.row()) * kTile;
                                if (load_a) {
                                    const int m0 = cur.chunk * kTile;
                                    if (a_mn_major) tma_load_3d(slot, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot, &map_a, full, k0, m0, cur.z);
                                } else {
                                    tma_load_3d(slot + kTileBytes, &map_b, full, 0, d.idx * kTile, cur.z);
                                }
                            }
                        }
#ifdef BSA_TC_TIMING
                        t_issue += clock64() - tic_issue;
#endif
                    }
                    ok = __shfl_sync(0xffffffffu, (int)ok, 0) != 0;
                    if (++stage == p.stages) { stage = 0; phase ^= 1; }
                }
            }
            pre = pre_next;
            cur.advance();
        }
#ifdef BSA_TC_TIMING
        t_all = clock64() - t_begin;
        if (lane == 0) { TC_TIME_OUT(warp * 3 + 0, t_all); TC_TIME_OUT(warp * 3 + 1, t_wait); TC_TIME_OUT(warp * 3 + 2, t_issue); }
#endif
        if (!ok && lane == 0) {
            // Give copies that were issued a bounded chance to land before the CTA exits.
            const unsigned long long t0 = global_ns();
            for (int s = 0; s < p.stages; ++s)
                while (!mbar_try_wait(&bars->full[s], 0) && !mbar_try_wait(&bars->full[s], 1) &&
                       global_ns() - t0 < kWaitLimitNs / 4) {}
        }
        __syncwarp();
    } else if (warp < kFirstEpilogueWarp) {
        // ------------------------------------------------------------ MMA issuers
        const int w = warp - kFirstMmaWarp;
        if (lane == 0 && w < p.issuers) {
            int stage = 0, acc = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t a_kstep = a_mn_major ? 2048u >> 4 : 32u >> 4;   // descriptor advance per K = 16
            const uint32_t b_kstep = b_mn_major ? 2048u >> 4 : 32u >> 4;
            const int kk_per_issuer = (kTile / 16) / p.issuers;            // 1 or 2 K = 16 slices of each stage
            // private partial accumulator of this issuer inside an accumulator buffer
            const uint32_t part_col = (uint32_t)(w * (kAccCols / p.issuers));
            TC_TIME_DECL(t_full); TC_TIME_DECL(t_acc); TC_TIME_DECL(t_all);
#ifdef BSA_TC_TIMING
            const long long t_begin = clock64();
#endif
            Cursor cur;
            cur.init(p);
            for (; ok && cur.valid(); cur.advance()) {
                int flushes, ksteps;
                item_shape(p, cur.count, flushes, ksteps);
                if (ksteps == 0) continue;          // empty group: the epilogue writes zeros on its own
                for (int f = 0; ok && f < flushes; ++f) {
                    const int nb = b_tiles(p, cur.count, cur.chunk, f);
                    const uint32_t idesc = nb == 2 ? p.idesc128 : p.idesc64;
                    TC_TIMED(t_acc, ok = mbar_wait(&bars->acc_empty[acc], acc_phase ^ 1, bars, p.status));
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + (uint32_t)(acc * kAccCols) + part_col;
                    for (int k = 0; k < ksteps; ++k) {
                        TC_TIMED(t_full, ok = mbar_wait(&bars->full[stage], phase, bars, p.status));
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t slot = smem_u32(stage_base + stage * stage_bytes);
                        const uint64_t da = make_tile_desc(slot, a_mn_major);
                        const uint64_t db = make_tile_desc(slot + kTileBytes, b_mn_major);
                        for (int s = 0; s < kk_per_issuer; ++s) {
                            const int kk = w + s * p.issuers;
                            tc_mma_f16(d, da + (uint64_t)(kk * a_kstep), db + (uint64_t)(kk * b_kstep), idesc,
                                       (k > 0 || s > 0) ? 1u : 0u);
                        }
                        tc_commit(&bars->empty[stage]);      // this issuer's reads of the stage are done
                        if (++stage == p.stages) { stage = 0; phase ^= 1; }
                    }
                    if (!ok) break;
                    tc_commit(&bars->acc_full[acc]);         // this issuer's partial is complete
                    if (++acc == 2) { acc = 0; acc_phase ^= 1; }
                }
            }
            // All MMAs issued by this thread must have retired before TMEM is freed.
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, bars, p.status);
#ifdef BSA_TC_TIMING
            t_all = clock64() - t_begin;
            if (w == 0) { TC_TIME_OUT(6, t_all); TC_TIME_OUT(7, t_full); TC_TIME_OUT(8, t_acc); }
#endif
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue
        const int quad = warp & 3;                   // TMEM sub-partition this warp may read
        const int et = threadIdx.x - kFirstEpilogueWarp * 32;   // 0..127 among the epilogue threads
        const int row = quad * 16 + lane;            // accumulator row held by this lane (lanes 0-15 only)
        const bool row_lane = lane < 16;
        const bool is_sdd = p.mode == BSA_MODE_SDD;
        const bool bf16_out = (p.idesc64 & (1u << 7)) != 0;
        const int part_stride = kAccCols / p.issuers;
        int acc = 0, out_buf = 0;
        uint32_t acc_phase = 0;
        bool ok = true;
        TC_TIME_DECL(t_accf); TC_TIME_DECL(t_ld); TC_TIME_DECL(t_store); TC_TIME_DECL(t_write); TC_TIME_DECL(t_all);
#ifdef BSA_TC_TIMING
        const long long t_begin = clock64();
#endif
        Cursor cur;
        cur.init(p);
        BlockDesc pre{0, 0};
        if (is_sdd && cur.valid()) pre = load_first_chunk(p.blocks, cur.first, cur.count, lane);
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (is_sdd && cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            int flushes, ksteps;
            item_shape(p, cur.count, flushes, ksteps);
            DescWindow win;
            win.begin(pre);
            for (int f = 0; ok && f < flushes; ++f) {
                const int tiles = b_tiles(p, cur.count, cur.chunk, f);
                const bool have_acc = ksteps > 0;
                if (have_acc) {
                    TC_TIMED(t_accf, ok = epilogue_all(mbar_wait(&bars->acc_full[acc], acc_phase, bars, p.status)));
                    if (!ok) break;
                    tc_fence_after();
                }
                for (int t = 0; t < tiles; ++t) {
                    int out_idx = 0;
                    if (is_sdd) out_idx = win.get(p.blocks, cur.first, cur.count, 2 * f + t, lane).idx;
                    float v[kTile];
#pragma unroll
                    for (int c = 0; c < kTile; ++c) v[c] = 0.f;
#ifdef BSA_TC_TIMING
                    const long long tic_ld = clock64();
#endif
                    if (have_acc) {
                        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16)
                                               + (uint32_t)(acc * kAccCols + t * kTile);
                        for (int part = 0; part < p.issuers; ++part) {
#pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t r[32];
                                tc_ld_32x32b_x32(taddr + (uint32_t)(part * part_stride + h * 32), r);
                                tc_wait_ld();
#pragma unroll
                                for (int c = 0; c < 32; ++c) v[h * 32 + c] += __uint_as_float(r[c]);
                            }
                        }
                    }
                    if (have_acc && t == tiles - 1) {
                        // accumulator fully read: hand the TMEM buffer back to the MMA warps
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&bars->acc_empty[acc]);
                    }
#ifdef BSA_TC_TIMING
                    t_ld += clock64() - tic_ld;
                    const long long tic_st = clock64();
#endif
                    // staging tile `out_buf` was last read by the store issued kOutBufs tiles ago
                    if (et == 0) tma_store_wait_read<kOutBufs - 1>();
                    asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
#ifdef BSA_TC_TIMING
                    t_store += clock64() - tic_st;
                    const long long tic_wr = clock64();
#endif
                    uint8_t* out = out_base + out_buf * kTileBytes;
                    if (row_lane) {
#pragma unroll
                        for (int c = 0; c < 8; ++c) {            // 16-byte chunk = 8 columns
                            uint32_t packed[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float lo = v[c * 8 + e * 2], hi = v[c * 8 + e * 2 + 1];
                                if (bf16_out) {
                                    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                                    packed[e] = *reinterpret_cast<uint32_t*>(&h);
                                } else {
                                    __half2 h = __floats2half2_rn(lo, hi);
                                    packed[e] = *reinterpret_cast<uint32_t*>(&h);
                                }
                            }
                            *reinterpret_cast<uint4*>(out + row * 128 + ((c ^ (row & 7)) << 4)) =
                                make_uint4(packed[0], packed[1], packed[2], packed[3]);
                        }
                    }
                    fence_async_shared();
                    asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueThreads) : "memory");
                    if (et == 0) {
                        if (is_sdd) {
                            tma_store_3d(&map_c, out, 0, out_idx * kTile, cur.z);
                        } else if (p.mode == BSA_MODE_DSD) {
                            tma_store_3d(&map_c, out, (cur.chunk * 2 + t) * kTile, cur.g * kTile, cur.z);
                        } else {
                            tma_store_3d(&map_c, out, cur.g * kTile, cur.chunk * kTile, cur.z);
                        }
                        tma_store_commit();
                    }
                    if (++out_buf == kOutBufs) out_buf = 0;
#ifdef BSA_TC_TIMING
                    t_write += clock64() - tic_wr;
#endif
                }
                if (have_acc && ++acc == 2) { acc = 0; acc_phase ^= 1; }
            }
            pre = pre_next;
            cur.advance();
        }
        if (et == 0) tma_store_wait_all();
#ifdef BSA_TC_TIMING
        t_all = clock64() - t_begin;
        if (et == 0) { TC_TIME_OUT(9, t_all); TC_TIME_OUT(10, t_accf); TC_TIME_OUT(11, t_ld); TC_TIME_OUT(12, t_store); TC_TIME_OUT(13, t_write); }
#endif
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == kFirstMmaWarp) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
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

// 3-D tensor map over a row-major [batches, rows, cols] 16-bit tensor with a 64x64x1 box and the
// 128-byte swizzle.  Out-of-range parts of a box read as zero and are not written.
bool make_map(CUtensorMap* map, int dtype, const void* base, int64_t batches, int64_t rows, int64_t cols) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * 2, (cuuint64_t)rows * (cuuint64_t)cols * 2};
    const cuuint32_t box[3] = {kTile, kTile, 1};
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

int sm_count() {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    return sms;
}

bool dense_dim_ok(int64_t v) { return v >= kTile && v % 8 == 0 && v < ((int64_t)1 << 31); }

int64_t slices_of(const MatmulArgs& g) {
    if (g.mode == BSA_MODE_DSD) return (g.size_n + 2 * kTile - 1) / (2 * kTile);
    if (g.mode == BSA_MODE_DDS) return (g.size_m + kTile - 1) / kTile;
    return 1;
}

}  // namespace

bool tc_supports(const MatmulArgs& g) {
    if (g.dtype != BSA_DTYPE_F16 && g.dtype != BSA_DTYPE_BF16) return false;
    if (g.block != kTile) return false;
    if (g.nnz <= 0 || g.nnz * kTile >= ((int64_t)1 << 31) || g.batches > 65535) return false;
    if (!dense_dim_ok(g.size_m) || !dense_dim_ok(g.size_n) || !dense_dim_ok(g.size_k)) return false;
    // work items are indexed with 32-bit integers
    if (g.batches * g.groups * slices_of(g) >= ((int64_t)1 << 30)) return false;
    return true;
}

int matmul_tc(const MatmulArgs& g) {
    // The opt-in shared-memory size is a per-device attribute, so it is set on every call (a cheap
    // host-side update).  Doing it first also binds the device's primary context to the calling
    // thread: cuTensorMapEncodeTiled below is a driver call and fails with "invalid context" on a
    // thread (e.g. an autograd worker) that has not made a runtime call needing the context yet.
    if (cudaFuncSetAttribute(tc_matmul_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes) != cudaSuccess) {
        cudaGetLastError();
        return BSA_ERR_LAUNCH;
    }
    if (cudaFree(nullptr) != cudaSuccess) { cudaGetLastError(); return BSA_ERR_LAUNCH; }
    CUtensorMap map_a, map_b, map_c;
    const int64_t sparse_rows = g.nnz * kTile;
    bool ok = true;
    // stored shapes: a dense operand is [rows, cols] = op^-1 of its logical shape
    if (g.mode == BSA_MODE_SDD) {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n);
        ok &= make_map(&map_c, g.dtype, g.c, g.batches, sparse_rows, kTile);
    } else if (g.mode == BSA_MODE_DSD) {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, sparse_rows, kTile);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n);
        ok &= make_map(&map_c, g.dtype, g.c, g.batches, g.size_m, g.size_n);
    } else {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, sparse_rows, kTile);
        ok &= make_map(&map_c, g.dtype, g.c, g.batches, g.size_m, g.size_n);
    }
    if (!ok) return BSA_ERR_DRIVER;

    TcParams p{};
    p.blocks = g.blocks; p.table = g.table; p.status = g.workspace;
    p.nnz = (int)g.nnz; p.groups = (int)g.groups; p.batches = (int)g.batches;
    p.size_m = (int)g.size_m; p.size_n = (int)g.size_n; p.size_k = (int)g.size_k;
    p.mode = g.mode; p.trans_a = g.trans_a; p.trans_b = g.trans_b;
    p.chunks = (int)slices_of(g);
    p.items = (int)(g.batches * g.groups * p.chunks);
    // two B tiles per stage (N = 128, two issuers) for sdd pairs and for dsd with more than 64 columns
    const bool wide = g.mode == BSA_MODE_SDD || (g.mode == BSA_MODE_DSD && g.size_n > kTile);
    p.slots = wide ? 3 : 2;
    p.stages = kStageBytesTotal / (p.slots * kTileBytes);
    p.issuers = wide ? 2 : 4;
    // instruction descriptor: fp32 accumulate, fp16 / bf16 operands, M = 64, N = 64 or 128
    const uint32_t fmt = g.dtype == BSA_DTYPE_BF16 ? 1u : 0u;
    const uint32_t common = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g.trans_a ? 1u : 0u) << 15)
                            | ((g.trans_b ? 0u : 1u) << 16) | ((uint32_t)(kTile >> 4) << 24);
    p.idesc64 = common | ((uint32_t)(kTile >> 3) << 17);
    p.idesc128 = common | ((uint32_t)(2 * kTile >> 3) << 17);

    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    const unsigned grid = (unsigned)(p.items < sms ? p.items : sms);
    tc_matmul_kernel<<<grid, kThreads, kSmemBytes, g.stream>>>(map_a, map_b, map_c, p);
    return launch_status();
}

}  // namespace bsa
