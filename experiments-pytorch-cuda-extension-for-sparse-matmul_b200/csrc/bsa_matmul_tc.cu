// tcgen05 / TMEM engine of the block-sparse matmul (sm_100a only).
//
// Replaces the CUDA-core kernels sparse_smm_{sdd,dsd,dds}_32x32x32_kernel
// (reference sparse/native/sparse_smm_gpu.cu:22-267) and the unfinished
// half-precision sparse_hmm_sdd_32x32x32_kernel (sparse_hmm_gpu.cu:26-142,
// fp16 accumulation) for 16-bit inputs with block 64 or 128: fp16 / bf16
// operands, fp32 accumulation in tensor memory.  (Block 128 is walked as 2 x 2
// tiles of 64 x 64 per block, see tile_desc.)
//
// Structure.  Everything is expressed in 64x64 16-bit tiles (8 KB, rows of
// 128 bytes, 128-byte swizzle), the one shape that is both a TMA box of a
// dense operand, a whole sparse block, and a legal UMMA operand in either
// major-ness (so trans_a / trans_b only flip descriptor bits and swap two TMA
// coordinates).  A persistent CTA per SM walks work items; an item is one
// group of the layout (a block row or block column) of one batch entry:
//   sdd  item = block row r.  Its blocks are taken two at a time; such a
//        pair is one accumulation: A = rows r of op(A), B0, B1 = rows c0, c1 of
//        op(B)^T placed back to back in shared memory (one N = 128 operand),
//        K-steps over the dense inner size.  Output: the pair's two blocks.
//   dsd  item = group m (and a 128-wide slice of N).  One accumulation over
//        the group's blocks: A = the sparse block, B0|B1 = the k-block rows of
//        op(B).  Output: C[m*64.., slice].
//   dds  item = group n (and a 64-tall slice of M).  One accumulation over the
//        group's blocks: A = op(A)[slice, k-block], B = the sparse block.
//        Output: C[slice, n*64..].
// Measured on B200: one thread issues a tcgen05.mma or a TMA copy only every
// 150-300 cycles whatever its size, a 64x64x16 MMA executes in ~32 cycles and
// 8 KB boxes need about four issuing threads to saturate the L2 -> SM path.
// Hence the warp roles (16 warps):
//   warps 0-3   TMA producers; K-step n of the CTA belongs to producer n % 4,
//               which loads all of its tiles.
//   warps 4-7   tcgen05.mma issuers.  sdd: two issuers alternate accumulations
//               over four accumulator buffers of 128 TMEM columns.
//               dsd / dds: the K-steps are dealt out to 4 (N = 64) or 2
//               (N = 128) issuers, each with a private partial accumulator, so
//               no ordering between issuers is needed; the epilogue adds them.
//               (Producers and issuers run their loops warp-uniformly and elect
//               a lane only around the TMA / tcgen05 instructions: issuing from
//               a diverged lane costs about twice as much per instruction.)
//   warps 8-15  two epilogue warpgroups taking alternate accumulations.
//               dsd / dds: tcgen05.ld, sum of partials, convert, 256-bit global
//               stores straight from registers (every lane owns a whole 128-byte
//               output row).  sdd: tcgen05.ld in the 16x256b shape, convert,
//               stmatrix into the warp's own 128-byte-swizzled 2 KB slab, one
//               asynchronous 16-row TMA tensor store per warp and tile.
//               No block-level synchronisation: the warps run independently.
// Shared-memory stages and the TMEM accumulator buffers are handed over
// with mbarriers.  Group offsets and block descriptors are prefetched one to
// two items ahead so no role waits on a dependent global load per step.
// Every mbarrier wait is bounded: on a time-out the CTA records
// BSA_ERR_DEVICE_TIMEOUT in the workspace word, stops issuing work, drains
// what it has in flight, frees its TMEM and returns.
#include "bsa_tc_common.cuh"

namespace bsa {
namespace {

constexpr int kMaxStages = 13;
constexpr int kStageTiles = 28;                 // 8 KB tiles of shared memory: stages of 2 or 3 tiles; sdd: 8 x 3 + 4 for output slabs
constexpr int kSddStagingTile0 = 24;            // sdd: tiles 24 .. 27 hold the epilogue warps' output slabs (8 stages x 3 tiles come first)
constexpr int kAccCols = 256;                   // TMEM columns per accumulator buffer (dsd / dds: 2 buffers)
constexpr int kTmemCols = 2 * kAccCols;
constexpr int kSddTiles = 2;                    // sdd: output tiles per accumulation (a buffer of 128 columns)
// sdd is the output-heavy mode: per 8 KB block it writes, the epilogue's chain (accumulator barrier -> TMEM load ->
// convert -> stmatrix -> proxy fence -> TMA store) takes about 1000 cycles, so it needs many accumulations in
// flight.  Four epilogue warpgroups drain eight accumulator buffers: an M = 64 accumulator occupies lanes 0-15 of
// each 32-lane quarter of tensor memory, and a second one fits into lanes 16-31 of the same columns (lane offset
// 16 in the MMA's D address and in the 16-lane tcgen05.ld shape): buffers 0-3 and 4-7 share their columns.
constexpr int kSddGroups = 4;
constexpr int kSddBufs = 2 * kSddGroups;
constexpr int kProducerWarps = 4;
constexpr int kMmaWarps = 4;
constexpr int kFirstMmaWarp = kProducerWarps;
constexpr int kFirstEpilogueWarp = kFirstMmaWarp + kMmaWarps;
constexpr int threads_of(int mode) { return (kFirstEpilogueWarp + 4 * (mode == BSA_MODE_SDD ? kSddGroups : 2)) * 32; }

// sdd: the epilogue warps do not walk the work items (a cursor and a descriptor window in each of their 16
// warps, advanced through every accumulation to use one in four).  The producer that loads an accumulation's
// first K-step posts what they need -- the ranks of the output blocks, their number, the batch entry -- in a
// ring of entries with one mbarrier each; accumulation number F uses entry F & 31 (the producers are at most
// 8 stages + 8 accumulator buffers ahead of the epilogue).
constexpr int kSddEntries = 32;
struct __align__(16) Barriers {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    uint64_t acc_full[kSddBufs];
    uint64_t acc_empty[kSddBufs];
    uint64_t ent_full[kSddEntries];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    int4 ents[kSddEntries];         // (rank of output tile 0, of tile 1, tiles, batch entry); tiles = 0: no more accumulations
};
constexpr int kSmemBytes = 1024 /* alignment slack */ + kStageTiles * kTileBytes + (int)sizeof(Barriers);

struct TcParams {
    const BlockDesc* blocks;
    const int32_t* table;
    uint32_t* status;        // workspace word
    int nnz, groups, batches;
    int size_m, size_n, size_k;
    int mode, trans_a, trans_b;
    int chunks;              // dsd: 128-wide slices of N; dds: 64-tall slices of M; sdd: 1
    int items;
    int nb_max;              // B tiles per stage: sdd 4, dsd 1 or 2, dds 1
    int stages;              // pipeline depth
    int issuers;             // MMA issuing warps in use
    uint32_t idesc;          // instruction descriptor without the N field
    uint16_t* c;             // output (16-bit elements)
    int ldc;                 // elements between output rows
    int c_vec8;              // rows start on 32-byte boundaries: 256-bit stores are legal
    int stride_z, stride_rem;  // gridDim.x divided by the items per batch entry: quotient and remainder
    long long c_elems;       // elements in the output (bounds check of every store)
    int split;               // block 128: every block is walked as 2 x 2 tiles of 64 x 64 (see tile_desc)
    int col_walk;            // the groups are block columns (dsd with trans_a, dds without trans_b)
};

// Block 128.  The kernel keeps working on 64x64 tiles: a real group (block row or column) is two
// virtual groups and a real block two K-steps / output tiles of each, i.e. the kernel sees the
// layout with every block split in 2 x 2, without that layout ever being built.  `groups`, `nnz`
// and `items` of TcParams count virtual units; the cursor reads table[g >> 1] and keeps first /
// count in real blocks.  Virtual descriptor i of virtual group g is real descriptor i >> 1 with
// one half taken from g & 1 and the other from i & 1 (which of row / column depends on the walk);
// its idx is 4 * idx + 2 * row_half + col_half, decoded again by sparse_xy.
__device__ __forceinline__ BlockDesc tile_desc(DescWindow& win, const TcParams& p, const Cursor& cur, int i, int lane) {
    if (!p.split) return win.get(p.blocks, cur.first, cur.count, i, lane);
    const BlockDesc d = win.get(p.blocks, cur.first, cur.count, i >> 1, lane);
    const int from_step = i & 1, from_group = cur.g & 1;
    const int rh = p.col_walk ? from_step : from_group, ch = p.col_walk ? from_group : from_step;
    BlockDesc v;
    v.idx = d.idx * 4 + rh * 2 + ch;
    v.packed = (int32_t)(((uint32_t)(2 * d.row() + rh) << 16) | (uint32_t)(2 * d.col() + ch));
    return v;
}
// TMA coordinates (column, row) of a tile inside the sparse tensor viewed as [nnz * block, block].
__device__ __forceinline__ void sparse_xy(const TcParams& p, int idx, int& x, int& y) {
    if (p.split) { x = (idx & 1) * kTile; y = (idx >> 2) * (2 * kTile) + ((idx >> 1) & 1) * kTile; }
    else         { x = 0; y = idx * kTile; }
}


// Number of accumulations (each ends in an epilogue) and K-steps per accumulation of an item.
template <int MODE>
__device__ __forceinline__ void item_shape(const TcParams& p, int count, int& flushes, int& ksteps) {
    if (MODE == BSA_MODE_SDD) {
        flushes = (count + kSddTiles - 1) / kSddTiles;
        ksteps = (p.size_k + kTile - 1) / kTile;
    } else {
        flushes = 1;
        ksteps = count;
    }
}

// Number of B tiles (64 output columns each) of one accumulation; there is always one A tile.
template <int MODE>
__device__ __forceinline__ int b_tiles(const TcParams& p, int count, int chunk, int flush) {
    if (MODE == BSA_MODE_SDD) return min(kSddTiles, count - kSddTiles * flush);
    if (MODE == BSA_MODE_DSD) return min(2, (p.size_n - chunk * 2 * kTile + kTile - 1) / kTile);
    return 1;
}

// Converts NCOLS fp32 values of one output row to the 16-bit output type and stores the first
// `cols_valid` of them (a multiple of 8) with 256-bit stores where the row alignment allows.
template <int NCOLS>
__device__ __forceinline__ void store_row(uint16_t* dst, const uint32_t (&v)[NCOLS], int cols_valid, bool vec8, bool bf16_out) {
#pragma unroll
    for (int c = 0; c < NCOLS / 16; ++c) {            // 32-byte piece = 16 columns
        uint32_t packed[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float lo = __uint_as_float(v[c * 16 + e * 2]), hi = __uint_as_float(v[c * 16 + e * 2 + 1]);
            if (bf16_out) {
                __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                packed[e] = *reinterpret_cast<uint32_t*>(&h);
            } else {
                __half2 h = __floats2half2_rn(lo, hi);
                packed[e] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        if (vec8 && c * 16 + 16 <= cols_valid) {
            st_global_v8(dst + c * 16, packed);
        } else {
            if (c * 16 + 8 <= cols_valid)
                *reinterpret_cast<uint4*>(dst + c * 16) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            if (c * 16 + 16 <= cols_valid)
                *reinterpret_cast<uint4*>(dst + c * 16 + 8) = make_uint4(packed[4], packed[5], packed[6], packed[7]);
        }
    }
}

// One instantiation per mode keeps each role's loop small (the sixteen warps of a CTA run
// four different code paths through the same instruction caches).
template <int MODE, bool BF16>
__global__ void __launch_bounds__(threads_of(MODE), 1)
tc_matmul_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                 const __grid_constant__ CUtensorMap map_c, const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;                                   // p.stages * (1 + p.nb_max) tiles
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kStageTiles * kTileBytes);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int stage_bytes = (1 + p.nb_max) * kTileBytes;
    constexpr bool is_sdd = MODE == BSA_MODE_SDD;
    constexpr int kBufs = is_sdd ? kSddBufs : 2;        // accumulator buffers in TMEM
    constexpr int kBufShift = is_sdd ? 3 : 1;
    constexpr int kGroups = is_sdd ? kSddGroups : 2;    // epilogue warpgroups
    constexpr int kBufCols = is_sdd ? 128 : kTmemCols / 2;
    // TMEM address (column and lane offset) of accumulator buffer `acc`
    auto acc_addr = [&](int acc) -> uint32_t {
        return is_sdd ? (uint32_t)((acc & 3) * kBufCols) + ((uint32_t)((acc >> 2) * 16) << 16) : (uint32_t)(acc * kBufCols);
    };
    // sdd: one issuer per accumulation; dsd / dds: every issuer reports on every accumulation
    const uint32_t arrivals = is_sdd ? 1u : (uint32_t)p.issuers;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) { mbar_init(&bars->full[s], 1); mbar_init(&bars->empty[s], 1); }
        for (int s = 0; s < kSddBufs; ++s) { mbar_init(&bars->acc_full[s], arrivals); mbar_init(&bars->acc_empty[s], 4); }
        if (is_sdd) for (int s = 0; s < kSddEntries; ++s) mbar_init(&bars->ent_full[s], 1);
        mbar_init(&bars->drain, (uint32_t)p.issuers);
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

    if (warp < kProducerWarps) {
        // ------------------------------------------------------------ TMA producers
        // Every producer walks all items (all 32 lanes together: descriptor windows are
        // warp-wide) and loads the K-steps whose sequence number is its own modulo 4.  Those
        // are steps warp, warp + 4, ... of the CTA, so (the stage count being a multiple of 4)
        // its stage pointer simply advances by 4, whatever the item and accumulation borders.
        int stage = warp, step0 = 0;         // step0: sequence number of the accumulation's first K-step
        int flush_no = 0;                    // sdd: number of the accumulation
        uint32_t phase = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p, p.split);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            int flushes, ksteps;
            item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
            DescWindow win;
            win.begin(p.blocks, cur.first, cur.count, pre, lane);
            for (int f = 0; ok && f < flushes; ++f) {
                const int nb = b_tiles<MODE>(p, cur.count << p.split, cur.chunk, f);
                // The stage count is a multiple of the producer count, so a stage is always
                // filled by the same producer.  This matters: an mbarrier parity wait can only
                // tell the current phase from the one before it, so a thread must take part in
                // every phase of each barrier it ever waits on.
                for (int k = (warp - step0) & (kProducerWarps - 1); ok && k < ksteps; k += kProducerWarps) {
                    {
                        int cols[4] = {0, 0, 0, 0}, ranks[kSddTiles] = {0, 0};
                        BlockDesc d{0, 0};
                        if (is_sdd) {
#pragma unroll
                            for (int j = 0; j < 4; ++j)
                                if (j < nb) {
                                    const BlockDesc dj = tile_desc(win, p, cur, kSddTiles * f + j, lane);
                                    cols[j] = dj.col();
                                    if (j < kSddTiles) ranks[j] = dj.idx;
                                }
                        } else {
                            d = tile_desc(win, p, cur, k, lane);
                        }
                        {
                            // the whole warp waits and computes the copies' operands (warp-uniform
                            // code keeps them in uniform registers); one elected lane issues
                            ok = __all_sync(0xffffffffu, mbar_wait(&bars->empty[stage], phase ^ 1, &bars->abort_flag, p.status)) != 0;
                            if (ok && elect_one()) {
                                uint8_t* slot = stage_base + stage * stage_bytes;
                                uint64_t* full = &bars->full[stage];
                                if (is_sdd && k == 0) {         // the accumulation's entry for the epilogue warps
                                    bars->ents[flush_no & (kSddEntries - 1)] = make_int4(ranks[0], ranks[1], nb, cur.z);
                                    mbar_arrive(&bars->ent_full[flush_no & (kSddEntries - 1)]);
                                }
                                mbar_expect_tx(full, (uint32_t)((1 + nb) * kTileBytes));
                                if (is_sdd) {
                                    const int k0 = k * kTile, m0 = cur.g * kTile;
                                    if (a_mn_major) tma_load_3d(slot, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot, &map_a, full, k0, m0, cur.z);
#pragma unroll
                                    for (int j = 0; j < 4; ++j) {
                                        if (j < nb) {
                                            const int n0 = cols[j] * kTile;
                                            if (b_mn_major) tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, n0, k0, cur.z);
                                            else            tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, k0, n0, cur.z);
                                        }
                                    }
                                } else if (MODE == BSA_MODE_DSD) {
                                    const int k0 = (p.trans_a ? d.row() : d.col()) * kTile;
                                    int sx, sy;
                                    sparse_xy(p, d.idx, sx, sy);
                                    tma_load_3d(slot, &map_a, full, sx, sy, cur.z);
                                    for (int j = 0; j < nb; ++j) {
                                        const int n0 = (cur.chunk * 2 + j) * kTile;
                                        if (b_mn_major) tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, n0, k0, cur.z);
                                        else            tma_load_3d(slot + (1 + j) * kTileBytes, &map_b, full, k0, n0, cur.z);
                                    }
                                } else {
                                    const int k0 = (p.trans_b ? d.col() : d.row()) * kTile;
                                    const int m0 = cur.chunk * kTile;
                                    if (a_mn_major) tma_load_3d(slot, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot, &map_a, full, k0, m0, cur.z);
                                    int sx, sy;
                                    sparse_xy(p, d.idx, sx, sy);
                                    tma_load_3d(slot + kTileBytes, &map_b, full, sx, sy, cur.z);
                                }
                            }
                            __syncwarp();
                        }
                    }
                    stage += kProducerWarps;
                    if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                }
                step0 += ksteps;
                ++flush_no;
            }
            pre = pre_next;
            cur.advance();
        }
        if (is_sdd && ok) {
            // No more accumulations: one closing entry for each of the epilogue groups.  Each is posted by the
            // producer that would have loaded its first K-step, i.e. the one that has posted every earlier entry
            // of that slot.  With two issuers the even and the odd accumulations are two pipelines (producers,
            // stages, issuer, accumulator buffers, epilogue groups, entry slots) that nothing keeps in step: a
            // producer of one may finish while the other is more than a ring behind, and a closing entry posted by
            // it into the other's slots would complete a phase that belongs to an accumulation still to come.
            const int ksteps = (p.size_k + kTile - 1) / kTile;
            for (int j = 0; j < kSddGroups; ++j) {
                const int e = flush_no + j;
                if (((step0 + j * ksteps) & (kProducerWarps - 1)) == warp && elect_one()) {
                    bars->ents[e & (kSddEntries - 1)] = make_int4(0, 0, 0, 0);
                    mbar_arrive(&bars->ent_full[e & (kSddEntries - 1)]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && *(volatile int*)&bars->abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp < kFirstEpilogueWarp) {
        // ------------------------------------------------------------ MMA issuers
        const int w = warp - kFirstMmaWarp;
        if (w < p.issuers) {
            // The whole warp runs the loop (warp-uniform code keeps the descriptors in uniform registers:
            // issuing from a single diverged lane costs about twice as much per instruction); one
            // elected lane executes the tcgen05 instructions.
            // Own stage pointer.  dsd / dds: this issuer's K-steps are w, w + issuers, ... of the CTA,
            // so the pointer advances by `issuers`.  sdd with two issuers: accumulations alternate,
            // so it runs through one accumulation's stages and then skips the other issuer's.
            int flush_no = 0, step0 = 0;
            int stage = is_sdd ? 0 : w;
            uint32_t phase = 0;
            bool ok = true;
            const uint32_t a_kstep = a_mn_major ? 2048u >> 4 : 32u >> 4;   // descriptor advance per K = 16
            const uint32_t b_kstep = b_mn_major ? 2048u >> 4 : 32u >> 4;
            // dsd / dds: private partial accumulator of this issuer inside the buffer
            const uint32_t part_col = is_sdd ? 0u : (uint32_t)(w * (kAccCols / p.issuers));
            const int issuer_mask = p.issuers - 1;       // issuers is 1, 2 or 4 (no runtime division here:
                                                         // it costs a lone thread hundreds of cycles)
            Cursor cur;
            cur.init(p, p.split);
            for (; ok && cur.valid(); cur.advance()) {
                int flushes, ksteps;
                item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
                if (ksteps == 0) continue;          // empty group: the epilogue writes zeros on its own
                for (int f = 0; ok && f < flushes; ++f, ++flush_no) {
                    const int acc = flush_no & (kBufs - 1);
                    if (is_sdd && p.issuers == 2 && (flush_no & 1) != w) {
                        // the other issuer's accumulation: skip its stages (the host guarantees
                        // that a stage always belongs to the same issuer)
                        stage += ksteps;
                        while (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                        continue;
                    }
                    const int nb = b_tiles<MODE>(p, cur.count << p.split, cur.chunk, f);
                    const uint32_t idesc = p.idesc | ((uint32_t)((nb * kTile) >> 3) << 17);
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_empty[acc], ((uint32_t)(flush_no >> kBufShift) & 1u) ^ 1u, &bars->abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + acc_addr(acc) + part_col;
                    bool issued = false;
                    // dsd / dds: K-step n belongs to issuer n % issuers (the stage count is a
                    // multiple of it, so a stage always belongs to the same issuer)
                    const int k_first = is_sdd ? 0 : ((w - step0) & issuer_mask);
                    const int k_inc = is_sdd ? 1 : p.issuers;
                    for (int k = k_first; k < ksteps; k += k_inc) {
                        {
                            ok = __all_sync(0xffffffffu, mbar_wait(&bars->full[stage], phase, &bars->abort_flag, p.status)) != 0;
                            if (!ok) break;
                            tc_fence_after();
                            const uint32_t slot = smem_u32(stage_base + stage * stage_bytes);
                            const uint64_t da = make_tile_desc(slot, a_mn_major);
                            const uint64_t db = make_tile_desc(slot + kTileBytes, b_mn_major);
                            if (elect_one()) {
#pragma unroll
                                for (int kk = 0; kk < kTile / 16; ++kk)
                                    tc_mma_f16(d, da + (uint64_t)(kk * a_kstep), db + (uint64_t)(kk * b_kstep), idesc,
                                               (issued || kk > 0) ? 1u : 0u);
                                tc_commit(&bars->empty[stage]);  // the stage is free once these MMAs have read it
                            }
                            __syncwarp();
                            issued = true;
                        }
                        stage += k_inc;
                        if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                    }
                    step0 += ksteps;
                    if (!ok) break;
                    // the accumulation (dsd / dds: this issuer's partial, if it had a K-step) is complete
                    if (elect_one()) {
                        if (issued) tc_commit(&bars->acc_full[acc]);
                        else        mbar_arrive(&bars->acc_full[acc]);
                    }
                    __syncwarp();
                }
            }
            // All MMAs issued by the elected lane (the same one every time) must have retired before
            // TMEM is freed.
            if (elect_one()) {
                tc_commit(&bars->drain);
                mbar_wait(&bars->drain, 0, &bars->abort_flag, p.status);
            }
            __syncwarp();
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue groups
        const int group = (warp - kFirstEpilogueWarp) >> 2;     // drains accumulator buffer `group`
        const int quad = warp & 3;                   // TMEM sub-partition this warp may read
        const int row = quad * 16 + lane;            // accumulator row held by this lane (lanes 0-15 only)
        const bool row_lane = lane < 16;
        constexpr bool bf16_out = BF16;
        bool ok = true;
        if (is_sdd) {
            // accumulation F of the CTA: entry F & 31 from the producers, accumulator buffer F & 7; group g takes
            // the accumulations F = g, g + 4, ...
            for (int flush = group; ok; flush += kSddGroups) {
                const int slot = flush & (kSddEntries - 1);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->ent_full[slot], (uint32_t)(flush / kSddEntries) & 1u, &bars->abort_flag, p.status)) != 0;
                if (!ok) break;
                const int4 ent = bars->ents[slot];
                const int tiles = ent.z;
                if (tiles == 0) break;              // no more accumulations
                const int acc = flush & (kBufs - 1);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[acc], (uint32_t)(flush >> kBufShift) & 1u, &bars->abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                // Sparse output tiles leave through shared memory and TMA: the warp converts its 16
                // accumulator rows, writes them with four stmatrix instructions (the 16x256b TMEM
                // load hands out exactly the m8n8 fragment layout) into its own 128-byte-swizzled
                // 2 KB staging slab and sends the slab to global memory with one bulk tensor store
                // (box 16 x 64).  About 30 instructions per lane and tile instead of 110 for a
                // shuffle-transpose / 128-bit store path, no synchronisation between warps, and
                // the stores are asynchronous (one slab per warp: the store of a tile reads it while
                // the warp loads and converts its next tile).
                const uint32_t tbase = tmem_base + ((uint32_t)(quad * 32) << 16) + acc_addr(acc);
                // lane -> row address of its 8x8 matrix: matrix i = lane / 8 holds rows (i & 1) * 8 ..
                // of 16-byte column unit u = 2k + (i >> 1)
                const int sm_row = ((lane >> 3) & 1) * 8 + (lane & 7);        // row inside the slab
                const uint32_t sm_unit = (uint32_t)(lane >> 4);
                const int slab0 = (warp - kFirstEpilogueWarp) * (16 * 128);         // this warp's slab
                auto store_tile = [&](const uint32_t (&r)[32], int t) {
                    const int out_idx = t == 0 ? ent.x : ent.y;
                    // a descriptor that does not belong to this layout is reported in the workspace
                    // (word 1 = offending tile index); the tensor map clips the store itself
                    const bool in_bounds = out_idx >= 0 && out_idx < p.nnz;
                    if (!in_bounds && lane == 0) {
                        atomicExch(p.status, (uint32_t)BSA_ERR_BAD_SHAPE);
                        atomicExch(p.status + 1, (uint32_t)out_idx);
                    }
                    const uint32_t slab = smem_u32(stage_base + kSddStagingTile0 * kTileBytes + slab0);
                    uint32_t w[16];                         // [4k + i]: matrices (u = 2k, rows a), (2k, b), (2k + 1, a), (2k + 1, b)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            const int u = 2 * k + (i >> 1), h = i & 1;
                            const float lo = __uint_as_float(r[4 * u + 2 * h]), hi = __uint_as_float(r[4 * u + 2 * h + 1]);
                            if (bf16_out) { __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi); w[4 * k + i] = *reinterpret_cast<uint32_t*>(&v); }
                            else          { __half2 v = __floats2half2_rn(lo, hi); w[4 * k + i] = *reinterpret_cast<uint32_t*>(&v); }
                        }
                    }
                    // the slab was sent with the tile before: that store must have read it
                    if (elect_one()) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    __syncwarp();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t addr = slab + (uint32_t)(sm_row * 128) + ((((uint32_t)(2 * k) + sm_unit) ^ (uint32_t)(sm_row & 7)) << 4);
                        asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                                     ::"r"(addr), "r"(w[4 * k]), "r"(w[4 * k + 1]), "r"(w[4 * k + 2]), "r"(w[4 * k + 3]) : "memory");
                    }
                    fence_async_shared();           // generic-proxy writes -> visible to the bulk store
                    __syncwarp();
                    // (issued from an elected lane of warp-uniform code: the copy's operands stay in
                    // uniform registers; the same lane every time, the bulk groups are per thread)
                    int sx, sy;
                    sparse_xy(p, out_idx, sx, sy);
                    if (elect_one()) {
                        if (in_bounds)
                            asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
                                         ::"l"(&map_c), "r"(slab), "r"(sx), "r"(sy + quad * 16), "r"(ent.w) : "memory");
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");   // (empty groups keep the count regular)
                    }
                };
                // one register buffer: the other groups' accumulations cover this one's TMEM load
                uint32_t r[32];
                for (int t = 0; t < tiles; ++t) {
                    tc_ld_16x256b_x8(tbase + (uint32_t)(t * kTile), r);
                    tc_wait_ld();
                    if (t + 1 >= tiles) release_accumulator(&bars->acc_empty[acc], lane);
                    store_tile(r, t);
                }
            }
        } else {
            const int parts = is_sdd ? 1 : p.issuers;
            const int part_stride = kAccCols / p.issuers;
            int flush_no = 0, step = 0;
            Cursor cur;
            cur.init(p, p.split);
            while (ok && cur.valid()) {
                int flushes, ksteps;
                item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
                const bool have_acc = ksteps > 0;
                for (int f = 0; ok && f < flushes; ++f) {
                    // accumulations alternate between the two buffers / groups; groups that write
                    // zeros for an empty group of blocks are chosen by item parity
                    const int owner = have_acc ? (flush_no & (kGroups - 1)) : (cur.item_no & (kGroups - 1));
                    const uint32_t acc_phase = (uint32_t)(flush_no >> kBufShift) & 1u;
                    const int acc = flush_no & (kBufs - 1);     // (dsd / dds: the group's own buffer)
                    const int step0 = step;             // sequence number of this accumulation's first K-step
                    step += ksteps;
                    if (have_acc) ++flush_no;
                    if (owner != group) continue;
                    const int tiles = b_tiles<MODE>(p, cur.count << p.split, cur.chunk, f);
                    if (have_acc) {
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[acc], acc_phase, &bars->abort_flag, p.status)) != 0;
                        if (!ok) break;
                        tc_fence_after();
                    }
                    for (int t = 0; t < tiles; ++t) {
                        // destination of this 64x64 tile: first element, valid rows and columns
                        size_t dst0;
                        int rows_valid = kTile, cols_valid = kTile;
                        if (MODE == BSA_MODE_DSD) {
                            const int n0 = (cur.chunk * 2 + t) * kTile;
                            dst0 = ((size_t)cur.z * p.size_m + (size_t)cur.g * kTile) * p.size_n + n0;
                            cols_valid = min(kTile, p.size_n - n0);
                        } else {
                            const int m0 = cur.chunk * kTile;
                            dst0 = ((size_t)cur.z * p.size_m + m0) * p.size_n + (size_t)cur.g * kTile;
                            rows_valid = min(kTile, p.size_m - m0);
                        }
                        // never write outside the output: a descriptor that does not belong to this
                        // layout is reported in the workspace instead (word 1 = offending offset >> 12)
                        const bool in_bounds = dst0 + (size_t)(rows_valid - 1) * p.ldc + cols_valid <= (size_t)p.c_elems;
                        if (!in_bounds && lane == 0) {
                            atomicExch(p.status, (uint32_t)BSA_ERR_BAD_SHAPE);
                            atomicExch(p.status + 1, (uint32_t)(dst0 >> 12));
                        }
                        const bool writer = row_lane && row < rows_valid && in_bounds;
                        uint16_t* dst = p.c + dst0 + (size_t)row * p.ldc;
                        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc_addr(acc) + (uint32_t)(t * kTile);
                        const bool last_tile = have_acc && t == tiles - 1;
                        if (!have_acc || parts == 1) {
                            uint32_t v[kTile];          // fp32 bit patterns of this lane's row
                            if (have_acc) {
                                tc_ld_32x32b_x64(taddr, v);
                                tc_wait_ld();
                            } else {
    #pragma unroll
                                for (int c = 0; c < kTile; ++c) v[c] = 0u;
                            }
                            if (last_tile) release_accumulator(&bars->acc_empty[acc], lane);
                            if (writer) store_row<kTile>(dst, v, cols_valid, p.c_vec8 != 0, bf16_out);
                        } else {
                            // dsd / dds: issuer w holds a partial sum iff one of the K-steps
                            // step0 .. step0 + ksteps - 1 is congruent to w; the first K-step's issuer
                            // always does, so its partial seeds the sum.  Two 32-column halves keep the
                            // register footprint small.
                            const int first_part = step0 & (parts - 1);
    #pragma unroll
                            for (int h = 0; h < 2; ++h) {
                                uint32_t v[32];
                                tc_ld_32x32b_x32(taddr + (uint32_t)(first_part * part_stride + h * 32), v);
                                tc_wait_ld();
                                for (int j = 1; j < parts && j < ksteps; ++j) {
                                    const int part = (first_part + j) & (parts - 1);
                                    uint32_t r[32];
                                    tc_ld_32x32b_x32(taddr + (uint32_t)(part * part_stride + h * 32), r);
                                    tc_wait_ld();
    #pragma unroll
                                    for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(r[c]));
                                }
                                if (last_tile && h == 1) release_accumulator(&bars->acc_empty[acc], lane);
                                if (writer) store_row<32>(dst + h * 32, v, cols_valid - h * 32, p.c_vec8 != 0, bf16_out);
                            }
                        }
                    }
                }
                cur.advance();
            }
        }
        // the staging tiles must have been read before the CTA gives its shared memory back
        if (is_sdd && elect_one()) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
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

bool dense_dim_ok(int64_t v) { return v >= kTile && v % 8 == 0 && v < ((int64_t)1 << 31); }

int64_t slices_of(const MatmulArgs& g) {
    if (g.mode == BSA_MODE_DSD) return (g.size_n + 2 * kTile - 1) / (2 * kTile);
    if (g.mode == BSA_MODE_DDS) return (g.size_m + kTile - 1) / kTile;
    return 1;
}

}  // namespace

bool tc_supports(const MatmulArgs& g) {
    if (g.dtype != BSA_DTYPE_F16 && g.dtype != BSA_DTYPE_BF16) return false;
    if (g.block != kTile && g.block != 2 * kTile) return false;
    const int split = g.block == 2 * kTile ? 1 : 0;
    if (g.nnz <= 0 || g.nnz * g.block >= ((int64_t)1 << 31) || (g.nnz << (2 * split)) >= ((int64_t)1 << 30) ||
        g.batches > 65535) return false;
    if (!dense_dim_ok(g.size_m) || !dense_dim_ok(g.size_n) || !dense_dim_ok(g.size_k)) return false;
    // work items are indexed with 32-bit integers
    if (g.batches * (g.groups << split) * slices_of(g) >= ((int64_t)1 << 30)) return false;
    return true;
}

int matmul_tc(const MatmulArgs& g) {
    // The opt-in shared-memory size is set once per kernel and device, and tensor maps are kept per
    // (address, shape): a launch-bound caller should not pay for driver calls per product.  (A map that
    // has to be encoded binds the device's primary context to the calling thread first:
    // cuTensorMapEncodeTiled is a driver call and fails with "invalid context" on a thread, e.g. an
    // autograd worker, that has not made a runtime call needing the context yet.)
    using KernelFn = void (*)(const CUtensorMap, const CUtensorMap, const CUtensorMap, const TcParams);
    const bool bf16 = g.dtype == BSA_DTYPE_BF16;
    KernelFn kernel;
    if (g.mode == BSA_MODE_SDD)      kernel = bf16 ? tc_matmul_kernel<BSA_MODE_SDD, true> : tc_matmul_kernel<BSA_MODE_SDD, false>;
    else if (g.mode == BSA_MODE_DSD) kernel = bf16 ? tc_matmul_kernel<BSA_MODE_DSD, true> : tc_matmul_kernel<BSA_MODE_DSD, false>;
    else                             kernel = bf16 ? tc_matmul_kernel<BSA_MODE_DDS, true> : tc_matmul_kernel<BSA_MODE_DDS, false>;
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kSmemBytes)) return BSA_ERR_LAUNCH;
    CUtensorMap map_a, map_b, map_c;
    const int split = g.block == 2 * kTile ? 1 : 0;
    const int64_t sparse_rows = g.nnz * g.block;     // the sparse tensor as a [nnz * block, block] matrix
    bool ok = true;
    // stored shapes: a dense operand is [rows, cols] = op^-1 of its logical shape
    if (g.mode == BSA_MODE_SDD) {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n);
        ok &= make_map(&map_c, g.dtype, g.c, g.batches, sparse_rows, g.block, 16);   // output leaves by TMA, 16 rows a time
    } else if (g.mode == BSA_MODE_DSD) {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, sparse_rows, g.block);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n);
    } else {
        ok &= make_map(&map_a, g.dtype, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map(&map_b, g.dtype, g.b, g.batches, sparse_rows, g.block);
    }
    if (!ok) return BSA_ERR_DRIVER;
    if (g.mode != BSA_MODE_SDD) map_c = map_a;      // unused by dsd / dds

    TcParams p{};
    p.blocks = g.blocks; p.table = g.table; p.status = g.workspace;
    p.split = split;
    p.col_walk = ((g.mode == BSA_MODE_DSD && g.trans_a) || (g.mode == BSA_MODE_DDS && !g.trans_b)) ? 1 : 0;
    p.nnz = (int)(g.nnz << (2 * split)); p.groups = (int)(g.groups << split); p.batches = (int)g.batches;
    p.size_m = (int)g.size_m; p.size_n = (int)g.size_n; p.size_k = (int)g.size_k;
    p.mode = g.mode; p.trans_a = g.trans_a; p.trans_b = g.trans_b;
    p.chunks = (int)slices_of(g);
    p.items = (int)(g.batches * p.groups * p.chunks);
    if (g.mode == BSA_MODE_SDD) { p.nb_max = kSddTiles; p.issuers = 2; }
    else if (g.mode == BSA_MODE_DSD && g.size_n > kTile) { p.nb_max = 2; p.issuers = 2; }
    else { p.nb_max = 1; p.issuers = 4; }
    // Every mbarrier must be waited on by the same threads in every phase (a parity wait cannot
    // tell phases two apart), so the stage count is a multiple of the producer count, and for sdd,
    // where the two issuers alternate accumulations of `ksteps` stages, a multiple of 2 * ksteps;
    // otherwise one issuer does all accumulations.
    const int ring_tiles = g.mode == BSA_MODE_SDD ? kSddStagingTile0 : kStageTiles;
    p.stages = (ring_tiles / (1 + p.nb_max)) / kProducerWarps * kProducerWarps;
    if (p.stages > kMaxStages) p.stages = kMaxStages / kProducerWarps * kProducerWarps;
    if (g.mode == BSA_MODE_SDD) {
        const int ksteps = (int)((g.size_k + kTile - 1) / kTile);
        if (p.stages % (2 * ksteps) != 0) p.issuers = 1;
    }
    // instruction descriptor: fp32 accumulate, fp16 / bf16 operands, M = 64; N is added per accumulation
    const uint32_t fmt = g.dtype == BSA_DTYPE_BF16 ? 1u : 0u;
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g.trans_a ? 1u : 0u) << 15)
              | ((g.trans_b ? 0u : 1u) << 16) | ((uint32_t)(kTile >> 4) << 24);

    p.c = static_cast<uint16_t*>(g.c);
    p.ldc = g.mode == BSA_MODE_SDD ? kTile : (int)g.size_n;
    p.c_vec8 = (reinterpret_cast<uintptr_t>(g.c) % 32 == 0 && p.ldc % 16 == 0) ? 1 : 0;
    p.c_elems = g.mode == BSA_MODE_SDD ? (long long)g.batches * g.nnz * g.block * g.block
                                       : (long long)g.batches * g.size_m * g.size_n;

    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    const unsigned grid = (unsigned)(p.items < sms ? p.items : sms);
    const int per_z = p.groups * p.chunks;
    p.stride_z = (int)grid / per_z;
    p.stride_rem = (int)grid % per_z;
    kernel<<<grid, threads_of(g.mode), kSmemBytes, g.stream>>>(map_a, map_b, map_c, p);
    return launch_status();
}

}  // namespace bsa
