// tcgen05 / TMEM engine of the block-sparse matmul for block size 32 (sm_100a only): fp16 and
// bf16 operands, and fp32 operands multiplied as a 3xTF32 split, all with fp32 accumulation in
// tensor memory.
//
// Block 32 is the only block size of the reference (sparse/native/sparse_smm_gpu.cu:22-267
// computes it on CUDA cores in fp32; sparse_hmm_gpu.cu:26-142 is its unfinished fp16 twin).
//
// Geometry.  Everything is a *panel* of 32 x 32 elements stored as 32 rows of 32 elements with
// the swizzle that spans one row (64-byte swizzle for 16-bit types, 128-byte for fp32).  A panel
// is at once a TMA box of a dense operand, a whole sparse block, and a slice of a UMMA operand
// in either major-ness:
//   K-major operand   rows are M/N indices; panels placed back to back continue the operand
//                     along M/N (stride byte offset = 8 rows); one MMA consumes 32 bytes of a row.
//   MN-major operand  rows are K indices; panels placed back to back hold consecutive 32-wide
//                     ranges of M/N (leading byte offset = one panel); one MMA consumes 1024
//                     bytes of rows (16 rows of 16-bit, 8 rows of fp32 elements).
// A K-step is 32 elements of K: two kind::f16 MMAs (K = 16) or four kind::tf32 MMAs (K = 8).
// The MMA shape is M = 64.  sdd has 32 rows of A only and loads that panel twice, so the accumulator
// rows 32-63 repeat rows 0-31 in the TMEM quarters 2 and 3 and all four warps of an epilogue
// warpgroup have output pieces to store (a warp reads its own quarter only); dsd keeps one A panel
// per stage (smaller stages, more of them in flight) and never reads the accumulator rows 32-63;
// dds, whose M is a slice of a dense dimension, uses all 64 rows.
//   sdd  item = block row r; its blocks are taken 8 (fp32: 4) at a time as one N = 256 (128)
//        accumulation over the dense inner size.
//   dsd  item = group m and a 128-wide slice of N; one accumulation over the group's blocks.
//   dds  item = group n and a 64-tall slice of M; one accumulation over the group's blocks.
//
// fp32.  kind::tf32 reads only the upper 19 bits of an fp32 word, so each operand x is split in
// shared memory into hi = x with the low 13 mantissa bits cleared (written back in place) and
// lo = x - hi (exact, written to a second copy of the stage); three MMAs per K = 8,
// hi*hi + hi*lo + lo*hi, leave a relative error of about 2^-20 per product, far inside the
// 1e-4 contract.  Non-finite inputs give NaN instead of Inf (Inf - Inf in the split).
//
// Warp roles (16 warps), barriers and bounded waits follow the block-64 engine:
//   warps 0-3   TMA producers, K-step n of the CTA belongs to producer n % 4
//   warps 4-7   tcgen05.mma issuers (sdd: one per accumulator buffer; dsd / dds: K-step n
//               belongs to issuer n % issuers, private partial accumulators)
//   warps 8-15  16-bit types: two epilogue warpgroups, one per accumulator buffer;
//               fp32: warps 8-11 one epilogue warpgroup, warps 12-15 split the stages
//               (splitter n % 4 owns K-step n) and hand them to the issuers.
#include "bsa_tc_common.cuh"

namespace bsa {
namespace {

constexpr int kBlk = 32;                        // block edge = panel edge in elements
constexpr int kMaxStages = 32;
constexpr int kPipeBytes = 27 * 8192;           // shared memory for all stages
constexpr int kAccCols = 256;                   // TMEM columns per accumulator buffer
constexpr int kTmemCols = 2 * kAccCols;
// sdd has four accumulator buffers: an M = 64 accumulator occupies lanes 0-15 of each 32-lane quarter of tensor
// memory, and a second one fits into lanes 16-31 of the same columns (lane offset 16 in the MMA's D address; a
// 32-lane TMEM load returns both).  Buffers 0 and 2 share columns 0-255, buffers 1 and 3 columns 256-511.  With two
// buffers the cycle MMAs -> barrier -> epilogue -> barrier of a buffer (2 600 cycles) bounded the kernel.
constexpr int kSddBufs = 4;
constexpr int kProducerWarps = 4;
constexpr int kFirstMmaWarp = 4;
constexpr int kFirstEpilogueWarp = 8;
constexpr int kFirstSplitWarp = 12;             // fp32 only
constexpr int kThreads = 16 * 32;

// sdd: the epilogue warps do not walk the work items.  The producer that loads an accumulation's first K-step
// posts where its output pieces go (element offsets into the sparse tensor, -1 for a rank outside the layout) in a
// ring of entries with one mbarrier each; accumulation number F uses entry F & 31 (the producers are at most
// 16 stages of one K-step each + 2 accumulator buffers ahead of the epilogue).
constexpr int kSddEntries = 32;
struct SddEntry {
    long long dst[8];               // first element of output piece t
    int pieces;                     // 0: no more accumulations
    int pad;
};
struct __align__(16) Barriers {
    uint64_t full[kMaxStages];      // TMA data of a stage has landed
    uint64_t ready[kMaxStages];     // fp32: the stage has been split into hi / lo
    uint64_t empty[kMaxStages];     // the MMAs that read a stage have retired
    uint64_t acc_full[4];           // dsd / dds: two accumulator buffers; sdd: four (see kSddBufs)
    uint64_t acc_empty[4];
    uint64_t ent_full[kSddEntries];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    SddEntry ents[kSddEntries];
};
constexpr int kSmemBytes = 1024 /* alignment slack */ + kPipeBytes + (int)sizeof(Barriers);

struct Tc32Params {
    const BlockDesc* blocks;
    const int32_t* table;
    uint32_t* status;        // workspace word
    int nnz, groups, batches;
    int size_m, size_n, size_k;
    int trans_a, trans_b;
    int chunks;              // dsd: 128-wide slices of N; dds: 64-tall slices of M; sdd: 1
    int items;
    int nb_shift;            // sdd: log2 of the blocks per accumulation
    int stages;              // pipeline depth (a multiple of 4)
    int stage_bytes;         // bytes of one stage (hi and, for fp32, lo copy)
    int lo_offset;           // fp32: distance from a panel to its lo copy
    int issuers;             // MMA issuing warps in use
    uint32_t idesc;          // instruction descriptor without the N field
    void* c;                 // output
    int ldc;                 // elements between output rows
    int stride_z, stride_rem;  // gridDim.x divided by the items per batch entry: quotient and remainder
    long long c_elems;       // elements in the output (bounds check of every store)
    int split;               // log2(block / 32): blocks of 64 / 128 are walked as 2 x 2 / 4 x 4 panels (see panel_of)
    int col_walk;            // the groups are block columns (dsd with trans_a, dds without trans_b)
    int block;               // block edge of the layout in elements
};

// Blocks of 64 and 128 (fp32 operands; 16-bit ones run on the block-64 engine).  The kernel keeps working on
// 32 x 32 panels: a real group (block row or column) is S = block / 32 virtual groups and a real block S K-steps /
// output panels of each, i.e. the kernel sees the layout with every block split in S x S, without that layout
// ever being built.  `groups` and `items` of Tc32Params count virtual groups; the cursor reads table[g >> split]
// and keeps first / count in real blocks.  Virtual descriptor i of virtual group g is real descriptor i >> split
// with one sub-index taken from g and the other from i (which of row / column depends on the walk).
struct Panel {
    int idx;                 // rank of the real block
    int rh, ch;              // panel row / column inside the block
    int row, col;            // panel coordinates in the split layout
};
__device__ __forceinline__ Panel panel_of(DescWindow& win, const Tc32Params& p, const Cursor& cur, int i, int lane) {
    const BlockDesc d = win.get(p.blocks, cur.first, cur.count, i >> p.split, lane);
    const int mask = (1 << p.split) - 1;
    const int from_step = i & mask, from_group = cur.g & mask;
    Panel v;
    v.idx = d.idx;
    v.rh = p.col_walk ? from_step : from_group;
    v.ch = p.col_walk ? from_group : from_step;
    v.row = (d.row() << p.split) + v.rh;
    v.col = (d.col() << p.split) + v.ch;
    return v;
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
}

// Descriptor of an operand made of panels (without the start address).  Bits: LBO >> 4 in
// [16,30), SBO >> 4 in [32,46), descriptor version 1 in [46,48), layout type in [61,64)
// (SWIZZLE_128B with 32-byte atoms = 1, SWIZZLE_128B = 2, SWIZZLE_64B = 4).
// An MN-major operand of 32-bit elements exists in one layout only: the 128-byte swizzle that
// permutes 32-byte pieces over groups of 4 rows (its TMA counterpart is
// CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B), so there the K groups are 4 rows (512 bytes) apart.
template <int ES>
__device__ __forceinline__ uint64_t panel_desc(bool mn_major) {
    constexpr uint32_t panel_bytes = kBlk * kBlk * ES;
    const bool atom32 = ES == 4 && mn_major;
    uint64_t d = (uint64_t)(mn_major ? (panel_bytes >> 4) : 1u) << 16;
    d |= (uint64_t)(((atom32 ? 4 : 8) * kBlk * ES) >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)(ES == 2 ? 4 : (atom32 ? 1 : 2)) << 61;
    return d;
}

// Number of accumulations (each ends in an epilogue) and K-steps per accumulation of an item.
template <int MODE>
__device__ __forceinline__ void item_shape(const Tc32Params& p, int count, int& flushes, int& ksteps) {
    if (MODE == BSA_MODE_SDD) {
        flushes = (count + (1 << p.nb_shift) - 1) >> p.nb_shift;
        ksteps = (p.size_k + kBlk - 1) / kBlk;
    } else {
        flushes = 1;
        ksteps = count;
    }
}

// Number of B panels (32 output columns each) of one accumulation.
template <int MODE>
__device__ __forceinline__ int b_panels(const Tc32Params& p, int count, int chunk, int flush) {
    if (MODE == BSA_MODE_SDD) return min(1 << p.nb_shift, count - (flush << p.nb_shift));
    if (MODE == BSA_MODE_DSD) return min(4, (p.size_n - chunk * 4 * kBlk + kBlk - 1) / kBlk);
    return 1;
}

// Stores the first `cols_valid` (a multiple of 8) of 32 fp32 accumulator values of one output
// row, converted to the output type, with 128-bit stores.
template <int DT>
__device__ __forceinline__ void store_piece(void* c, size_t elem, const uint32_t (&v)[32], int cols_valid) {
    if (DT == BSA_DTYPE_F32) {
        float* dst = static_cast<float*>(c) + elem;
#pragma unroll
        for (int q = 0; q < 8; ++q)
            if (q * 4 + 4 <= cols_valid)
                *reinterpret_cast<uint4*>(dst + q * 4) = make_uint4(v[q * 4], v[q * 4 + 1], v[q * 4 + 2], v[q * 4 + 3]);
    } else {
        uint16_t* dst = static_cast<uint16_t*>(c) + elem;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float lo = __uint_as_float(v[q * 8 + e * 2]), hi = __uint_as_float(v[q * 8 + e * 2 + 1]);
                if (DT == BSA_DTYPE_BF16) {
                    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                } else {
                    __half2 h = __floats2half2_rn(lo, hi);
                    w[e] = *reinterpret_cast<uint32_t*>(&h);
                }
            }
            if (q * 8 + 8 <= cols_valid) *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(w[0], w[1], w[2], w[3]);
        }
    }
}

template <int MODE, int DT>
__global__ void __launch_bounds__(kThreads, 1)
tc32_matmul_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const Tc32Params p) {
    constexpr int ES = DT == BSA_DTYPE_F32 ? 4 : 2;
    constexpr bool kSplit = DT == BSA_DTYPE_F32;
    constexpr int kPanelBytes = kBlk * kBlk * ES;
    constexpr int kMmasPerStep = kBlk * ES / 32;              // 32 bytes of K per MMA
    constexpr int kEpilogueGroups = kSplit ? 1 : 2;
    constexpr bool is_sdd = MODE == BSA_MODE_SDD;
    constexpr bool kWideB = MODE == BSA_MODE_DSD && ES == 2;   // dsd, 16-bit: the dense operand's panels are copied in pairs
    // The MMA is M = 64.  dds fills both A panels with a 64-tall slice of its dense operand.  sdd has 32 rows of A
    // only and loads them twice: accumulator rows 32-63 then repeat rows 0-31 in the TMEM quarters 2 and 3, and
    // the epilogue warps of those quarters, which would otherwise idle, take every other output piece.
    // dsd loads its 32 rows of A once and keeps one panel of A per stage (rows 32-63 of the MMA then read whatever
    // follows and their accumulator rows are never read): its stages are smaller and more of them are in flight,
    // which is what bounds it (2 KB of the sparse operand per stage against the memory latency).
    constexpr int kAPanels = MODE == BSA_MODE_DSD ? 1 : 2;
    constexpr bool kDupA = MODE == BSA_MODE_SDD;

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stage_base = smem;
    Barriers* bars = reinterpret_cast<Barriers*>(smem + kPipeBytes);
    int* abort_flag = &bars->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // sdd: one issuer per accumulation; dsd / dds: every issuer reports on every accumulation
    const uint32_t arrivals = is_sdd ? 1u : (uint32_t)p.issuers;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMaxStages; ++s) {
            mbar_init(&bars->full[s], 1); mbar_init(&bars->ready[s], 1); mbar_init(&bars->empty[s], 1);
        }
        for (int s = 0; s < 4; ++s) { mbar_init(&bars->acc_full[s], arrivals); mbar_init(&bars->acc_empty[s], 4); }
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

    const bool a_mn_major = p.trans_a != 0;      // op(A) panel arrives with M contiguous
    const bool b_mn_major = p.trans_b == 0;      // op(B) panel arrives with N contiguous

    if (warp < kProducerWarps && !is_sdd && p.split == 0) {
        // ------------------------------------------------------------ TMA producers, dsd / dds at block 32
        // K-step n of the CTA belongs to producer n % 4 and to stage n % stages, as below, but a producer does
        // not broadcast a block's descriptor and issue its copies from one lane, one K-step after the other:
        // lane l of the warp holds descriptor base + l of the group's blocks (the descriptor window), so in every
        // batch of up to 16 consecutive K-steps the (up to four) lanes that hold this producer's blocks each wait
        // for their own stage, arm its barrier and issue their block's copies -- one instruction for the copies of
        // several K-steps, no shuffles.  (One warp taking all K-steps of a batch was slower: a copy costs about
        // 100 cycles of its warp whichever lane issues it.)
        int n0 = 0;                              // K-steps of the CTA before the current item
        bool ok = true;
        const int batch = p.stages >= 16 ? 16 : (p.stages >= 8 ? 8 : 4);       // divides 32, at most `stages`
        Cursor cur;
        cur.init(p, p.split);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int count = cur.count;
            const int nb = b_panels<MODE>(p, count, cur.chunk, 0);
            DescWindow win;
            win.begin(p.blocks, cur.first, count, pre, lane);
            for (int kb = 0; ok && kb < count; kb += batch) {
                win.seek(p.blocks, cur.first, count, kb, lane);
                const int l = lane - (kb - win.base);
                const int n = n0 + kb + l;
                const bool has = l >= 0 && l < batch && kb + l < count && (n & (kProducerWarps - 1)) == warp;
                const BlockDesc d = win.mine;
                const int round = n / p.stages, stage = n - round * p.stages;      // (once per batch and lane)
                const uint32_t use = (uint32_t)round & 1u;
                ok = __all_sync(0xffffffffu, !has || mbar_wait(&bars->empty[stage], use ^ 1u, abort_flag, p.status)) != 0;
                if (ok && has) {
                    uint8_t* slot = stage_base + stage * p.stage_bytes;
                    uint8_t* slot_b = slot + kAPanels * kPanelBytes;
                    uint64_t* full = &bars->full[stage];
                    mbar_expect_tx(full, (uint32_t)((kAPanels + (kWideB ? (nb + 1) & ~1 : nb)) * kPanelBytes));
                    const int sy = d.idx * kBlk;             // the sparse tensor viewed as [nnz * 32, 32]
                    if (MODE == BSA_MODE_DSD) {
                        const int k0 = (p.trans_a ? d.row() : d.col()) * kBlk;
                        tma_load_3d(slot, &map_a, full, 0, sy, cur.z);
                        for (int j = 0; j < nb; j += kWideB ? 2 : 1) {
                            const int c0 = (cur.chunk * 4 + j) * kBlk;
                            if (b_mn_major) tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, c0, k0, cur.z);
                            else            tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, k0, c0, cur.z);
                        }
                    } else {
                        const int k0 = (p.trans_b ? d.col() : d.row()) * kBlk;
#pragma unroll
                        for (int j = 0; j < 2; ++j) {
                            const int m0 = (cur.chunk * 2 + j) * kBlk;   // past the end: the box reads as zero
                            if (a_mn_major) tma_load_3d(slot + j * kPanelBytes, &map_a, full, m0, k0, cur.z);
                            else            tma_load_3d(slot + j * kPanelBytes, &map_a, full, k0, m0, cur.z);
                        }
                        tma_load_3d(slot_b, &map_b, full, 0, sy, cur.z);
                    }
                }
                __syncwarp();
            }
            n0 += count;
            pre = pre_next;
            cur.advance();
        }
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp < kProducerWarps) {
        // ------------------------------------------------------------ TMA producers
        // Producer w loads K-steps w, w + 4, ... of the CTA; the stage count is a multiple of 4,
        // so its stage pointer advances by 4 and a stage is always filled by the same producer
        // (an mbarrier parity wait cannot tell phases two apart, so a thread must take part in
        // every phase of each barrier it waits on).
        int stage = warp, step0 = 0;
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
                const int nb = b_panels<MODE>(p, cur.count << p.split, cur.chunk, f);
                for (int k = (warp - step0) & (kProducerWarps - 1); ok && k < ksteps; k += kProducerWarps) {
                    if (is_sdd && p.split == 0) {
                        // Block 32.  Lane l of the warp holds descriptor base + l of the row's blocks (the descriptor
                        // window), and an accumulation's blocks never straddle a window: the lanes that hold them issue
                        // the copies of their own K panels and write their own output offsets -- no broadcasts, and one
                        // instruction for up to eight copies (broadcasting eight descriptors and issuing ten copies from
                        // one lane took 3 500 of the 4 600 cycles a producer spent per K-step).
                        const int i0 = f << p.nb_shift;
                        win.seek(p.blocks, cur.first, cur.count, i0, lane);
                        const int j = lane - (i0 - win.base);
                        const bool has = j >= 0 && j < nb;
                        const BlockDesc dj = win.mine;
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status)) != 0;
                        if (ok) {
                            uint8_t* slot = stage_base + stage * p.stage_bytes;
                            uint64_t* full = &bars->full[stage];
                            SddEntry& e = bars->ents[flush_no & (kSddEntries - 1)];
                            // first element of the output piece; a rank outside the layout is reported, not written
                            if (k == 0 && has)
                                e.dst[j] = (dj.idx < 0 || dj.idx >= p.nnz) ? -1ll - (long long)(uint32_t)dj.idx
                                                                            : (long long)(((size_t)cur.z * p.nnz + dj.idx) * (kBlk * kBlk));
                            __syncwarp();
                            const int k0 = k * kBlk, m0 = cur.g * kBlk;
                            if (elect_one()) {
                                if (k == 0) {               // the accumulation's entry for the epilogue warps
                                    e.pieces = nb;
                                    mbar_arrive(&bars->ent_full[flush_no & (kSddEntries - 1)]);
                                }
                                mbar_expect_tx(full, (uint32_t)((kAPanels + nb) * kPanelBytes));
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    if (a_mn_major) tma_load_3d(slot + h * kPanelBytes, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot + h * kPanelBytes, &map_a, full, k0, m0, cur.z);
                                }
                            }
                            __syncwarp();
                            if (has) {
                                const int n0 = dj.col() * kBlk;
                                if (b_mn_major) tma_load_3d(slot + (2 + j) * kPanelBytes, &map_b, full, n0, k0, cur.z);
                                else            tma_load_3d(slot + (2 + j) * kPanelBytes, &map_b, full, k0, n0, cur.z);
                            }
                        }
                        __syncwarp();
                        stage += kProducerWarps;
                        if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                        continue;
                    }
                    int cols[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    long long dsts[8] = {0, 0, 0, 0, 0, 0, 0, 0};
                    Panel d{0, 0, 0, 0, 0};
                    if (is_sdd) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (j < nb) {
                                const Panel out = panel_of(win, p, cur, (f << p.nb_shift) + j, lane);
                                cols[j] = out.col;
                                // first element of the output piece; a rank outside the layout is reported, not written
                                if (k == 0)
                                    dsts[j] = (out.idx < 0 || out.idx >= p.nnz) ? -1ll - (long long)(uint32_t)out.idx
                                        : (long long)((((size_t)cur.z * p.nnz + out.idx) * p.block + out.rh * kBlk) * p.block + out.ch * kBlk);
                            }
                    } else {
                        d = panel_of(win, p, cur, k, lane);
                    }
                    // TMA coordinates of the panel inside the sparse tensor viewed as [nnz * block, block]
                    const int sx = d.ch * kBlk, sy = d.idx * p.block + d.rh * kBlk;
                    {
                        // the whole warp waits (warp-uniform code keeps the copies' operands in uniform
                        // registers); one elected lane issues
                        ok = __all_sync(0xffffffffu, mbar_wait(&bars->empty[stage], phase ^ 1, abort_flag, p.status)) != 0;
                        if (ok && elect_one()) {
                            uint8_t* slot = stage_base + stage * p.stage_bytes;
                            uint8_t* slot_b = slot + kAPanels * kPanelBytes;
                            uint64_t* full = &bars->full[stage];
                            if (is_sdd && k == 0) {         // the accumulation's entry for the epilogue warps
                                SddEntry& e = bars->ents[flush_no & (kSddEntries - 1)];
#pragma unroll
                                for (int j = 0; j < 8; ++j) e.dst[j] = dsts[j];
                                e.pieces = nb;
                                mbar_arrive(&bars->ent_full[flush_no & (kSddEntries - 1)]);
                            }
                            mbar_expect_tx(full, (uint32_t)((kAPanels + (kWideB ? (nb + 1) & ~1 : nb)) * kPanelBytes));
                            if (is_sdd) {
                                const int k0 = k * kBlk, m0 = cur.g * kBlk;
#pragma unroll
                                for (int h = 0; h < 2; ++h) {
                                    if (a_mn_major) tma_load_3d(slot + h * kPanelBytes, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot + h * kPanelBytes, &map_a, full, k0, m0, cur.z);
                                }
#pragma unroll
                                for (int j = 0; j < 8; ++j) {
                                    if (j < nb) {
                                        const int n0 = cols[j] * kBlk;
                                        if (b_mn_major) tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, n0, k0, cur.z);
                                        else            tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, k0, n0, cur.z);
                                    }
                                }
                            } else if (MODE == BSA_MODE_DSD) {
                                const int k0 = (p.trans_a ? d.row : d.col) * kBlk;
                                tma_load_3d(slot, &map_a, full, sx, sy, cur.z);
                                // 16-bit: the dense panels come in pairs, one box each (see encode_map32)
                                for (int j = 0; j < nb; j += kWideB ? 2 : 1) {
                                    const int n0 = (cur.chunk * 4 + j) * kBlk;
                                    if (b_mn_major) tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, n0, k0, cur.z);
                                    else            tma_load_3d(slot_b + j * kPanelBytes, &map_b, full, k0, n0, cur.z);
                                }
                            } else {
                                const int k0 = (p.trans_b ? d.col : d.row) * kBlk;
#pragma unroll
                                for (int j = 0; j < 2; ++j) {
                                    const int m0 = (cur.chunk * 2 + j) * kBlk;   // past the end: the box reads as zero
                                    if (a_mn_major) tma_load_3d(slot + j * kPanelBytes, &map_a, full, m0, k0, cur.z);
                                    else            tma_load_3d(slot + j * kPanelBytes, &map_a, full, k0, m0, cur.z);
                                }
                                tma_load_3d(slot_b, &map_b, full, sx, sy, cur.z);
                            }
                        }
                        __syncwarp();
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
            // No more accumulations: one closing entry for each of the epilogue groups, posted by the producer that
            // would have loaded its first K-step -- the one that has posted every earlier entry of that slot.  (With
            // two issuers the even and the odd accumulations are two pipelines that nothing keeps in step; a closing
            // entry posted into the other pipeline's slot by a producer that finished more than a ring ahead of it
            // would complete a phase that belongs to an accumulation still to come.)
            const int ksteps = (p.size_k + kBlk - 1) / kBlk;
            for (int j = 0; j < 2; ++j) {
                const int e = flush_no + j;
                if (((step0 + j * ksteps) & (kProducerWarps - 1)) == warp && elect_one()) {
                    bars->ents[e & (kSddEntries - 1)].pieces = 0;
                    mbar_arrive(&bars->ent_full[e & (kSddEntries - 1)]);
                }
            }
        }
        __syncwarp();
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp < kFirstEpilogueWarp) {
        // ------------------------------------------------------------ MMA issuers
        const int w = warp - kFirstMmaWarp;
        if (w < p.issuers) {
            // (the whole warp runs the loop so that the descriptors stay in uniform registers; one
            // elected lane executes the tcgen05 instructions)
            // dsd / dds: this issuer's K-steps are w, w + issuers, ... of the CTA.  sdd with two
            // issuers: accumulations alternate, so it runs through one accumulation's stages and
            // then skips the other issuer's (the host guarantees fixed stage ownership).
            int flush_no = 0, step0 = 0;
            int stage = is_sdd ? 0 : w;
            uint32_t phase = 0;
            bool ok = true;
            // dsd, 16-bit, N contiguous: a pair of panels arrives as 32 rows of 128 bytes with the 128-byte swizzle:
            // 8-row groups along K 1024 bytes apart, pairs along N 4096 bytes apart, 16 rows of K = 2048 bytes per MMA
            const uint64_t wide_b = ((uint64_t)(4096u >> 4) << 16) | ((uint64_t)(1024u >> 4) << 32) | ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
            const uint64_t desc_a0 = panel_desc<ES>(a_mn_major), desc_b0 = (kWideB && b_mn_major) ? wide_b : panel_desc<ES>(b_mn_major);
            const uint32_t a_kstep = a_mn_major ? 1024u >> 4 : 32u >> 4;   // descriptor advance per MMA
            const uint32_t b_kstep = (kWideB && b_mn_major) ? 2048u >> 4 : (b_mn_major ? 1024u >> 4 : 32u >> 4);
            const uint32_t lo = (uint32_t)p.lo_offset >> 4;
            const uint32_t part_col = is_sdd ? 0u : (uint32_t)(w * (kAccCols / p.issuers));
            const int issuer_mask = p.issuers - 1;       // issuers is 1, 2 or 4
            Cursor cur;
            cur.init(p, p.split);
            for (; ok && cur.valid(); cur.advance()) {
                int flushes, ksteps;
                item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
                if (ksteps == 0) continue;          // empty group: the epilogue writes zeros on its own
                for (int f = 0; ok && f < flushes; ++f, ++flush_no) {
                    const int acc = is_sdd ? (flush_no & (kSddBufs - 1)) : (flush_no & 1);
                    const uint32_t acc_use = (uint32_t)(is_sdd ? flush_no >> 2 : flush_no >> 1) & 1u;
                    if (is_sdd && p.issuers == 2 && (flush_no & 1) != w) {
                        stage += ksteps;
                        while (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                        continue;
                    }
                    const int nb = b_panels<MODE>(p, cur.count << p.split, cur.chunk, f);
                    const uint32_t idesc = p.idesc | ((uint32_t)((nb * kBlk) >> 3) << 17);
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_empty[acc], acc_use ^ 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    const uint32_t d = tmem_base + (uint32_t)((acc & 1) * kAccCols) + ((uint32_t)((acc >> 1) * 16) << 16) + part_col;
                    bool issued = false;
                    const int k_first = is_sdd ? 0 : ((w - step0) & issuer_mask);
                    const int k_inc = is_sdd ? 1 : p.issuers;
                    for (int k = k_first; k < ksteps; k += k_inc) {
                        ok = __all_sync(0xffffffffu, mbar_wait(kSplit ? &bars->ready[stage] : &bars->full[stage], phase, abort_flag, p.status)) != 0;
                        if (!ok) break;
                        tc_fence_after();
                        const uint32_t slot = smem_u32(stage_base + stage * p.stage_bytes);
                        const uint64_t da = desc_a0 | (uint64_t)((slot & 0x3FFFFu) >> 4);
                        const uint64_t db = desc_b0 | (uint64_t)(((slot + kAPanels * kPanelBytes) & 0x3FFFFu) >> 4);
                        if (elect_one()) {
#pragma unroll
                            for (int kk = 0; kk < kMmasPerStep; ++kk) {
                                const uint64_t a = da + (uint64_t)(kk * a_kstep), b = db + (uint64_t)(kk * b_kstep);
                                const uint32_t accumulate = (issued || kk > 0) ? 1u : 0u;
                                if (kSplit) {
                                    tc_mma_tf32(d, a, b + lo, idesc, accumulate);     // hi * lo
                                    tc_mma_tf32(d, a + lo, b, idesc, 1u);             // lo * hi
                                    tc_mma_tf32(d, a, b, idesc, 1u);                  // hi * hi
                                } else {
                                    tc_mma_f16(d, a, b, idesc, accumulate);
                                }
                            }
                            tc_commit(&bars->empty[stage]);  // the stage is free once these MMAs have read it
                        }
                        __syncwarp();
                        issued = true;
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
                mbar_wait(&bars->drain, 0, abort_flag, p.status);
            }
        }
        __syncwarp();
    } else if (kSplit && warp >= kFirstSplitWarp) {
        // ------------------------------------------------------------ fp32 hi / lo splitters
        // Splitter s handles K-steps s, s + 4, ... of the CTA (the stages producer s fills).
        const int s = warp - kFirstSplitWarp;
        int stage = s, step0 = 0;
        uint32_t phase = 0;
        bool ok = true;
        Cursor cur;
        cur.init(p, p.split);
        for (; ok && cur.valid(); cur.advance()) {
            int flushes, ksteps;
            item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
            for (int f = 0; ok && f < flushes; ++f) {
                const int nb = b_panels<MODE>(p, cur.count << p.split, cur.chunk, f);
                for (int k = (s - step0) & 3; ok && k < ksteps; k += 4) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->full[stage], phase, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    uint8_t* slot = stage_base + stage * p.stage_bytes;
                    // both A panels and nb B panels
                    const int chunks16 = (kAPanels + nb) * (kPanelBytes / 16);
                    for (int i = lane; i < chunks16; i += 32) {
                        uint4* hi_ptr = reinterpret_cast<uint4*>(slot) + i;
                        uint4* lo_ptr = reinterpret_cast<uint4*>(slot + p.lo_offset) + i;
                        const uint4 x = *hi_ptr;
                        uint4 h, l;
                        h.x = x.x & 0xFFFFE000u; l.x = __float_as_uint(__uint_as_float(x.x) - __uint_as_float(h.x));
                        h.y = x.y & 0xFFFFE000u; l.y = __float_as_uint(__uint_as_float(x.y) - __uint_as_float(h.y));
                        h.z = x.z & 0xFFFFE000u; l.z = __float_as_uint(__uint_as_float(x.z) - __uint_as_float(h.z));
                        h.w = x.w & 0xFFFFE000u; l.w = __float_as_uint(__uint_as_float(x.w) - __uint_as_float(h.w));
                        *hi_ptr = h;
                        *lo_ptr = l;
                    }
                    fence_async_shared();        // generic-proxy writes -> visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->ready[stage]);
                    stage += 4;
                    if (stage >= p.stages) { stage -= p.stages; phase ^= 1; }
                }
                step0 += ksteps;
            }
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ epilogue groups
        const int group = (warp - kFirstEpilogueWarp) >> 2;     // 16-bit: drains accumulator buffer `group`
        const int quad = warp & 3;                   // TMEM sub-partition this warp may read
        // accumulator row held by this lane (lanes 0-15 only); sdd / dsd: output row, the quarters 2 and 3 repeat 0 and 1
        const int row = (!kDupA ? quad : (quad & 1)) * 16 + lane;
        const int half = !kDupA ? 0 : quad >> 1;       // sdd: this warp takes the pieces t with t % 2 == half
        constexpr int kPieceStep = !kDupA ? 1 : 2;
        const bool row_lane = lane < 16;
        const bool quad_active = MODE != BSA_MODE_DSD || quad < 2;
        const int parts = is_sdd ? 1 : p.issuers;
        const int part_stride = kAccCols / p.issuers;
        int flush_no = 0, step = 0;
        bool ok = true;
        if (is_sdd) {
            // Accumulation F of the CTA: entry F & 31 from the producers, accumulator buffer F & 1; with two
            // groups, group g takes the accumulations F = g, g + 2, ...  The TMEM load of piece t + 1 is in
            // flight while piece t is converted and stored (two register buffers).
            for (int flush = kEpilogueGroups == 1 ? 0 : group; ok; flush += kEpilogueGroups) {
                const int slot = flush & (kSddEntries - 1);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->ent_full[slot], (uint32_t)(flush / kSddEntries) & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                const SddEntry& ent = bars->ents[slot];
                const int pieces = ent.pieces;
                if (pieces == 0) break;             // no more accumulations
                const int acc = flush & (kSddBufs - 1);
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[acc], (uint32_t)(flush >> 2) & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                if (quad_active) {
                    const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)((acc & 1) * kAccCols);
                    // the buffer's rows are in lanes 0-15 (buffers 0, 1) or 16-31 (buffers 2, 3) of the loaded 32
                    const bool my_lane = (lane >> 4) == (acc >> 1);
                    const int my_row = (quad & 1) * 16 + (lane & 15);
                    auto store = [&](const uint32_t (&v)[32], int t) {
                        const long long dst0 = ent.dst[t];
                        // never write outside the output: a descriptor that does not belong to this layout is
                        // reported in the workspace instead (word 1 = its rank)
                        const bool in_bounds = dst0 >= 0 && (size_t)dst0 + (size_t)(kBlk - 1) * p.ldc + kBlk <= (size_t)p.c_elems;
                        if (!in_bounds && lane == 0) {
                            atomicExch(p.status, (uint32_t)BSA_ERR_BAD_SHAPE);
                            atomicExch(p.status + 1, dst0 < 0 ? (uint32_t)(-1ll - dst0) : (uint32_t)(dst0 >> 12));
                        }
                        if (my_lane && in_bounds) store_piece<DT>(p.c, (size_t)dst0 + (size_t)my_row * p.ldc, v, kBlk);
                    };
                    uint32_t va[32], vb[32];
                    if (half < pieces) tc_ld_32x32b_x32(taddr + (uint32_t)(half * kBlk), va);
                    for (int t = half; t < pieces; t += 4) {
                        tc_wait_ld();
                        if (t + 2 < pieces) tc_ld_32x32b_x32(taddr + (uint32_t)((t + 2) * kBlk), vb);
                        store(va, t);
                        if (t + 2 >= pieces) break;
                        tc_wait_ld();
                        if (t + 4 < pieces) tc_ld_32x32b_x32(taddr + (uint32_t)((t + 4) * kBlk), va);
                        store(vb, t + 2);
                    }
                }
                release_accumulator(&bars->acc_empty[acc], lane);
            }
        }
        Cursor cur;
        cur.init(p, p.split);
        BlockDesc pre{0, 0};
        if (is_sdd && cur.valid()) pre = load_first_chunk(p.blocks, cur.first, cur.count, lane);
        while (!is_sdd && ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (is_sdd && cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            int flushes, ksteps;
            item_shape<MODE>(p, cur.count << p.split, flushes, ksteps);
            const bool have_acc = ksteps > 0;
            DescWindow win;
            if (is_sdd) win.begin(p.blocks, cur.first, cur.count, pre, lane);
            for (int f = 0; ok && f < flushes; ++f) {
                // accumulations alternate between the two buffers; with two groups, group b drains
                // buffer b and zeros for an empty group of blocks are written by item parity
                const int acc = flush_no & 1;
                const int owner = kEpilogueGroups == 1 ? 0 : (have_acc ? acc : (cur.item_no & 1));
                const uint32_t acc_phase = (uint32_t)(flush_no >> 1) & 1u;
                const int step0 = step;             // sequence number of this accumulation's first K-step
                step += ksteps;
                if (have_acc) ++flush_no;
                if (owner != group) continue;
                const int pieces = b_panels<MODE>(p, cur.count << p.split, cur.chunk, f);
                if (have_acc) {
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_full[acc], acc_phase, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                }
                if (quad_active) {
                    for (int t = half; t < pieces; t += kPieceStep) {
                        // destination of this 32-column piece: first element, valid rows and columns
                        size_t dst0;
                        int rows_valid = kBlk, cols_valid = kBlk;
                        if (is_sdd) {
                            const Panel out = panel_of(win, p, cur, (f << p.nb_shift) + t, lane);
                            // a rank outside the layout makes the bounds check below fail (reported, not written)
                            dst0 = (out.idx < 0 || out.idx >= p.nnz) ? (size_t)p.c_elems
                                               : (((size_t)cur.z * p.nnz + out.idx) * p.block + out.rh * kBlk) * p.block + out.ch * kBlk;
                        } else if (MODE == BSA_MODE_DSD) {
                            const int n0 = (cur.chunk * 4 + t) * kBlk;
                            dst0 = ((size_t)cur.z * p.size_m + (size_t)cur.g * kBlk) * p.size_n + n0;
                            cols_valid = min(kBlk, p.size_n - n0);
                        } else {
                            const int m0 = cur.chunk * 2 * kBlk;
                            dst0 = ((size_t)cur.z * p.size_m + m0) * p.size_n + (size_t)cur.g * kBlk;
                            rows_valid = min(2 * kBlk, p.size_m - m0);
                        }
                        // never write outside the output: a descriptor that does not belong to this
                        // layout is reported in the workspace instead (word 1 = offending offset >> 12)
                        const bool in_bounds = dst0 + (size_t)(rows_valid - 1) * p.ldc + cols_valid <= (size_t)p.c_elems;
                        if (!in_bounds && lane == 0) {
                            atomicExch(p.status, (uint32_t)BSA_ERR_BAD_SHAPE);
                            atomicExch(p.status + 1, (uint32_t)(dst0 >> 12));
                        }
                        const bool writer = row_lane && row < rows_valid && in_bounds;
                        const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(acc * kAccCols + t * kBlk);
                        uint32_t v[32];             // fp32 bit patterns of 32 columns of this lane's row
                        if (have_acc) {
                            // dsd / dds: issuer j holds a partial sum iff one of the K-steps step0 ..
                            // step0 + ksteps - 1 is congruent to j; the first K-step's issuer always does
                            const int first_part = step0 & (parts - 1);
                            tc_ld_32x32b_x32(taddr + (uint32_t)(first_part * part_stride), v);
                            tc_wait_ld();
                            for (int j = 1; j < parts && j < ksteps; ++j) {
                                const int part = (first_part + j) & (parts - 1);
                                uint32_t r[32];
                                tc_ld_32x32b_x32(taddr + (uint32_t)(part * part_stride), r);
                                tc_wait_ld();
#pragma unroll
                                for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) + __uint_as_float(r[c]));
                            }
                        } else {
#pragma unroll
                            for (int c = 0; c < 32; ++c) v[c] = 0u;
                        }
                        if (writer) store_piece<DT>(p.c, dst0 + (size_t)row * p.ldc, v, cols_valid);
                    }
                }
                if (have_acc) release_accumulator(&bars->acc_empty[acc], lane);
            }
            pre = pre_next;
            cur.advance();
        }
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
// 3-D tensor map over a row-major [batches, rows, cols] tensor with a 32x32x1 box and the swizzle
// that spans a box row (fp32 operands used MN-major: its variant with 32-byte atoms, see
// panel_desc).  Out-of-range parts of a box read as zero.
// `wide`: the 16-bit dense operand of dsd, whose panels come two at a time: an MN-major pair is one box of
// 32 rows x 64 elements with the 128-byte swizzle, a K-major pair one box of 64 rows x 32 elements.
bool encode_map32(CUtensorMap* map, int dtype, bool mn_major, const void* base, int64_t batches, int64_t rows,
                  int64_t cols, bool wide = false) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t es = dtype == BSA_DTYPE_F32 ? 4 : 2;
    const cuuint64_t dims[3] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)batches};
    const cuuint64_t strides[2] = {(cuuint64_t)cols * es, (cuuint64_t)rows * (cuuint64_t)cols * es};
    const cuuint32_t box[3] = {(cuuint32_t)(wide && mn_major ? 2 * kBlk : kBlk), (cuuint32_t)(wide && !mn_major ? 2 * kBlk : kBlk), 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUtensorMapDataType type = dtype == BSA_DTYPE_F32    ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                     : dtype == BSA_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                               : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    const CUresult res = fn(map, type, 3, const_cast<void*>(base), dims, strides, box, elem,
                            CU_TENSOR_MAP_INTERLEAVE_NONE,
                            dtype != BSA_DTYPE_F32 ? (wide && mn_major ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B)
                            : mn_major             ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                   : CU_TENSOR_MAP_SWIZZLE_128B,
                            CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (res != CUDA_SUCCESS)
        std::fprintf(stderr, "bsa: cuTensorMapEncodeTiled failed with CUresult %d (base %p, dims %lld x %lld x %lld)\n",
                     (int)res, base, (long long)batches, (long long)rows, (long long)cols);
    return res == CUDA_SUCCESS;
}

bool make_map32(CUtensorMap* map, int dtype, bool mn_major, const void* base, int64_t batches, int64_t rows,
                int64_t cols, bool wide = false) {
    return cached_map(map, MapKey{base, batches, rows, cols, dtype, (mn_major ? 1 : 0) + (wide ? 2 : 0)},
                      [&](CUtensorMap* m) { return encode_map32(m, dtype, mn_major, base, batches, rows, cols, wide); });
}

bool dense_dim_ok32(int64_t v) { return v >= kBlk && v % 8 == 0 && v < ((int64_t)1 << 31); }

int64_t slices_of32(const MatmulArgs& g) {
    if (g.mode == BSA_MODE_DSD) return (g.size_n + 4 * kBlk - 1) / (4 * kBlk);
    if (g.mode == BSA_MODE_DDS) return (g.size_m + 2 * kBlk - 1) / (2 * kBlk);
    return 1;
}

using Kernel32Fn = void (*)(const CUtensorMap, const CUtensorMap, const Tc32Params);

template <int MODE>
Kernel32Fn pick_dtype(int dtype) {
    if (dtype == BSA_DTYPE_F32) return tc32_matmul_kernel<MODE, BSA_DTYPE_F32>;
    if (dtype == BSA_DTYPE_BF16) return tc32_matmul_kernel<MODE, BSA_DTYPE_BF16>;
    return tc32_matmul_kernel<MODE, BSA_DTYPE_F16>;
}

}  // namespace

bool tc32_supports(const MatmulArgs& g) {
    if (g.dtype != BSA_DTYPE_F16 && g.dtype != BSA_DTYPE_BF16 && g.dtype != BSA_DTYPE_F32) return false;
    // block 32 in every type; fp32 (3xTF32) also at blocks 64 and 128, walked as 2 x 2 / 4 x 4 panels
    if (g.block != kBlk && !(g.dtype == BSA_DTYPE_F32 && (g.block == 2 * kBlk || g.block == 4 * kBlk))) return false;
    if (g.nnz <= 0 || g.nnz * g.block >= ((int64_t)1 << 31) || g.batches > 65535) return false;
    if (!dense_dim_ok32(g.size_m) || !dense_dim_ok32(g.size_n) || !dense_dim_ok32(g.size_k)) return false;
    // work items are indexed with 32-bit integers
    if (g.batches * g.groups * (g.block / kBlk) * slices_of32(g) >= ((int64_t)1 << 30)) return false;
    return true;
}

int matmul_tc32(const MatmulArgs& g) {
    const Kernel32Fn kernel = g.mode == BSA_MODE_SDD   ? pick_dtype<BSA_MODE_SDD>(g.dtype)
                              : g.mode == BSA_MODE_DSD ? pick_dtype<BSA_MODE_DSD>(g.dtype)
                                                       : pick_dtype<BSA_MODE_DDS>(g.dtype);
    if (!ensure_dynamic_smem(reinterpret_cast<const void*>(kernel), kSmemBytes)) return BSA_ERR_LAUNCH;
    const bool f32 = g.dtype == BSA_DTYPE_F32;
    const int panel_bytes = kBlk * kBlk * (f32 ? 4 : 2);
    CUtensorMap map_a, map_b;
    const int64_t sparse_rows = g.nnz * g.block;      // the sparse tensor as a [nnz * block, block] matrix
    const int split = g.block == 4 * kBlk ? 2 : (g.block == 2 * kBlk ? 1 : 0);
    bool ok = true;
    // stored shapes: a dense operand is [rows, cols] = op^-1 of its logical shape
    if (g.mode == BSA_MODE_SDD) {
        ok &= make_map32(&map_a, g.dtype, g.trans_a, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map32(&map_b, g.dtype, !g.trans_b, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n);
    } else if (g.mode == BSA_MODE_DSD) {
        ok &= make_map32(&map_a, g.dtype, g.trans_a, g.a, g.batches, sparse_rows, g.block);
        ok &= make_map32(&map_b, g.dtype, !g.trans_b, g.b, g.batches, g.trans_b ? g.size_n : g.size_k, g.trans_b ? g.size_k : g.size_n,
                         /*wide=*/!f32);
    } else {
        ok &= make_map32(&map_a, g.dtype, g.trans_a, g.a, g.batches, g.trans_a ? g.size_k : g.size_m, g.trans_a ? g.size_m : g.size_k);
        ok &= make_map32(&map_b, g.dtype, !g.trans_b, g.b, g.batches, sparse_rows, g.block);
    }
    if (!ok) return BSA_ERR_DRIVER;

    Tc32Params p{};
    p.blocks = g.blocks; p.table = g.table; p.status = g.workspace;
    p.split = split; p.block = g.block;
    p.col_walk = ((g.mode == BSA_MODE_DSD && g.trans_a) || (g.mode == BSA_MODE_DDS && !g.trans_b)) ? 1 : 0;
    p.nnz = (int)g.nnz; p.groups = (int)(g.groups << split); p.batches = (int)g.batches;
    p.size_m = (int)g.size_m; p.size_n = (int)g.size_n; p.size_k = (int)g.size_k;
    p.trans_a = g.trans_a; p.trans_b = g.trans_b;
    p.chunks = (int)slices_of32(g);
    p.items = (int)(g.batches * p.groups * p.chunks);
    int nb_max;                                    // B panels per stage
    if (g.mode == BSA_MODE_SDD) { p.nb_shift = f32 ? 2 : 3; nb_max = 1 << p.nb_shift; p.issuers = 2; }
    else if (g.mode == BSA_MODE_DSD && g.size_n > 2 * kBlk) { nb_max = 4; p.issuers = 2; }
    else if (g.mode == BSA_MODE_DSD) { nb_max = 2; p.issuers = 4; }
    else { nb_max = 1; p.issuers = 4; }
    p.lo_offset = ((g.mode == BSA_MODE_DSD ? 1 : 2) + nb_max) * panel_bytes;
    p.stage_bytes = p.lo_offset * (f32 ? 2 : 1);
    // Every mbarrier must be waited on by the same threads in every phase (a parity wait cannot
    // tell phases two apart), so the stage count is a multiple of the producer count, and for sdd,
    // where two issuers alternate accumulations of `ksteps` stages, a multiple of 2 * ksteps;
    // otherwise one issuer does all accumulations.
    p.stages = (kPipeBytes / p.stage_bytes) / kProducerWarps * kProducerWarps;
    if (p.stages > kMaxStages) p.stages = kMaxStages;
    if (p.stages < kProducerWarps) return BSA_ERR_LAUNCH;
    if (g.mode == BSA_MODE_SDD) {
        const int ksteps = (int)((g.size_k + kBlk - 1) / kBlk);
        if (p.stages % (2 * ksteps) != 0) p.issuers = 1;
    }
    // instruction descriptor: fp32 accumulate, operand format (f16 0, bf16 1, tf32 2), majors, M = 64;
    // N is added per accumulation
    const uint32_t fmt = f32 ? 2u : (g.dtype == BSA_DTYPE_BF16 ? 1u : 0u);
    p.idesc = (1u << 4) | (fmt << 7) | (fmt << 10) | ((g.trans_a ? 1u : 0u) << 15)
              | ((g.trans_b ? 0u : 1u) << 16) | ((uint32_t)(64 >> 4) << 24);

    p.c = g.c;
    p.ldc = g.mode == BSA_MODE_SDD ? g.block : (int)g.size_n;
    p.c_elems = g.mode == BSA_MODE_SDD ? (long long)g.batches * g.nnz * g.block * g.block
                                       : (long long)g.batches * g.size_m * g.size_n;

    const int sms = sm_count();
    if (sms <= 0) return BSA_ERR_LAUNCH;
    const unsigned grid = (unsigned)(p.items < sms ? p.items : sms);
    const int per_z = p.groups * p.chunks;
    p.stride_z = (int)grid / per_z;
    p.stride_rem = (int)grid % per_z;
    kernel<<<grid, kThreads, kSmemBytes, g.stream>>>(map_a, map_b, p);
    return launch_status();
}

}  // namespace bsa
