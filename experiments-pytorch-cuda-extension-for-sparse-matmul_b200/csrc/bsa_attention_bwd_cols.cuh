// Fused attention backward, dK and dV by block columns, head dim 64: two independent pipelines per CTA.
// Included by bsa_attention_bwd.cu inside its anonymous namespace (it uses BwdParams and the helpers
// of bsa_tc_common.cuh).
//
// A pipeline walks its own block columns (pipeline number = 2 * CTA + g of 2 * grid pipelines) with
// its own producer warp, two issuer warps, compute warpgroup, shared-memory tiles, tensor-memory
// buffers and barriers; one CTA per SM with all 512 TMEM columns.  Per block (r, c), with the keys
// of block column c on the TMEM lanes and the queries of block row r along the columns:
//   T1 = K_c Q_r^T = S^T,  T2 = V_c dO_r^T = dP^T,
//   P^T = exp2(c2 * S^T - lse2_q),  dS^T = P^T o (scale * dP^T - scale * D_q)   (lse2, D per column),
//   dV_c += P^T dO_r,  dK_c += dS^T Q_r   with the A operands (P^T, dS^T) read from tensor memory.
// Tensor memory of a pipeline (256 columns; an M = 64 accumulator occupies lanes 0-15 of each 32-lane
// quarter, a second one fits into lanes 16-31 of the same columns):
//   lanes  0-15:  dV columns 0-63 | dK columns 64-127 | P^T buffers 0, 1 at 128, 160 | dS^T buffers 0, 1 at 192, 224
//   lanes 16-31:  T1 buffer b at columns 128 b .. + 63, T2 buffer b at 128 b + 64 .. + 127
// so T is double buffered (the products of block t + 1 run while block t is worked on) and so are the
// operand buffers.  (A TMEM A operand is used at lane offset 0 with its D at lane offset 0 only.)
//   warps 0-7, 8-15  compute warps of pipeline 0, 1: warp w works on the TMEM quarter w % 4 (16 key rows) and on the
//                    query columns 32 * ((w / 4) % 2) .. + 31 of every block (the backward has no reduction along a row,
//                    so the columns of a block split freely over two warps: twice the warps on a block's arithmetic)
//   warps 16, 19     producer: the column's X pair (K_c, V_c), then per block the Y pair (Q_r, dO_r) and the 512 bytes of
//                    (lse2, D) of its query rows (four stages)
//   warps 17, 20     issuer of T1 and T2
//   warps 18, 21     issuer of the two accumulations
constexpr int kBwdColItems = 8;
struct __align__(16) BwdColBarriers {
    uint64_t x_full[2], x_empty[2];             // [pipeline]
    uint64_t y_full[2][4], y_free[2][4];        // [pipeline][block & 3]: y_free = the accumulations of the block have retired
    uint64_t t_full[2][2], t_empty[2][2];       // [pipeline][block & 1]
    uint64_t op_full[2][2], op_free[2][2];      // [pipeline][block & 1]: the operand buffers
    uint64_t o_full[2], o_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    BlockDesc descs[2][4];                      // [pipeline][block & 3]: written by the producer for the compute warps
    uint64_t col_full[2][kBwdColItems];         // [pipeline][column & 7]: the column's entry in `cols` is valid
    int4 cols[2][kBwdColItems];                 // (batch entry, block column, blocks, -): written by the producer; blocks = 0: no more columns
};
constexpr int kBwdColRing = 4;
constexpr int kBwdColTiles = 2 + 2 * kBwdColRing;       // per pipeline: K, V, (Q, dO) x 4
constexpr int kBwdColWarps = 22;

template <bool BF16, bool MASKED>
__global__ void __launch_bounds__(kBwdColWarps * 32, 1)
attention_backward_cols_pipes_kernel(const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                     const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                                     const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t* stats_smem = smem + 2 * kBwdColTiles * kTileBytes;              // [pipeline][stage] x 64 float2
    BwdColBarriers* bars = reinterpret_cast<BwdColBarriers*>(stats_smem + 2 * kBwdColRing * kBwdStatBytes);
    int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = warp < 16 ? warp >> 3 : (warp - 16) / 3;         // pipeline of this warp
    const int role = warp < 16 ? 3 : (warp - 16) % 3;              // 0 producer, 1 T issuer, 2 accumulation issuer, 3 compute
    uint8_t* x_smem = smem + g * kBwdColTiles * kTileBytes;        // K_c, V_c
    uint8_t* y_smem = x_smem + 2 * kTileBytes;                     // [stage][Q_r, dO_r]
    uint8_t* st_smem = stats_smem + g * kBwdColRing * kBwdStatBytes;

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->x_full[i], 1); mbar_init(&bars->x_empty[i], 1);
            for (int s = 0; s < kBwdColRing; ++s) { mbar_init(&bars->y_full[i][s], 1); mbar_init(&bars->y_free[i][s], 1); }
            for (int s = 0; s < 2; ++s) {
                mbar_init(&bars->t_full[i][s], 1); mbar_init(&bars->t_empty[i][s], 8);
                mbar_init(&bars->op_full[i][s], 8); mbar_init(&bars->op_free[i][s], 1);
            }
            for (int s = 0; s < kBwdColItems; ++s) mbar_init(&bars->col_full[i][s], 1);
            mbar_init(&bars->o_full[i], 1); mbar_init(&bars->o_empty[i], 8);
        }
        mbar_init(&bars->drain, 4);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (warp == 16) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;
    const uint32_t dv_tmem = tmem_base + (uint32_t)(g * 256);              // dV: lanes 0-15 of columns 0 .. 63
    const uint32_t dk_tmem = dv_tmem + 64u;                                // dK: lanes 0-15 of columns 64 .. 127
    const uint32_t pt_tmem = dv_tmem + 128u;                               // P^T buffer b: lanes 0-15 of columns 128 + 32 b ..
    const uint32_t ds_tmem = dv_tmem + 192u;                               // dS^T buffer b: lanes 0-15 of columns 192 + 32 b ..
    const uint32_t t_tmem = dv_tmem + (16u << 16);                         // T1 / T2 buffer b: lanes 16-31 of columns 128 b (+ 64) ..
    const int walker = 2 * (int)blockIdx.x + g, walkers = 2 * (int)gridDim.x;

    if (role == 0) {
        // ------------------------------------------------------------ producer
        int t0 = 0, i_no = 0;                       // blocks and non-empty columns before the current column
        bool ok = true;
        Cursor cur;
        cur.init_as(p, walker, walkers, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n == 0) {
                // a column without blocks: zero gradient rows (the other roles never see the column)
                const size_t row0 = (size_t)cur.z * p.seq_k + (size_t)cur.g * kTile;
                for (int c = lane; c < kTile * kTile / 8; c += 32) {
                    reinterpret_cast<uint4*>(p.out0 + row0 * kTile)[c] = make_uint4(0u, 0u, 0u, 0u);
                    reinterpret_cast<uint4*>(p.out1 + row0 * kTile)[c] = make_uint4(0u, 0u, 0u, 0u);
                }
            } else {
                // the X pair once the last T products of the column before have retired
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_empty[g], ((uint32_t)i_no & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (ok && elect_one()) {
                    // The column's entry for the issuers and the compute warps: they are at most three columns
                    // behind (the wait above: the compute warps have taken the T tiles two blocks before that
                    // column's last).
                    bars->cols[g][i_no & (kBwdColItems - 1)] = make_int4(cur.z, cur.g, n, 0);
                    mbar_arrive(&bars->col_full[g][i_no & (kBwdColItems - 1)]);
                    mbar_expect_tx(&bars->x_full[g], (uint32_t)(2 * kTileBytes));
                    tma_load_3d(x_smem, &map_k, &bars->x_full[g], 0, cur.g * kTile, cur.z);
                    tma_load_3d(x_smem + kTileBytes, &map_v, &bars->x_full[g], 0, cur.g * kTile, cur.z);
                }
                __syncwarp();
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j) {
                    const BlockDesc desc = win.get(p.blocks, cur.first, cur.count, j, lane);
                    const int row = desc.row();
                    const int t = t0 + j, st = t & (kBwdColRing - 1);
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_free[g][st], ((uint32_t)(t >> 2) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                    if (ok && elect_one()) {
                        uint64_t* full = &bars->y_full[g][st];
                        bars->descs[g][st] = desc;      // for the compute warps; the slot is free like the stage
                        mbar_expect_tx(full, (uint32_t)(2 * kTileBytes + kBwdStatBytes));
                        tma_load_3d(y_smem + (2 * st) * kTileBytes, &map_q, full, 0, row * kTile, cur.z);
                        tma_load_3d(y_smem + (2 * st + 1) * kTileBytes, &map_do, full, 0, row * kTile, cur.z);
                        bulk_load_1d(st_smem + st * kBwdStatBytes, p.stats + (size_t)cur.z * p.seq_q + (size_t)row * kTile,
                                     kBwdStatBytes, full);
                    }
                    __syncwarp();
                }
                t0 += n;
                ++i_no;
            }
            pre = pre_next;
            cur.advance();
        }
        if (ok && elect_one()) {                    // no more columns
            bars->cols[g][i_no & (kBwdColItems - 1)] = make_int4(0, 0, 0, 0);
            mbar_arrive(&bars->col_full[g][i_no & (kBwdColItems - 1)]);
        }
        __syncwarp();
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (role == 1) {
        // ------------------------------------------------------------ issuer of T1 = K_c Q_r^T and T2 = V_c dO_r^T
        const uint64_t x1_desc = make_tile_desc(smem_u32(x_smem), false);
        const uint64_t x2_desc = make_tile_desc(smem_u32(x_smem + kTileBytes), false);
        int t0 = 0, i_no = 0;
        bool ok = true;
        while (ok) {
            // the column's entry from the producer (columns without blocks never get here)
            const int slot = i_no & (kBwdColItems - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->col_full[g][slot], (uint32_t)(i_no / kBwdColItems) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int n = bars->cols[g][slot].z;
            if (n == 0) break;                      // no more columns
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
            for (int j = 0; ok && j < n; ++j) {
                const int t = t0 + j, st = t & (kBwdColRing - 1), b = t & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[g][st], (uint32_t)(t >> 2) & 1u, abort_flag, p.status)) != 0;
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_empty[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                const uint64_t y1 = make_tile_desc(smem_u32(y_smem + (2 * st) * kTileBytes), false);
                const uint64_t y2 = make_tile_desc(smem_u32(y_smem + (2 * st + 1) * kTileBytes), false);
                const uint32_t d1 = t_tmem + (uint32_t)(128 * b), d2 = d1 + 64u;
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(d1, x1_desc + (uint64_t)(kk * 2), y1 + (uint64_t)(kk * 2), p.idesc_t, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(d2, x2_desc + (uint64_t)(kk * 2), y2 + (uint64_t)(kk * 2), p.idesc_t, kk > 0 ? 1u : 0u);
                    tc_commit(&bars->t_full[g][b]);
                    if (j == n - 1) tc_commit(&bars->x_empty[g]);      // the last reads of the X pair
                }
                __syncwarp();
            }
            t0 += n;
            ++i_no;
        }
        // All MMAs issued by the elected lane (the same one every time) must have retired before TMEM is freed.
        if (elect_one()) {
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else if (role == 2) {
        // ------------------------------------------------------------ issuer of dV += P^T dO_r and dK += dS^T Q_r
        int t0 = 0, i_no = 0;
        bool ok = true;
        while (ok) {
            // the column's entry from the producer (columns without blocks never get here)
            const int slot = i_no & (kBwdColItems - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->col_full[g][slot], (uint32_t)(i_no / kBwdColItems) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int n = bars->cols[g][slot].z;
            if (n == 0) break;                      // no more columns
            // the accumulators are free once the column before has been read out
            if (i_no > 0) ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_empty[g], (uint32_t)(i_no - 1) & 1u, abort_flag, p.status)) != 0;
            for (int j = 0; ok && j < n; ++j) {
                const int t = t0 + j, st = t & (kBwdColRing - 1), b = t & 1;
                // (the block's Y stage has landed: its T products, which the operand tiles come from, waited for it)
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->op_full[g][b], (uint32_t)(t >> 1) & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                // A = operand tile in tensor memory, B = a Y tile with N = head_dim contiguous
                const uint64_t bq = make_tile_desc(smem_u32(y_smem + (2 * st) * kTileBytes), true);
                const uint64_t bdo = make_tile_desc(smem_u32(y_smem + (2 * st + 1) * kTileBytes), true);
                const uint32_t a_p = pt_tmem + (uint32_t)(32 * b), a_ds = ds_tmem + (uint32_t)(32 * b);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16_ts(dv_tmem, a_p + (uint32_t)(8 * kk), bdo + (uint64_t)(kk * (2048 >> 4)), p.idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16_ts(dk_tmem, a_ds + (uint32_t)(8 * kk), bq + (uint64_t)(kk * (2048 >> 4)), p.idesc_acc, (j > 0 || kk > 0) ? 1u : 0u);
                    tc_commit(&bars->y_free[g][st]);        // the Y stage is free
                    tc_commit(&bars->op_free[g][b]);        // the operand buffers are free
                    if (j == n - 1) tc_commit(&bars->o_full[g]);
                }
                __syncwarp();
            }
            t0 += n;
            ++i_no;
        }
        if (elect_one()) {
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ compute warpgroup
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int half = (warp >> 2) & 1;           // this warp's half of a block's query columns: 32 * half .. + 31
        const int q4 = lane & 3;                    // position in the quad: columns 32 * half + 8u + 2 * q4 + {0, 1}, u < 4
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows (keys) of the 64-row tile: row_a, row_a + 8
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const bool masked_op = MASKED && (p.causal != 0 || p.kpm != nullptr || p.quadrants != 0);
        const float c2 = p.scale_log2, sc = p.scale;
        const uint64_t c2p = f2_pack(c2, c2), scp = f2_pack(sc, sc);
        int t0 = 0, i_no = 0;
        bool ok = true;
        while (ok) {
            // The column's entry from the producer (which walks the work items; columns without blocks never get here).
            const int slot = i_no & (kBwdColItems - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->col_full[g][slot], (uint32_t)(i_no / kBwdColItems) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int4 item = bars->cols[g][slot];
            const int n = item.z;
            if (n == 0) break;                      // no more columns
            const size_t out_a = ((size_t)item.x * p.seq_k + (size_t)item.y * kTile + row_a) * kTile;
            const size_t out_b = out_a + (size_t)8 * kTile;
            {
                const uint8_t* kpm_row = (MASKED && p.kpm) ? p.kpm + (size_t)(item.x / p.kpm_div) * p.kpm_stride : nullptr;
                const int pos_a = item.y * kTile + row_a;        // key position of row a (row b: + 8)
                // a whole key row is padding or not
                bool pad_a = false, pad_b = false;
                if (MASKED && kpm_row) { pad_a = kpm_row[pos_a] != 0; pad_b = kpm_row[pos_a + 8] != 0; }
                for (int j = 0; ok && j < n; ++j) {
                    const int t = t0 + j, st = t & (kBwdColRing - 1), b = t & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_full[g][b], (uint32_t)(t >> 1) & 1u, abort_flag, p.status)) != 0;
                    // (complete already: the block's T products waited for the stage; observed here for the statistics)
                    if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[g][st], (uint32_t)(t >> 2) & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r1[16], r2[16];
                    tc_ld_16x256b_x4(t_tmem + lane_field + (uint32_t)(128 * b + 32 * half), r1);
                    tc_ld_16x256b_x4(t_tmem + lane_field + (uint32_t)(128 * b + 64 + 32 * half), r2);
                    const BlockDesc d = bars->descs[g][st];         // the block's descriptor, from the producer
                    const int q0 = d.row() * kTile + 32 * half + 2 * q4;        // query position of column u = 0, e = 0
                    // Masked positions (bit 2u + e of the low byte: row a, column 32 half + 8u + 2 q4 + e; bits 8-15: row b):
                    // padded key rows, queries before the key (causal), quadrants outside a block-32 layout (the lane's
                    // rows are keys: column half quad / 2; the warp's query columns lie in the row half `half`).
                    uint32_t mask = 0u;
                    if (MASKED && masked_op) {
                        if (p.quadrants && !(((uint32_t)d.idx >> (2 * half + (quad >> 1))) & 1u)) mask = 0xFFFFu;
                        if (pad_a) mask |= 0x00FFu;
                        if (pad_b) mask |= 0xFF00u;
                        if (p.causal && pos_a + 8 > d.row() * kTile + 32 * half) {
#pragma unroll
                            for (int u = 0; u < 4; ++u)
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int qpos = q0 + 8 * u + e;
                                    if (pos_a > qpos) mask |= 1u << (2 * u + e);
                                    if (pos_a + 8 > qpos) mask |= 1u << (8 + 2 * u + e);
                                }
                        }
                    }
                    // (lse2, D) of this lane's 16 query columns, brought into the block's stage by the producer:
                    // cs[u] = those of columns 32 half + 8u + 2 q4 and + 1
                    float4 cs[4];
                    {
                        const float4* src = reinterpret_cast<const float4*>(st_smem + st * kBwdStatBytes) + 16 * half + q4;
#pragma unroll
                        for (int u = 0; u < 4; ++u) cs[u] = src[4 * u];        // 8 columns = 4 float4 apart
                    }
                    tc_wait_ld();
                    release_accumulator(&bars->t_empty[g][b], lane);    // T is in registers: its buffer may be overwritten
                    // Are the operand buffers free (accumulations of block t - 2 retired)?  Tested now, needed later.
                    const bool op_free = t < 2 || mbar_test(&bars->op_free[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u);
                    // wp / wd [2u + h]: columns 32 half + 8u + 2 q4 + {0, 1} of row a (h = 0) / row b (h = 1) of P^T / dS^T:
                    // the register order of the 16x128b store
                    uint32_t wp[8], wd[8];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint64_t nl = f2_pack(-cs[u].x, -cs[u].z);                 // -lse2 of the two columns
                        const uint64_t nd = f2_pack(-cs[u].y * sc, -cs[u].w * sc);       // -D * scale
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint64_t e2 = f2_fma(f2_pack(__uint_as_float(r1[4 * u + 2 * h]), __uint_as_float(r1[4 * u + 2 * h + 1])), c2p, nl);
                            float e0, e1;
                            f2_unpack(e2, e0, e1);
                            e0 = attn_exp2(e0); e1 = attn_exp2(e1);
                            if (MASKED && masked_op) {
                                if ((mask >> (8 * h + 2 * u)) & 1u) e0 = 0.f;
                                if ((mask >> (8 * h + 2 * u + 1)) & 1u) e1 = 0.f;
                            }
                            const uint64_t g2 = f2_fma(f2_pack(__uint_as_float(r2[4 * u + 2 * h]), __uint_as_float(r2[4 * u + 2 * h + 1])), scp, nd);
                            float d0, d1;
                            f2_unpack(f2_mul(f2_pack(e0, e1), g2), d0, d1);
                            wp[2 * u + h] = pack2<BF16>(e0, e1);
                            wd[2 * u + h] = pack2<BF16>(d0, d1);
                        }
                    }
                    // the operand buffers must have been read by the MMAs that used them last (those of block t - 2)
                    if (!__all_sync(0xffffffffu, op_free) &&
                        !__all_sync(0xffffffffu, mbar_wait(&bars->op_free[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status))) { ok = false; break; }
                    tc_fence_after();
                    tc_st_16x128b_x4(pt_tmem + lane_field + (uint32_t)(32 * b + 16 * half), wp);
                    tc_st_16x128b_x4(ds_tmem + lane_field + (uint32_t)(32 * b + 16 * half), wd);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->op_full[g][b]);
                }
                t0 += n;
                if (!ok) break;
                // ---- end of the column: dV and dK to global memory
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                uint32_t av[16], ak[16];            // this warp's 32 head-dim columns of dV and dK
                tc_ld_16x256b_x4(dv_tmem + lane_field + (uint32_t)(32 * half), av);
                tc_ld_16x256b_x4(dk_tmem + lane_field + (uint32_t)(32 * half), ak);
                tc_wait_ld();
                release_accumulator(&bars->o_empty[g], lane);          // the next column may overwrite the accumulators
#pragma unroll
                for (int a = 0; a < 2; ++a) {
                    uint16_t* out = a == 0 ? p.out0 : p.out1;
                    const uint32_t (&acc)[16] = a == 0 ? av : ak;
                    uint32_t ta[4], tb[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        ta[u] = pack2<BF16>(__uint_as_float(acc[4 * u]), __uint_as_float(acc[4 * u + 1]));
                        tb[u] = pack2<BF16>(__uint_as_float(acc[4 * u + 2]), __uint_as_float(acc[4 * u + 3]));
                    }
                    quad_transpose(ta, q4);         // now columns 32 half + 8 * q4 .. + 7 of the row
                    quad_transpose(tb, q4);
                    *reinterpret_cast<uint4*>(out + out_a + 32 * half + 8 * q4) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                    *reinterpret_cast<uint4*>(out + out_b + 32 * half + 8 * q4) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                }
                ++i_no;
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 16) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}
