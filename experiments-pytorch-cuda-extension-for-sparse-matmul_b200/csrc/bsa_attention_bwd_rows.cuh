// Fused attention backward, dQ by block rows, head dim 64: two independent pipelines per CTA.
// Included by bsa_attention_bwd.cu inside its anonymous namespace (it uses BwdParams and the helpers
// of bsa_tc_common.cuh).
//
// The same organisation as the forward kernel for head dim 64: a pipeline is a producer warp, an
// issuer warp and a compute warpgroup with their own shared-memory tiles (X = (Q_r, dO_r), two stages
// of Y = (K_c, V_c)), their own tensor-memory buffers and barriers, and walks its own block rows
// (pipeline number = 2 * CTA + g of 2 * grid pipelines); two CTAs share an SM, so four block rows are
// in flight per SM, each at its own point of its row.  (The general kernel lets two compute groups
// share a row with alternate blocks, with in-order issuers and one producer for both: every
// hand-over between the groups serialises the CTA.)
//
// Per block (r, c):  T1 = Q_r K_c^T = S,  T2 = dO_r V_c^T = dP  (both into tensor memory),
//   dS = scale * exp2(c2 * S - lse2_r) o (dP - D_r)  packed to 16 bits into tensor memory,
//   dQ_r += dS K_c  with the A operand (dS) read from tensor memory.
// Tensor memory of a pipeline (128 columns; an M = 64 accumulator occupies lanes 0-15 of each
// 32-lane quarter, a second one fits into lanes 16-31 of the same columns):
//   columns   0 ..  63   lanes 0-15: dQ accumulator       lanes 16-31: T1
//   columns  64 .. 127   lanes 0-15: dS buffers 0, 1 (32 columns each)   lanes 16-31: T2
// (a TMEM A operand is used at lane offset 0 with its D at lane offset 0 only).
//   warps 0, 2   producer of pipeline 0, 1: the row's X pair, then every block's Y pair (stage t & 1)
//   warps 1, 3   issuer: T1 and T2 of block t, then the accumulation of block t - 1
//   warps 4-7, 8-11   compute warpgroup; at the end of the row dQ goes to global memory.
constexpr int kBwdRowRing = 8;
struct __align__(16) BwdRowBarriers {
    uint64_t x_full[2], x_empty[2];             // [pipeline]
    uint64_t y_full[2][2], acc_done[2][2];      // [pipeline][block & 1]: acc_done = the Y stage and the dS buffer are free
    uint64_t t_full[2], t_empty[2];
    uint64_t ds_full[2][2];
    uint64_t o_full[2], o_empty[2];
    uint64_t drain;
    uint32_t tmem_base;
    int abort_flag;
    BlockDesc descs[2][2];                      // [pipeline][block & 1]: written by the producer for the compute warps
    uint64_t row_full[2][kBwdRowRing];          // [pipeline][row & 7]: the row's entry in `rows` is valid
    int4 rows[2][kBwdRowRing];                  // (batch entry, block row, blocks, -): written by the producer; blocks = 0: no more rows
};
constexpr int kBwdRowTiles = 6;                 // per pipeline: Q, dO, (K, V) x 2

template <bool BF16, bool MASKED>
__global__ void __launch_bounds__(12 * 32, 2)
attention_backward_rows_pipes_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_do,
                                     const __grid_constant__ CUtensorMap map_k, const __grid_constant__ CUtensorMap map_v,
                                     const BwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    BwdRowBarriers* bars = reinterpret_cast<BwdRowBarriers*>(smem + 2 * kBwdRowTiles * kTileBytes);
    int* abort_flag = &bars->abort_flag;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = warp < 4 ? warp >> 1 : (warp - 4) >> 2;          // pipeline of this warp
    uint8_t* x_smem = smem + g * kBwdRowTiles * kTileBytes;        // Q_r, dO_r
    uint8_t* y_smem = x_smem + 2 * kTileBytes;                     // [stage][K_c, V_c]

    if (threadIdx.x == 0) {
        for (int i = 0; i < 2; ++i) {
            mbar_init(&bars->x_full[i], 1); mbar_init(&bars->x_empty[i], 1);
            mbar_init(&bars->t_full[i], 1); mbar_init(&bars->t_empty[i], 4);
            for (int s = 0; s < 2; ++s) {
                mbar_init(&bars->y_full[i][s], 1); mbar_init(&bars->acc_done[i][s], 1);
                mbar_init(&bars->ds_full[i][s], 4);
            }
            mbar_init(&bars->o_full[i], 1); mbar_init(&bars->o_empty[i], 4);
            for (int s = 0; s < kBwdRowRing; ++s) mbar_init(&bars->row_full[i][s], 1);
        }
        mbar_init(&bars->drain, 2);
        bars->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_shared();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;"
                     ::"r"(smem_u32(&bars->tmem_base)), "r"(256u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *(volatile uint32_t*)&bars->tmem_base;
    const uint32_t dq_tmem = tmem_base + (uint32_t)(g * 128);              // dQ: lanes 0-15 of columns 0 .. 63
    const uint32_t t1_tmem = dq_tmem + (16u << 16);                        // T1: lanes 16-31 of columns 0 .. 63
    const uint32_t t2_tmem = t1_tmem + 64u;                                // T2: lanes 16-31 of columns 64 .. 127
    const uint32_t ds_tmem = dq_tmem + 64u;                                // dS buffer b: lanes 0-15 of columns 64 + 32 b ..
    const int walker = 2 * (int)blockIdx.x + g, walkers = 2 * (int)gridDim.x;

    if (warp == 0 || warp == 2) {
        // ------------------------------------------------------------ producer
        int t0 = 0, i_no = 0;                       // blocks and non-empty rows before the current row
        bool ok = true;
        Cursor cur;
        cur.init_as(p, walker, walkers, 0, true);
        BlockDesc pre = cur.valid() ? load_first_chunk(p.blocks, cur.first, cur.count, lane) : BlockDesc{0, 0};
        while (ok && cur.valid()) {
            BlockDesc pre_next{0, 0};
            if (cur.has_next()) pre_next = load_first_chunk(p.blocks, cur.next_first(), cur.next_count(), lane);
            const int n = cur.count;
            if (n == 0) {
                // a row without blocks: zero gradient rows (the other roles never see the row)
                const size_t row0 = (size_t)cur.z * p.seq_q + (size_t)cur.g * kTile;
                for (int c = lane; c < kTile * kTile / 8; c += 32)
                    reinterpret_cast<uint4*>(p.out0 + row0 * kTile)[c] = make_uint4(0u, 0u, 0u, 0u);
            } else {
                // the X pair once the last T products of the row before have retired
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_empty[g], ((uint32_t)i_no & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (ok && elect_one()) {
                    // The row's entry for the issuer and the compute warps: they are at most two rows behind
                    // (the wait above: the compute warps have taken the T tiles of the block before that row's last).
                    bars->rows[g][i_no & (kBwdRowRing - 1)] = make_int4(cur.z, cur.g, n, 0);
                    mbar_arrive(&bars->row_full[g][i_no & (kBwdRowRing - 1)]);
                    mbar_expect_tx(&bars->x_full[g], (uint32_t)(2 * kTileBytes));
                    tma_load_3d(x_smem, &map_q, &bars->x_full[g], 0, cur.g * kTile, cur.z);
                    tma_load_3d(x_smem + kTileBytes, &map_do, &bars->x_full[g], 0, cur.g * kTile, cur.z);
                }
                __syncwarp();
                DescWindow win;
                win.begin(p.blocks, cur.first, cur.count, pre, lane);
                for (int j = 0; ok && j < n; ++j) {
                    const BlockDesc desc = win.get(p.blocks, cur.first, cur.count, j, lane);
                    const int col = desc.col();
                    const int t = t0 + j, st = t & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->acc_done[g][st], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status)) != 0;
                    if (ok && elect_one()) {
                        bars->descs[g][st] = desc;      // for the compute warps; the slot is free like the stage
                        mbar_expect_tx(&bars->y_full[g][st], (uint32_t)(2 * kTileBytes));
                        tma_load_3d(y_smem + (2 * st) * kTileBytes, &map_k, &bars->y_full[g][st], 0, col * kTile, cur.z);
                        tma_load_3d(y_smem + (2 * st + 1) * kTileBytes, &map_v, &bars->y_full[g][st], 0, col * kTile, cur.z);
                    }
                    __syncwarp();
                }
                t0 += n;
                ++i_no;
            }
            pre = pre_next;
            cur.advance();
        }
        if (ok && elect_one()) {                    // no more rows
            bars->rows[g][i_no & (kBwdRowRing - 1)] = make_int4(0, 0, 0, 0);
            mbar_arrive(&bars->row_full[g][i_no & (kBwdRowRing - 1)]);
        }
        __syncwarp();
        if (lane == 0 && *(volatile int*)abort_flag) {
            let_copies_land();      // (issued by this warp; see the helper)
        }
        __syncwarp();
    } else if (warp == 1 || warp == 3) {
        // ------------------------------------------------------------ issuer
        // Order within a row: T1 and T2 of block t, then the accumulation of block t - 1; the row's last
        // accumulation follows, before the next row's first products (which would otherwise keep the end of
        // this row -- the compute warps wait for the last accumulation to read dQ out -- behind the arrival
        // of the next row's X pair).  The events come in this order: T(t - 1) is in the compute warps'
        // registers when they start on block t - 1, their dS(t - 1) is complete when they are done with it.
        const uint64_t x1_desc = make_tile_desc(smem_u32(x_smem), false);
        const uint64_t x2_desc = make_tile_desc(smem_u32(x_smem + kTileBytes), false);
        int t0 = 0, i_no = 0;
        bool ok = true;
        auto issue_acc = [&](int t, int row, bool first, bool last) -> bool {      // dQ (+)= dS K of block t
            const int b = t & 1;
            // the accumulator is free once the row before has been read out
            if (first && row > 0 &&
                !__all_sync(0xffffffffu, mbar_wait(&bars->o_empty[g], (uint32_t)(row - 1) & 1u, abort_flag, p.status)))
                return false;
            if (!__all_sync(0xffffffffu, mbar_wait(&bars->ds_full[g][b], (uint32_t)(t >> 1) & 1u, abort_flag, p.status))) return false;
            tc_fence_after();
            // A = dS in tensor memory, B = the K tile of the block's stage with N = head_dim contiguous
            const uint64_t db = make_tile_desc(smem_u32(y_smem + (2 * b) * kTileBytes), true);
            const uint32_t a = ds_tmem + (uint32_t)(32 * b);
            if (elect_one()) {
#pragma unroll
                for (int kk = 0; kk < kTile / 16; ++kk)
                    tc_mma_f16_ts(dq_tmem, a + (uint32_t)(8 * kk), db + (uint64_t)(kk * (2048 >> 4)), p.idesc_acc,
                                  (!first || kk > 0) ? 1u : 0u);
                tc_commit(&bars->acc_done[g][b]);       // the Y stage and the dS buffer are free
                if (last) tc_commit(&bars->o_full[g]);
            }
            __syncwarp();
            return true;
        };
        while (ok) {
            // the row's entry from the producer (rows without blocks never get here)
            const int slot = i_no & (kBwdRowRing - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->row_full[g][slot], (uint32_t)(i_no / kBwdRowRing) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int n = bars->rows[g][slot].z;
            if (n == 0) break;                      // no more rows
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->x_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
            for (int j = 0; ok && j < n; ++j) {
                const int t = t0 + j, st = t & 1;
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->y_full[g][st], (uint32_t)(t >> 1) & 1u, abort_flag, p.status)) != 0;
                if (ok) ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_empty[g], ((uint32_t)t & 1u) ^ 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                const uint64_t y1 = make_tile_desc(smem_u32(y_smem + (2 * st) * kTileBytes), false);
                const uint64_t y2 = make_tile_desc(smem_u32(y_smem + (2 * st + 1) * kTileBytes), false);
                if (elect_one()) {
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(t1_tmem, x1_desc + (uint64_t)(kk * 2), y1 + (uint64_t)(kk * 2), p.idesc_t, kk > 0 ? 1u : 0u);
#pragma unroll
                    for (int kk = 0; kk < kTile / 16; ++kk)
                        tc_mma_f16(t2_tmem, x2_desc + (uint64_t)(kk * 2), y2 + (uint64_t)(kk * 2), p.idesc_t, kk > 0 ? 1u : 0u);
                    tc_commit(&bars->t_full[g]);
                    if (j == n - 1) tc_commit(&bars->x_empty[g]);      // the last reads of the X pair
                }
                __syncwarp();
                if (j >= 1) ok = issue_acc(t - 1, i_no, j == 1, false);
            }
            if (ok) ok = issue_acc(t0 + n - 1, i_no, n == 1, true);
            t0 += n;
            ++i_no;
        }
        // All MMAs issued by the elected lane (the same one every time) must have retired before TMEM is freed.
        if (elect_one()) {
            tc_commit(&bars->drain);
            mbar_wait(&bars->drain, 0, abort_flag, p.status);
        }
        __syncwarp();
    } else {
        // ------------------------------------------------------------ compute warpgroup
        const int quad = warp & 3;                  // TMEM sub-partition this warp may read
        const int q4 = lane & 3;                    // position in the quad: columns 8u + 2 * q4 + {0, 1}
        const int row_a = quad * 16 + (lane >> 2);  // this lane's two rows of the 64-row tile: row_a, row_a + 8
        const uint32_t lane_field = (uint32_t)(quad * 32) << 16;
        const bool masked_op = MASKED && (p.causal != 0 || p.kpm != nullptr || p.quadrants != 0);
        const float c2 = p.scale_log2, sc = p.scale;
        const uint64_t c2p = f2_pack(c2, c2), scp = f2_pack(sc, sc);
        int t0 = 0, i_no = 0;
        bool ok = true;
        // Statistics of this lane's two query rows of block row `z, r`: (lse in log2 units, or +inf for a row
        // without scores; D = sum_d dO_d O_d).  The four lanes of a quad take 16 head-dim columns each and two
        // shuffles add the parts; the kernel by columns reads the pairs from `stats_out`.
        auto row_stats = [&](int z, int r, float2& sa, float2& sb) {
            const size_t row_i = (size_t)z * p.seq_q + (size_t)r * kTile + row_a;
            float d_a = dot16<BF16>(p.o + row_i * kTile + 16 * q4, p.dout + row_i * kTile + 16 * q4);
            float d_b = dot16<BF16>(p.o + (row_i + 8) * kTile + 16 * q4, p.dout + (row_i + 8) * kTile + 16 * q4);
            const float l_a = p.lse[row_i], l_b = p.lse[row_i + 8];
            d_a += __shfl_xor_sync(0xffffffffu, d_a, 1); d_a += __shfl_xor_sync(0xffffffffu, d_a, 2);
            d_b += __shfl_xor_sync(0xffffffffu, d_b, 1); d_b += __shfl_xor_sync(0xffffffffu, d_b, 2);
            sa = make_float2(l_a == -INFINITY ? INFINITY : l_a * kLog2e, d_a);
            sb = make_float2(l_b == -INFINITY ? INFINITY : l_b * kLog2e, d_b);
            if (q4 == 0) { p.stats_out[row_i] = sa; p.stats_out[row_i + 8] = sb; }
        };
        bool have_stats = false;                    // the statistics of the next row were computed at the end of the row before
        float2 nst_a = make_float2(0.f, 0.f), nst_b = nst_a;
        while (ok) {
            // The row's entry from the producer (which walks the work items; rows without blocks never get here).
            const int slot = i_no & (kBwdRowRing - 1);
            ok = __all_sync(0xffffffffu, mbar_wait(&bars->row_full[g][slot], (uint32_t)(i_no / kBwdRowRing) & 1u, abort_flag, p.status)) != 0;
            if (!ok) break;
            const int4 row = bars->rows[g][slot];
            const int n = row.z;
            if (n == 0) break;                      // no more rows
            const size_t out_a = ((size_t)row.x * p.seq_q + (size_t)row.y * kTile + row_a) * kTile;
            const size_t out_b = out_a + (size_t)8 * kTile;
            {
                const uint8_t* kpm_row = (MASKED && p.kpm) ? p.kpm + (size_t)(row.x / p.kpm_div) * p.kpm_stride : nullptr;
                const int pos_a = row.y * kTile + row_a;         // query position of row a (row b: + 8)
                float2 st_a = nst_a, st_b = nst_b;
                if (!have_stats) row_stats(row.x, row.y, st_a, st_b);
                // per row: -lse2 for the exponent and -D * scale for dS = P * (dP * scale - D * scale)
                const uint64_t nla = f2_pack(-st_a.x, -st_a.x), nlb = f2_pack(-st_b.x, -st_b.x);
                const uint64_t nda = f2_pack(-st_a.y * sc, -st_a.y * sc), ndb = f2_pack(-st_b.y * sc, -st_b.y * sc);
                for (int j = 0; ok && j < n; ++j) {
                    const int t = t0 + j, b = t & 1;
                    ok = __all_sync(0xffffffffu, mbar_wait(&bars->t_full[g], (uint32_t)t & 1u, abort_flag, p.status)) != 0;
                    if (!ok) break;
                    tc_fence_after();
                    uint32_t r1[32], r2[32];
                    tc_ld_16x256b_x8(t1_tmem + lane_field, r1);
                    tc_ld_16x256b_x8(t2_tmem + lane_field, r2);
                    // Masked positions (bit 2u + e of the low half: row a, column 8u + 2 q4 + e; high half: row b):
                    // above the diagonal, padded keys, quadrants outside a block-32 layout.  Computed while the
                    // products are on their way from tensor memory; the block's descriptor comes from the producer.
                    uint32_t mask = 0u;
                    if (MASKED && masked_op) {
                        const BlockDesc d = bars->descs[g][b];
                        const int col = d.col();
                        if (p.quadrants) {
                            const uint32_t present = (uint32_t)d.idx >> (2 * (quad >> 1));
                            if (!(present & 1u)) mask |= 0x00FF00FFu;
                            if (!(present & 2u)) mask |= 0xFF00FF00u;
                        }
                        const int k0 = col * kTile + 2 * q4;
                        if (p.causal && col * kTile + kTile - 1 > pos_a) {
#pragma unroll
                            for (int u = 0; u < 8; ++u)
#pragma unroll
                                for (int e = 0; e < 2; ++e) {
                                    const int kpos = k0 + 8 * u + e;
                                    if (kpos > pos_a) mask |= 1u << (2 * u + e);
                                    if (kpos > pos_a + 8) mask |= 1u << (16 + 2 * u + e);
                                }
                        }
                        if (kpm_row) {
#pragma unroll
                            for (int u = 0; u < 8; ++u) {
                                if (kpm_row[k0 + 8 * u]) mask |= 0x00010001u << (2 * u);
                                if (kpm_row[k0 + 8 * u + 1]) mask |= 0x00010001u << (2 * u + 1);
                            }
                        }
                    }
                    tc_wait_ld();
                    release_accumulator(&bars->t_empty[g], lane);       // T is in registers: the next block's products may run
                    // Is the dS buffer free (accumulation of block t - 2 retired)?  Tested now, needed after the arithmetic.
                    const bool ds_free = t < 2 || mbar_test(&bars->acc_done[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u);
                    // w[2u + h]: columns 8u + 2 q4 + {0, 1} of row a (h = 0) / row b (h = 1): the register order of the
                    // 16x128b store.  Per pair of columns: P = exp2(c2 * S - lse2), dS = P * (dP * scale - D * scale).
                    uint32_t w[16];
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
#pragma unroll
                        for (int h = 0; h < 2; ++h) {
                            const uint64_t e2 = f2_fma(f2_pack(__uint_as_float(r1[4 * u + 2 * h]), __uint_as_float(r1[4 * u + 2 * h + 1])),
                                                       c2p, h ? nlb : nla);
                            float e0, e1;
                            f2_unpack(e2, e0, e1);
                            e0 = attn_exp2(e0); e1 = attn_exp2(e1);
                            if (MASKED && masked_op) {
                                if ((mask >> (16 * h + 2 * u)) & 1u) e0 = 0.f;
                                if ((mask >> (16 * h + 2 * u + 1)) & 1u) e1 = 0.f;
                            }
                            const uint64_t g2 = f2_fma(f2_pack(__uint_as_float(r2[4 * u + 2 * h]), __uint_as_float(r2[4 * u + 2 * h + 1])),
                                                       scp, h ? ndb : nda);
                            float d0, d1;
                            f2_unpack(f2_mul(f2_pack(e0, e1), g2), d0, d1);
                            w[2 * u + h] = pack2<BF16>(d0, d1);
                        }
                    }
                    // the dS buffer must have been read by the MMAs that used it last (those of block t - 2)
                    if (!__all_sync(0xffffffffu, ds_free) &&
                        !__all_sync(0xffffffffu, mbar_wait(&bars->acc_done[g][b], ((uint32_t)(t >> 1) & 1u) ^ 1u, abort_flag, p.status))) { ok = false; break; }
                    tc_fence_after();
                    tc_st_16x128b_x8(ds_tmem + lane_field + (uint32_t)(32 * b), w);
                    tc_wait_st();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&bars->ds_full[g][b]);
                }
                t0 += n;
                if (!ok) break;
                // The next row's statistics while this row's last accumulation is in flight (their loads would
                // otherwise be waited for at the start of the next row, with its first products ready), if the
                // producer has posted the row already -- it is one to two rows ahead.
                {
                    const int next = (i_no + 1) & (kBwdRowRing - 1);
                    have_stats = __all_sync(0xffffffffu, mbar_test(&bars->row_full[g][next], (uint32_t)((i_no + 1) / kBwdRowRing) & 1u)) != 0;
                    if (have_stats) {
                        const int4 nrow = bars->rows[g][next];
                        have_stats = nrow.z > 0;
                        if (have_stats) row_stats(nrow.x, nrow.y, nst_a, nst_b);
                    }
                }
                // ---- end of the row: dQ to global memory
                ok = __all_sync(0xffffffffu, mbar_wait(&bars->o_full[g], (uint32_t)i_no & 1u, abort_flag, p.status)) != 0;
                if (!ok) break;
                tc_fence_after();
                uint32_t acc[2][16];
                tc_ld_16x256b_x4(dq_tmem + lane_field, acc[0]);
                tc_ld_16x256b_x4(dq_tmem + lane_field + 32u, acc[1]);
                tc_wait_ld();
                release_accumulator(&bars->o_empty[g], lane);          // the next row's accumulation may overwrite dQ
#pragma unroll
                for (int hc = 0; hc < 2; ++hc) {
                    uint32_t ta[4], tb[4];
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        ta[u] = pack2<BF16>(__uint_as_float(acc[hc][4 * u]), __uint_as_float(acc[hc][4 * u + 1]));
                        tb[u] = pack2<BF16>(__uint_as_float(acc[hc][4 * u + 2]), __uint_as_float(acc[hc][4 * u + 3]));
                    }
                    quad_transpose(ta, q4);         // now columns 32 hc + 8 * q4 .. + 7 of the row
                    quad_transpose(tb, q4);
                    *reinterpret_cast<uint4*>(p.out0 + out_a + 32 * hc + 8 * q4) = make_uint4(ta[0], ta[1], ta[2], ta[3]);
                    *reinterpret_cast<uint4*>(p.out0 + out_b + 32 * hc + 8 * q4) = make_uint4(tb[0], tb[1], tb[2], tb[3]);
                }
                ++i_no;
            }
        }
    }

    // ---------------------------------------------------------------- teardown
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(256u) : "memory");
    }
}
