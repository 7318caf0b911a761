// fp16 GEMM on CTA pairs: one 256 x BN output tile per pair of SMs (tcgen05.mma.cta_group::2).
//
// Same roles as the one-CTA kernel (TMA producer warp, MMA warp, eight epilogue warps, two
// accumulators in TMEM), but the two CTAs of a cluster share every MMA: each loads its own 128
// rows of A and its own half of the B tile, the even CTA issues a 256 x BN x 16 instruction that
// reads both shared memories, and each CTA finishes the 128 rows that land in its own TMEM.
// Per SM that is 32 KB of operands per 64-deep k-block instead of 48 KB, which takes the main
// loop off the L2 -> shared-memory bandwidth limit of one SM.
//
// Synchronisation across the pair:
//   full[s]        lives in the even CTA; both producers' TMA loads complete on it;
//   empty[s]       one per CTA; the MMA warp's commit is multicast to both;
//   tmem_full[a]   one per CTA; multicast commit after the last k-block of a tile;
//   tmem_empty[a]  lives in the even CTA; the 16 epilogue warps of the pair arrive on it.
// No multicast loads are used: every byte is fetched once, by the CTA that owns it.
//
// Finished tiles leave through shared memory: each epilogue warp stages 32 rows x 64 columns (4 KB, in
// the 128-byte swizzle a tensor map expects) and one lane issues a bulk tensor store, instead of every
// lane writing 16-byte pieces of 32 different rows.  Ragged edges are clipped by the tensor map.
#include "gemm_common.cuh"

#include <cooperative_groups.h>

namespace b200ml {

using namespace gemm;

namespace {

template <int BN>
struct PairSmem {
    static constexpr int B_TILE_BYTES = (BN / 2) * BK * 2;  // this CTA's half of the B tile
    static constexpr int STAGE_BYTES = A_TILE_BYTES + B_TILE_BYTES;
    static constexpr int STAGES = (BN == 256) ? 6 : 8;
    static constexpr int OUT_BYTES = EPI_WARPS * 32 * 128;  // one 32-row x 128-byte staging tile per epilogue warp
    static constexpr int BAR_BYTES = (2 * STAGES + 4) * 8 + 16;
    static constexpr int TOTAL = STAGES * STAGE_BYTES + OUT_BYTES + BAR_BYTES + 1024;
};

template <int BN, bool B_MN, bool TMA_OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                     const __grid_constant__ CUtensorMap tmap_c, const GemmArgs args) {
    using S = PairSmem<BN>;
    constexpr int STAGES = S::STAGES;
    constexpr int HALF_N = BN / 2;
    constexpr uint32_t TMEM_COLS = 2 * BN;
    constexpr uint32_t IDESC = ptx::make_idesc_f16(2 * BM, BN, 0, B_MN ? 1 : 0);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* out_stage = smem + STAGES * S::STAGE_BYTES;  // 1024-byte aligned: every stage is a multiple of 1 KB
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(out_stage + S::OUT_BYTES);
    uint64_t* empty_bar = full_bar + STAGES;
    uint64_t* tmem_full_bar = empty_bar + STAGES;
    uint64_t* tmem_empty_bar = tmem_full_bar + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tmem_empty_bar + 2);

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();  // 0: leader (issues the MMAs), 1: peer
    const int pair = blockIdx.x >> 1;
    const int num_pairs = gridDim.x >> 1;
    const int num_kb = (args.k + BK - 1) / BK;

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        if (TMA_OUT) ptx::prefetch_tensormap(&tmap_c);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < STAGES; ++s) {
                ptx::mbar_init(&full_bar[s], 1);   // the leader's producer arms it for both CTAs' bytes
                ptx::mbar_init(&empty_bar[s], 1);  // one multicast commit
            }
            for (int a = 0; a < 2; ++a) {
                ptx::mbar_init(&tmem_full_bar[a], 1);
                ptx::mbar_init(&tmem_empty_bar[a], 2 * EPI_WARPS);  // epilogue warps of both CTAs
            }
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc_pair(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // both CTAs' barriers exist before any remote arrive or load completion
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // A constant B (weights) does not depend on the kernel in front of this one: the B halves of the first tile's first
    // stages are requested before the dependency wait and stream in under the predecessor's tail.  The stages are fresh
    // (their empty barriers pass), the A halves and everything else follow after the wait.
    const int early = (args.b_early && pair < args.num_tiles) ? (num_kb < STAGES ? num_kb : STAGES) : 0;
    if (warp == 0 && early > 0) {
        if (ptx::elect_one()) {
            const int rest = pair / args.tiles_m;
            const int nt = rest % args.tiles_n;
            const int batch = rest / args.tiles_n;
            const int bi = batch % args.batch_inner, bo = batch / args.batch_inner;
            const int n0 = nt * BN + static_cast<int>(cta) * HALF_N;
            for (int kb = 0; kb < early; ++kb) {
                uint8_t* sb = smem + kb * S::STAGE_BYTES + A_TILE_BYTES;
                const uint32_t bar = ptx::leader_addr(&full_bar[kb]);
                if (cta == 0) ptx::mbar_expect_tx(&full_bar[kb], 2 * S::STAGE_BYTES);
                if (B_MN) {
#pragma unroll
                    for (int j = 0; j < HALF_N / 64; ++j)
                        ptx::tma_load_4d_pair(sb + j * (64 * BK * 2), &tmap_b, bar, n0 + j * 64, kb * BK,
                                              bi * args.b_use_inner, bo * args.b_use_outer);
                } else {
                    ptx::tma_load_4d_pair(sb, &tmap_b, bar, kb * BK, n0, bi * args.b_use_inner, bo * args.b_use_outer);
                }
            }
        }
        __syncwarp();
    }
    pdl_wait();  // everything above overlaps the previous kernel's tail

    if (warp == 0) {
        // ------------------------------ TMA producer (both CTAs) ------------------------------
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < args.num_tiles; tile += num_pairs) {
                const int mt = tile % args.tiles_m;
                const int rest = tile / args.tiles_m;
                const int nt = rest % args.tiles_n;
                const int batch = rest / args.tiles_n;
                const int bi = batch % args.batch_inner;
                const int bo = batch / args.batch_inner;
                const int m0 = mt * (2 * BM) + static_cast<int>(cta) * BM;
                const int n0 = nt * BN + static_cast<int>(cta) * HALF_N;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
                        atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    uint8_t* sa = smem + stage * S::STAGE_BYTES;
                    uint8_t* sb = sa + A_TILE_BYTES;
                    const uint32_t bar = ptx::leader_addr(&full_bar[stage]);
                    const bool b_done = tile == pair && kb < early;  // requested before the dependency wait
                    if (cta == 0 && !b_done) ptx::mbar_expect_tx(&full_bar[stage], 2 * S::STAGE_BYTES);
                    ptx::tma_load_4d_pair(sa, &tmap_a, bar, kb * BK, m0, bi * args.a_use_inner, bo * args.a_use_outer);
                    if (b_done) {
                    } else if (B_MN) {
#pragma unroll
                        for (int j = 0; j < HALF_N / 64; ++j)
                            ptx::tma_load_4d_pair(sb + j * (64 * BK * 2), &tmap_b, bar, n0 + j * 64, kb * BK,
                                                  bi * args.b_use_inner, bo * args.b_use_outer);
                    } else {
                        ptx::tma_load_4d_pair(sb, &tmap_b, bar, kb * BK, n0, bi * args.b_use_inner,
                                              bo * args.b_use_outer);
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (leader CTA only) ------------------------------
        if (cta == 0 && ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int acc = 0;
            uint32_t acc_phase = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < args.num_tiles; tile += num_pairs) {
                if (!ptx::mbar_wait(&tmem_empty_bar[acc], acc_phase ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_MMA);
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + acc * BN;
                for (int kb = 0; kb < num_kb; ++kb) {
                    if (!ptx::mbar_wait(&full_bar[stage], phase)) {
                        atomicExch(args.status, DEV_TIMEOUT_MMA);
                        ok = false;
                        break;
                    }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(smem + stage * S::STAGE_BYTES);
                    const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        const uint64_t a_desc = ptx::make_smem_desc_sw128(a_addr + kk * (UMMA_K * 2), 16, 1024);
                        const uint64_t b_desc =
                            B_MN ? ptx::make_smem_desc_sw128(b_addr + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                 : ptx::make_smem_desc_sw128(b_addr + kk * (UMMA_K * 2), 16, 1024);
                        ptx::mma_f16_ss_pair(d_tmem, a_desc, b_desc, IDESC, (kb | kk) != 0 ? 1u : 0u);
                    }
                    ptx::mma_commit_pair(&empty_bar[stage], 3);  // frees the stage in both CTAs
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) break;
                ptx::mma_commit_pair(&tmem_full_bar[acc], 3);
                acc ^= 1;
                if (acc == 0) acc_phase ^= 1;
            }
        }
    } else {
        // ------------------------------ epilogue (both CTAs, own 128 rows) ------------------------------
        const int quarter = warp & 3;
        const int half = (warp - 2) >> 2;
        constexpr int WCOLS = BN / 2;
        constexpr int CHUNKS = WCOLS / 32;
        constexpr int GROUP = CHUNKS >= 2 ? 2 : 1;
        const int row_in_tile = static_cast<int>(cta) * BM + quarter * 32 + lane;
        int acc = 0;
        uint32_t acc_phase = 0;
        EpilogueParams ep;
        ep.flags = args.epilogue;
        ep.alpha = args.alpha;
        ep.bias_scale = args.bias_scale;
        ep.residual_scale = args.residual_scale;
        for (int tile = pair; tile < args.num_tiles; tile += num_pairs) {
            const int mt = tile % args.tiles_m;
            const int rest = tile / args.tiles_m;
            const int nt = rest % args.tiles_n;
            const int batch = rest / args.tiles_n;
            const int bi = batch % args.batch_inner;
            const int bo = batch / args.batch_inner;
            const int row = mt * (2 * BM) + row_in_tile;
            const int n0 = nt * BN + half * WCOLS;
            if (!ptx::mbar_wait(&tmem_full_bar[acc], acc_phase)) {
                if (lane == 0) atomicExch(args.status, DEV_TIMEOUT_EPILOGUE);
                break;
            }
            ptx::tc_fence_after();
            __half* c_row = args.c + bo * args.c_so + bi * args.c_si + static_cast<int64_t>(row) * args.ldc;
            const __half* r_row = args.residual
                                      ? args.residual + bo * args.r_so + bi * args.r_si + static_cast<int64_t>(row) * args.ldr
                                      : nullptr;
            const bool row_ok = row < args.m;
            const bool vec = args.vec_ok != 0;
            const uint32_t t_base = tmem_base + acc * BN + half * WCOLS + (static_cast<uint32_t>(quarter * 32) << 16);
            if constexpr (TMA_OUT) {
                // 64 columns at a time: TMEM -> registers -> epilogue math -> swizzled staging tile -> bulk store
                static_assert(CHUNKS % 2 == 0, "the staged path moves two 32-column chunks per store");
                uint8_t* stage_row = out_stage + (warp - 2) * 4096 + lane * 128;
                const bool has_bias = (ep.flags & B200ML_EPI_BIAS) && args.bias != nullptr;
                const bool has_res = (ep.flags & B200ML_EPI_RESIDUAL) && r_row != nullptr;
#pragma unroll 1
                for (int c = 0; c < CHUNKS; c += 2) {
                    const int col0 = n0 + c * 32;
                    if (col0 >= args.n) break;  // warp-uniform
                    uint32_t r[2][32];
                    EpiloguePrefetch pf[2];
#pragma unroll
                    for (int u = 0; u < 2; ++u) ptx::tmem_ld_32x32b_x32(t_base + (c + u) * 32, r[u]);
                    if (row_ok) {
#pragma unroll
                        for (int u = 0; u < 2; ++u)
                            epilogue_prefetch_32(ep, pf[u], r_row, args.bias, col0 + u * 32, args.n, true);
                    }
                    ptx::tmem_ld_wait();
                    if (lane == 0) ptx::tma_store_wait_read<0>();  // the previous store has read the staging tile
                    __syncwarp();
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        uint4 o[4];
                        epilogue_pack_32(ep, r[u], pf[u], has_bias, has_res && row_ok, o);
#pragma unroll
                        for (int g = 0; g < 4; ++g)
                            *reinterpret_cast<uint4*>(stage_row + (((u * 4 + g) ^ (lane & 7)) << 4)) = o[g];
                    }
                    ptx::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        ptx::tma_store_4d(&tmap_c, out_stage + (warp - 2) * 4096, col0, mt * (2 * BM) + static_cast<int>(cta) * BM + quarter * 32, bi, bo);
                        ptx::tma_store_commit();
                    }
                }
            } else {
#pragma unroll 1
            for (int c = 0; c < CHUNKS; c += GROUP) {
                const int col0 = n0 + c * 32;
                if (col0 >= args.n) break;  // warp-uniform
                uint32_t r[GROUP][32];
                EpiloguePrefetch pf[GROUP];
#pragma unroll
                for (int u = 0; u < GROUP; ++u) ptx::tmem_ld_32x32b_x32(t_base + (c + u) * 32, r[u]);
                if (row_ok) {
#pragma unroll
                    for (int u = 0; u < GROUP; ++u)
                        epilogue_prefetch_32(ep, pf[u], r_row, args.bias, col0 + u * 32, args.n, vec);
                }
                ptx::tmem_ld_wait();
                if (row_ok) {
#pragma unroll
                    for (int u = 0; u < GROUP; ++u) {
                        if (col0 + u * 32 < args.n)
                            epilogue_store_32(ep, r[u], pf[u], c_row, r_row, args.bias, col0 + u * 32, args.n, vec);
                    }
                }
            }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::leader_addr(&tmem_empty_bar[acc]));
            acc ^= 1;
            if (acc == 0) acc_phase ^= 1;
        }
        if (TMA_OUT && lane == 0) ptx::tma_store_wait<0>();  // every bulk store of this warp has landed
    }

    // ------------------------------ teardown ------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync();  // neither CTA leaves while the other may still touch its barriers or shared memory
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            for (int i = 0; i < 200; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

template <int BN, bool B_MN, bool TMA_OUT>
int launch_pair_impl(const b200ml_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmArgs& args,
                cudaStream_t stream) {
    using S = PairSmem<BN>;
    auto kernel = gemm_f16_pair_kernel<BN, B_MN, TMA_OUT>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, S::TOTAL));
        configured[ctx->device & 63] = true;
    }
    const int max_pairs = ctx->sm_count / 2;
    const int pairs = args.num_tiles < max_pairs ? args.num_tiles : max_pairs;
    B200ML_CUDA(launch_pdl(kernel, dim3(2 * pairs), dim3(GEMM_THREADS), S::TOTAL, stream, ta, tb, tc, args));
    return check_launch("gemm_f16_pair");
}

template <int BN, bool B_MN>
int launch_pair(const b200ml_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, GemmArgs& args,
                cudaStream_t stream) {
    return args.tma_store ? launch_pair_impl<BN, B_MN, true>(ctx, ta, tb, tc, args, stream)
                          : launch_pair_impl<BN, B_MN, false>(ctx, ta, tb, tc, args, stream);
}

}  // namespace

// 256 x BN tiles on CTA pairs.  BN is 256 or 128; args.tiles_m / tiles_n / num_tiles are already in
// units of those tiles.  The B tensor map's box covers this CTA's half of the tile.
int gemm_f16_pair(const b200ml_ctx* ctx, const b200ml_gemm_params* p, GemmArgs& args, int bn, cudaStream_t stream) {
    CUtensorMap ta, tb, tc;
    int rc = make_tmap(ctx, &ta, p->a, p->k, p->m, p->lda, p->batch_inner, p->a_stride_inner, p->batch_outer,
                       p->a_stride_outer, BK, BM, "A");
    if (rc) return rc;
    // C leaves through bulk tensor stores (64 columns x 32 rows per store) when its rows are 16-byte aligned
    // and N is a whole number of 64-column pieces; otherwise the warps store their rows themselves.
    args.tma_store = 0;
    tc = ta;
    if (args.vec_ok && p->n % 64 == 0 && (p->batch_inner == 1 || p->c_stride_inner % 8 == 0) &&
        (p->batch_outer == 1 || p->c_stride_outer % 8 == 0)) {
        rc = make_tmap(ctx, &tc, p->c, p->n, p->m, p->ldc, p->batch_inner, p->c_stride_inner, p->batch_outer,
                       p->c_stride_outer, 64, 32, "C");
        if (rc) return rc;
        args.tma_store = 1;
    }
    if (p->b_layout == 1) {
        rc = make_tmap(ctx, &tb, p->b, p->k, p->n, p->ldb, p->batch_inner, p->b_stride_inner, p->batch_outer,
                       p->b_stride_outer, BK, bn / 2, "B");
        if (rc) return rc;
        return bn == 256 ? launch_pair<256, false>(ctx, ta, tb, tc, args, stream)
                         : launch_pair<128, false>(ctx, ta, tb, tc, args, stream);
    }
    rc = make_tmap(ctx, &tb, p->b, p->n, p->k, p->ldb, p->batch_inner, p->b_stride_inner, p->batch_outer,
                   p->b_stride_outer, 64, BK, "B");
    if (rc) return rc;
    return bn == 256 ? launch_pair<256, true>(ctx, ta, tb, tc, args, stream)
                     : launch_pair<128, true>(ctx, ta, tb, tc, args, stream);
}

}  // namespace b200ml
