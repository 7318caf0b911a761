// fp16 GEMM whose epilogue also applies LayerNorm over the output row:
//     Y = LayerNorm(act(alpha * A.B + bias) + residual) * gamma + beta
// for outputs of up to 1024 columns.  One cluster of N / 256 CTAs covers a 128-row block of the whole
// output width; each CTA computes a 128 x 256 tile exactly like the one-CTA GEMM (TMA ring -> tcgen05.mma
// -> TMEM), then the CTAs of the cluster exchange per-row partial sums through distributed shared
// memory (sum and sum of squares in fp32), and normalise their own columns.  The finished
// pre-normalisation row is parked in TMEM (fp32) between the two passes, so nothing is re-read from memory.
// This removes the separate LayerNorm kernel (one read and one write of the activation) behind the
// attention output projection and the second FFN matrix product.
// The residual comes in the same way it goes out: once the main loop's loads are issued, the producer turns the
// next two pipeline stages into sixteen 32-row x 64-column tiles of the residual (TMA, 128-byte swizzle), which land
// while the last products run; each lane then reads its row's 16-byte pieces from shared memory instead of issuing
// 16-byte loads to 32 different rows of global memory.
// The normalised rows leave through shared memory (the pipeline stages are free by then): each epilogue
// warp stages 32 rows x 64 columns in the 128-byte swizzle of a tensor map and one lane issues a bulk
// tensor store; rows past M are clipped by the tensor map.
#include "gemm_ln_epilogue.cuh"

namespace b200ml {

using namespace gemm;

namespace {

constexpr int LN_BN = 256;
constexpr int LN_STAGES = 4;
constexpr int LN_STAGE_BYTES = A_TILE_BYTES + LN_BN * BK * 2;
constexpr int LN_SMEM = LN_STAGES * LN_STAGE_BYTES + 256 /* barriers */ + 6 * BM * 4 /* row statistics */ + 1024;

template <int CLUSTER, bool B_MN>
__global__ void __cluster_dims__(CLUSTER, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_f16_ln_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                   const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_r,
                   const LnArgs la) {
    const GemmArgs& args = la.g;
    constexpr uint32_t TMEM_COLS = LN_BN;
    constexpr uint32_t IDESC = ptx::make_idesc_f16(BM, LN_BN, 0, B_MN ? 1 : 0);

    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + LN_STAGES * LN_STAGE_BYTES);
    uint64_t* empty_bar = full_bar + LN_STAGES;
    uint64_t* tmem_full_bar = empty_bar + LN_STAGES;
    uint64_t* res_full_bar = tmem_full_bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(res_full_bar + 1);
    float* red = reinterpret_cast<float*>(smem + LN_STAGES * LN_STAGE_BYTES + 256);  // [4][128]: sum and sum of squares per column half
    float* stats = red + 4 * BM;                                                       // [2][128]: this CTA's row sum and sum of squares

    pdl_launch_dependents();
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();
    const int mt = blockIdx.x / CLUSTER;  // one 128-row block per cluster
    const int m0 = mt * BM;
    const int n0 = static_cast<int>(rank) * LN_BN;
    const int num_kb = (args.k + BK - 1) / BK;
    const bool res_tiles = (args.epilogue & B200ML_EPI_RESIDUAL) && args.residual != nullptr;
    // residual tile t (0..15: epilogue warp t / 2, its 64-column half t % 2) lives in the two stages after the last k-block
    auto res_tile = [&](int t) -> uint8_t* {
        const int sx = num_kb % LN_STAGES, sy = (num_kb + 1) % LN_STAGES;
        return t < 12 ? smem + sx * LN_STAGE_BYTES + t * 4096 : smem + sy * LN_STAGE_BYTES + (t - 12) * 4096;
    };

    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmap_a);
        ptx::prefetch_tensormap(&tmap_b);
        ptx::prefetch_tensormap(&tmap_c);
        if (res_tiles) ptx::prefetch_tensormap(&tmap_r);
    }
    if (warp == 1) {
        if (lane == 0) {
            for (int s = 0; s < LN_STAGES; ++s) {
                ptx::mbar_init(&full_bar[s], 1);
                ptx::mbar_init(&empty_bar[s], 1);
            }
            ptx::mbar_init(tmem_full_bar, 1);
            ptx::mbar_init(res_full_bar, 1);
            ptx::fence_mbar_init();
        }
        __syncwarp();
        ptx::tmem_alloc(tmem_slot, TMEM_COLS);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // A constant B (weights): its parts of the first stages are requested before the dependency wait (see gemm_tc.cu)
    const int early = args.b_early ? (num_kb < LN_STAGES ? num_kb : LN_STAGES) : 0;
    if (warp == 0 && early > 0) {
        if (ptx::elect_one()) {
            for (int kb = 0; kb < early; ++kb) {
                uint8_t* sb = smem + kb * LN_STAGE_BYTES + A_TILE_BYTES;
                ptx::mbar_expect_tx(&full_bar[kb], LN_STAGE_BYTES);
                if (B_MN) {
#pragma unroll
                    for (int j = 0; j < LN_BN / 64; ++j)
                        ptx::tma_load_4d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[kb], n0 + j * 64, kb * BK, 0, 0);
                } else {
                    ptx::tma_load_4d(sb, &tmap_b, &full_bar[kb], kb * BK, n0, 0, 0);
                }
            }
        }
        __syncwarp();
    }
    pdl_wait();

    if (warp == 0) {
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(&empty_bar[stage], phase ^ 1)) {
                    atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                    break;
                }
                uint8_t* sa = smem + stage * LN_STAGE_BYTES;
                uint8_t* sb = sa + A_TILE_BYTES;
                const bool b_done = kb < early;  // requested before the dependency wait
                if (!b_done) ptx::mbar_expect_tx(&full_bar[stage], LN_STAGE_BYTES);
                ptx::tma_load_4d(sa, &tmap_a, &full_bar[stage], kb * BK, m0, 0, 0);
                if (b_done) {
                } else if (B_MN) {
#pragma unroll
                    for (int j = 0; j < LN_BN / 64; ++j)
                        ptx::tma_load_4d(sb + j * (64 * BK * 2), &tmap_b, &full_bar[stage], n0 + j * 64, kb * BK, 0, 0);
                } else {
                    ptx::tma_load_4d(sb, &tmap_b, &full_bar[stage], kb * BK, n0, 0, 0);
                }
                if (++stage == LN_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (res_tiles) {
                // two more turns of the ring: the stages after the last k-block take the residual tiles
                bool ok = true;
                for (int extra = 0; extra < 2 && ok; ++extra) {
                    ok = ptx::mbar_wait(&empty_bar[stage], phase ^ 1);
                    if (++stage == LN_STAGES) {
                        stage = 0;
                        phase ^= 1;
                    }
                }
                if (!ok) {
                    atomicExch(args.status, DEV_TIMEOUT_PRODUCER);
                } else {
                    ptx::mbar_expect_tx(res_full_bar, 16 * 4096);
#pragma unroll 1
                    for (int t = 0; t < 16; ++t) {
                        const int w = t >> 1;  // epilogue warp index: quarter = (w + 2) & 3, column half = w >> 2
                        const int q = (w + 2) & 3, h = w >> 2;
                        ptx::tma_load_4d(res_tile(t), &tmap_r, res_full_bar, n0 + h * 128 + (t & 1) * 64, m0 + q * 32, 0, 0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (ptx::elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int kb = 0; kb < num_kb; ++kb) {
                if (!ptx::mbar_wait(&full_bar[stage], phase)) {
                    atomicExch(args.status, DEV_TIMEOUT_MMA);
                    ok = false;
                    break;
                }
                ptx::tc_fence_after();
                const uint32_t a_addr = ptx::smem_u32(smem + stage * LN_STAGE_BYTES);
                const uint32_t b_addr = a_addr + A_TILE_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                    const uint64_t a_desc = ptx::make_smem_desc_sw128(a_addr + kk * (UMMA_K * 2), 16, 1024);
                    const uint64_t b_desc = B_MN ? ptx::make_smem_desc_sw128(b_addr + kk * (UMMA_K * 128), 64 * BK * 2, 1024)
                                                 : ptx::make_smem_desc_sw128(b_addr + kk * (UMMA_K * 2), 16, 1024);
                    ptx::mma_f16_ss(tmem_base, a_desc, b_desc, IDESC, (kb | kk) != 0 ? 1u : 0u);
                }
                ptx::mma_commit(&empty_bar[stage]);
                if (++stage == LN_STAGES) {
                    stage = 0;
                    phase ^= 1;
                }
            }
            if (ok) ptx::mma_commit(tmem_full_bar);
        }
    }

    ResidualTiles res;
    res.first = smem + (num_kb % LN_STAGES) * LN_STAGE_BYTES;
    res.second = smem + ((num_kb + 1) % LN_STAGES) * LN_STAGE_BYTES;
    res.split = 12;
    res.present = res_tiles;
    // every product has finished by pass B (tmem_full), so the first pipeline stage is free to stage the output
    layernorm_epilogue<CLUSTER, 2>(la, &tmap_c, tmem_base, smem, res, red, stats, tmem_full_bar, res_full_bar, m0, n0, 0, 1, warp, lane);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_acq_rel();  // #2: no CTA leaves while a peer may still read its statistics
    if (warp == 1) {
        ptx::tc_fence_after();
        if (*reinterpret_cast<volatile int32_t*>(args.status) != DEV_OK) {
            for (int i = 0; i < 200; ++i) __nanosleep(1000);
        }
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

template <int CLUSTER, bool B_MN>
int launch_ln(const b200ml_ctx* ctx, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc, const CUtensorMap& tr,
              const LnArgs& la, int tiles_m, cudaStream_t stream) {
    auto kernel = gemm_f16_ln_kernel<CLUSTER, B_MN>;
    static bool configured[64] = {};
    if (!configured[ctx->device & 63]) {
        B200ML_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LN_SMEM));
        configured[ctx->device & 63] = true;
    }
    B200ML_CUDA(launch_pdl(kernel, dim3(tiles_m * CLUSTER), dim3(GEMM_THREADS), LN_SMEM, stream, ta, tb, tc, tr, la));
    return check_launch("gemm_f16_ln");
}

}  // namespace

// Returns B200ML_ERR_UNSUPPORTED (without a launch) for shapes the fused kernel does not cover.
int gemm_f16_layernorm(const b200ml_ctx* ctx, const b200ml_gemm_params* p, cudaStream_t stream) {
    const int64_t batches = p->batch_outer * p->batch_inner;
    const bool shape_ok = batches == 1 && p->a_layout == 0 && p->n % LN_BN == 0 && p->n >= LN_BN && p->n <= 1024 &&
                          (p->n / LN_BN == 1 || p->n / LN_BN == 2 || p->n / LN_BN == 4) && p->m < (1ll << 24);
    bool vec = aligned16(p->a) && p->lda % 8 == 0 && aligned16(p->b) && p->ldb % 8 == 0 && aligned16(p->c) && p->ldc % 8 == 0;
    if (p->residual) vec = vec && aligned16(p->residual) && p->ldr % 8 == 0;
    if (p->bias) vec = vec && aligned16(p->bias);
    if (p->ln_gamma) vec = vec && aligned16(p->ln_gamma);
    if (p->ln_beta) vec = vec && aligned16(p->ln_beta);
    const bool act_ok = (p->epilogue & (B200ML_EPI_GELU | B200ML_EPI_SWISH)) == 0;  // only ReLU is folded in before the norm
    if (!shape_ok || !vec || !act_ok)
        return fail(B200ML_ERR_UNSUPPORTED,
                    "gemm + layernorm: needs fp16, N in {256, 512, 1024}, one batch, 16-byte aligned rows, no GELU / Swish");
    LnArgs la{};
    GemmArgs& args = la.g;
    args.m = (int32_t)p->m;
    args.n = (int32_t)p->n;
    args.k = (int32_t)p->k;
    args.epilogue = p->epilogue;
    args.ldc = p->ldc;
    args.ldr = p->ldr;
    args.alpha = p->alpha;
    args.bias_scale = p->bias_scale;
    args.residual_scale = p->residual_scale;
    args.vec_ok = 1;
    args.c = static_cast<__half*>(p->c);
    args.bias = static_cast<const __half*>(p->bias);
    args.residual = static_cast<const __half*>(p->residual);
    args.status = ctx->status_dev;
    args.b_early = (p->flags & B200ML_GEMM_B_CONSTANT) ? 1 : 0;
    la.gamma = static_cast<const __half*>(p->ln_gamma);
    la.beta = static_cast<const __half*>(p->ln_beta);
    la.eps = p->ln_eps;
    la.cluster = (int32_t)(p->n / LN_BN);
    const int tiles_m = (int)ceil_div(p->m, BM);
    CUtensorMap ta, tb, tc;
    int rc = make_tmap(ctx, &tc, p->c, p->n, p->m, p->ldc, 1, 0, 1, 0, 64, 32, "C");
    if (rc) return rc;
    CUtensorMap tr = tc;
    if ((p->epilogue & B200ML_EPI_RESIDUAL) && p->residual) {
        rc = make_tmap(ctx, &tr, p->residual, p->n, p->m, p->ldr, 1, 0, 1, 0, 64, 32, "residual");
        if (rc) return rc;
    }
    rc = make_tmap(ctx, &ta, p->a, p->k, p->m, p->lda, 1, 0, 1, 0, BK, BM, "A");
    if (rc) return rc;
    if (p->b_layout == 1) {
        rc = make_tmap(ctx, &tb, p->b, p->k, p->n, p->ldb, 1, 0, 1, 0, BK, LN_BN, "B");
        if (rc) return rc;
        switch (la.cluster) {
            case 1: return launch_ln<1, false>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
            case 2: return launch_ln<2, false>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
            default: return launch_ln<4, false>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
        }
    }
    rc = make_tmap(ctx, &tb, p->b, p->n, p->k, p->ldb, 1, 0, 1, 0, 64, BK, "B");
    if (rc) return rc;
    switch (la.cluster) {
        case 1: return launch_ln<1, true>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
        case 2: return launch_ln<2, true>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
        default: return launch_ln<4, true>(ctx, ta, tb, tc, tr, la, tiles_m, stream);
    }
}

}  // namespace b200ml
